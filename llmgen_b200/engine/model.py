"""A decoder assembled from a `ModelSpec`: embedding, blocks in run order, final norm on the
wanted rows, output projection.

The forward pass is a plain sequence of kernel launches on the current stream (no DAG, no
placement: one model on one GPU needs neither; the reference builds a graph and a liveness plan
for the same fixed node list, src/graph/scheduler.zig:313-317).  Only the rows whose logits
are wanted reach the final norm and the output projection; the reference norms all rows, then
gathers (src/models/qwen3.zig:321-330), which gives the same values since the norm is
row-wise.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import build as kernel_build
from ..kernels import ops
from ..parts.base import LayerCache
from ..parts.linear import linear
from ..parts.registry import build_block, build_norm, model_kernel_modules
from ..parts.spec import ModelSpec
from .context import StepContext


class DecoderModel:
    def __init__(self, spec: ModelSpec, weights, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine computes in float32 or bfloat16, not {dtype}")
        # the kernels this model's parts need, and the host runtime (cache manager, scheduler) beside them
        kernel_build.ensure_built(list(model_kernel_modules(spec)) + ["runtime"])
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.embedding = weights.device_tensor(spec.embedding, dtype, device)
        self.layers = [build_block(ls, weights, dtype, device) for ls in spec.layers]
        self.final_norm = build_norm(spec.final_norm, weights, dtype, device)
        self.lm_head = weights.device_tensor(spec.lm_head, dtype, device)   # the embedding itself when tied
        weights.release()
        for item in spec.run_order:
            if not 0 <= item.layer < len(self.layers):
                raise ValueError(f"run list names layer {item.layer}, the model has {len(self.layers)}")
        self.bad_token_flag = ops.bad_token_flag(device)      # read by the engine with every step's results

    # -- what the engine needs to size caches and limits
    def mixers(self):
        return [getattr(layer, "mixer", None) for layer in self.layers]

    def max_positions(self) -> int:
        limit = self.spec.max_positions
        for m in self.mixers():
            mp = m.max_positions() if m is not None and hasattr(m, "max_positions") else None
            if mp is not None:
                limit = min(limit, mp)
        return limit

    def weight_bytes(self) -> int:
        """Bytes of device memory held by the model's tensors (shared storage counted once)."""
        storages: Dict[int, int] = {}
        seen = set()

        def collect(obj):
            if isinstance(obj, torch.Tensor):
                if obj.is_cuda:
                    st = obj.untyped_storage()
                    storages[st.data_ptr()] = st.nbytes()
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    collect(v)
            elif hasattr(obj, "__dict__") and id(obj) not in seen:
                seen.add(id(obj))
                for v in vars(obj).values():
                    collect(v)

        collect(self)
        return sum(storages.values())

    # -- one pass
    def hidden_states(self, ctx: StepContext, caches: List[LayerCache]):
        """Run embedding and all run items; returns (residual float32 [T, H], pending delta)."""
        T, H = ctx.n_tokens, self.spec.hidden_size
        resid = ctx.workspace.buffer("residual", T, H, torch.float32)
        ops.embed_rows(resid, self.embedding, ctx.ids, self.bad_token_flag, ids_from=ctx.ids_from, sampled=ctx.prev_sampled,
                       scale=float(self.spec.embedding_scale))
        delta = None
        for item, cache in zip(self.spec.run_order, caches):
            delta = self.layers[item.layer].forward(ctx, resid, delta, cache)
        return resid, delta

    def logits(self, ctx: StepContext, resid: torch.Tensor, delta: Optional[torch.Tensor],
               rows: torch.Tensor, n_rows: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """float32 logits [n_rows, vocab] of the token rows listed in `rows` (int32, device)."""
        H, V = self.spec.hidden_size, self.spec.vocab_size
        ws = ctx.workspace
        normed = ws.buffer("final_normed", n_rows, H, self.dtype, capacity_rows=max(n_rows, 64))
        self.final_norm.add_norm(resid, delta, normed, rows=rows)
        if out is None:
            out = torch.empty((n_rows, V), dtype=torch.float32, device=self.device)
        out = linear(normed, self.lm_head, out)
        if self.spec.logit_cap > 0:
            ops.logit_cap(out, float(self.spec.logit_cap))
        return out

    def forward(self, ctx: StepContext, caches: List[LayerCache], rows: torch.Tensor, n_rows: int,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        resid, delta = self.hidden_states(ctx, caches)
        return self.logits(ctx, resid, delta, rows, n_rows, out)
