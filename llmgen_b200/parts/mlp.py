"""Dense gated feed-forward (SwiGLU for Qwen3)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward
from .linear import GEMM_MODULES, gated_product_usable, linear, linear_sliced
from .registry import register_feed_forward
from .spec import GatedMLPSpec, WeightDecl

GATE_UP_GROUP = 16   # rows of gate, then rows of up, alternating: what the gated epilogue expects


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, group: int = GATE_UP_GROUP) -> torch.Tensor:
    """[2F, H]: rows [2 g k, 2 g k + g) are gate rows [g k, g k + g), the next g rows the same up
    rows (values untouched)."""
    F, H = w_gate.shape
    if F % group != 0:
        raise ValueError(f"intermediate size {F} is not a multiple of {group}")
    return torch.stack([w_gate.view(F // group, group, H), w_up.view(F // group, group, H)], dim=1).reshape(2 * F, H)


class GatedMLP(FeedForward):
    """down( silu(x Wg^T) * (x Wu^T) ).  Gate and up are packed into one [2F, H] matrix at load
    (values untouched) so that one product yields both.  In bfloat16 the rows alternate in groups
    of 16 and the tensor-core product applies the activation in its epilogue, so the [T, 2F]
    intermediate is never written; when the few-rows product is cut along K, and in float32, the
    activation is one pass over the packed result (or its partial sums).  The down projection may
    come back as partial sums (`ops.Partials`) that the next norm adds up.  The reference runs gate, up, silu and mul
    as four nodes, each rounded to bfloat16 (src/models/qwen3.zig:153-162); here act * up is
    rounded once."""

    @staticmethod
    def weight_decls(spec: GatedMLPSpec):
        return [WeightDecl(spec.gate_proj, (spec.intermediate_size, spec.hidden_size)),
                WeightDecl(spec.up_proj, (spec.intermediate_size, spec.hidden_size)),
                WeightDecl(spec.down_proj, (spec.hidden_size, spec.intermediate_size))]

    @staticmethod
    def kernel_modules(spec):
        return ("elementwise",) + GEMM_MODULES

    def __init__(self, spec: GatedMLPSpec, weights, dtype, device):
        if spec.activation != "silu":
            raise ValueError(f"gated feed-forward: activation {spec.activation!r} is not supported")
        self.spec = spec
        self.dtype = dtype
        F = spec.intermediate_size
        # packed on the device: each matrix goes up through the loader's pinned stage as the file holds it
        w_gate = weights.device_tensor(spec.gate_proj, dtype, device, keep=False)
        w_up = weights.device_tensor(spec.up_proj, dtype, device, keep=False)
        if dtype == torch.bfloat16 and F % GATE_UP_GROUP == 0:
            self.group = GATE_UP_GROUP
            packed = interleave_gate_up(w_gate, w_up)
        else:
            self.group = F
            packed = torch.cat([w_gate, w_up], dim=0)
        self.w_gate_up = packed.contiguous()
        self.w_down = weights.device_tensor(spec.down_proj, dtype, device)

    def workspace_bytes(self, tokens: int) -> int:
        """Bytes of activations this part keeps in the step's workspace for `tokens` rows: the packed gate/up
        product, the activation and the output, and the float32 slices of two products cut along K."""
        F, H = self.spec.intermediate_size, self.spec.hidden_size
        elem = 2 if self.dtype == torch.bfloat16 else 4
        return tokens * (2 * F + F + H) * elem + 2 * ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x):
        T = x.shape[0]
        F, H = self.spec.intermediate_size, self.spec.hidden_size
        ws = ctx.workspace
        act = ws.buffer("ffn_act", T, F, self.dtype)
        gated = self.group == GATE_UP_GROUP and F % GATE_UP_GROUP == 0 and gated_product_usable(x, self.w_gate_up)
        cluster = min(ops.gemm_skinny_cluster_splits(T, 2 * F, H), 4) if gated and T <= ops.SKINNY_CLUSTER_MAX_ROWS else 1
        if gated and T <= ops.ROWS8_GATED_BEST_ROWS and ops.gemm_rows8_gated_usable(x, self.w_gate_up):
            # a few rows: W straight from global memory into mma.sync, the activation in the same kernel (csrc/gemm_rows8.cu)
            ops.gemm_rows8_gated(act, x, self.w_gate_up)
        elif cluster >= 2:
            # few rows: K is cut, the slices are added up inside a thread-block cluster and the activation
            # follows there, so neither the packed product nor a kernel for the activation is needed
            # (0.982 -> 0.967 ms a decode step at batch 8 against slices and an activation kernel)
            ops.gemm_skinny(act, x, self.w_gate_up, ops.SKINNY_CLUSTER_GATED, splits=cluster)
        elif gated and T <= ops.SKINNY_BEST_ROWS and ops.gemm_skinny_splits(T, 2 * F, H) == 1:
            ops.gemm_skinny(act, x, self.w_gate_up, ops.SKINNY_GATED)
        elif gated and T > ops.SKINNY_BEST_ROWS:
            ops.gemm_tc(act, x, self.w_gate_up, gated=True)
        else:
            gate_up = linear_sliced(ws, "ffn_gate_up", x, self.w_gate_up, self.dtype)
            ops.silu_mul(act, gate_up, group=self.group)
        return linear_sliced(ws, "ffn_out", act, self.w_down, self.dtype)


register_feed_forward("gated_mlp", GatedMLP)
