"""Dense gated feed-forward (SwiGLU for Qwen3)."""
from __future__ import annotations

import os

import torch

from ..kernels import ops
from .base import FeedForward
from . import linear as linear_module
from .linear import GEMM_MODULES, gated_product_usable, linear, linear_sliced
from .registry import register_feed_forward
from .spec import GatedMLPSpec, WeightDecl


CLUSTER_GATED = os.environ.get("LLMGEN_GATED", "") != "separate"    # "separate": slices, then a kernel for the activation
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
        w_gate, w_up = weights.host_tensor(spec.gate_proj), weights.host_tensor(spec.up_proj)
        if dtype == torch.bfloat16 and F % GATE_UP_GROUP == 0:
            self.group = GATE_UP_GROUP
            packed = interleave_gate_up(w_gate, w_up)
        else:
            self.group = F
            packed = torch.cat([w_gate, w_up], dim=0)
        self.w_gate_up = packed.to(device=device, dtype=dtype).contiguous()
        self.w_down = weights.device_tensor(spec.down_proj, dtype, device)

    fuses_neighbours = True      # takes operands that are not computed yet, adds to the residual when offered it

    def forward(self, ctx, x, add_to: torch.Tensor = None):
        T = x.shape[0]
        F, H = self.spec.intermediate_size, self.spec.hidden_size
        ws = ctx.workspace
        if isinstance(x, ops.AddNormRows):
            # the residual add and the norm before, the sum of the slices and the activation after: one product
            splits = 0
            if self.group == GATE_UP_GROUP and CLUSTER_GATED and linear_module._FORCE == "" and linear_module._SPLITK == "":
                splits = ops.gemm_skinny_addnorm_splits(x, self.w_gate_up, True)
            if splits >= 2:
                act = ws.buffer("ffn_act", T, F, self.dtype)
                ops.gemm_skinny_addnorm(act, x, self.w_gate_up, splits, gated=True)
                return linear_sliced(ws, "ffn_out", act, self.w_down, self.dtype, add_to=add_to)
            x = x.materialize(ws.buffer("ffn_x", T, H, self.dtype))
        few = self.dtype == torch.bfloat16 and T <= linear_module.FUSE_CHAIN_MAX_ROWS and linear_module.FUSE_CHAIN
        if not isinstance(x, torch.Tensor) and not few:
            x = x.materialize(ws.buffer("ffn_x", T, H, self.dtype))
        lazy = not isinstance(x, torch.Tensor)
        whole = (not lazy and self.group == GATE_UP_GROUP and gated_product_usable(x, self.w_gate_up)
                 and ops.gemm_skinny_splits(T, 2 * F, H) == 1)          # one block column streams all of K: gated epilogue
        if few and (lazy or add_to is not None) and not whole:
            # few rows: the norm before, the activation between and the residual sum after are
            # folded into the two products where the few-rows kernel can take them
            gate_up = linear_sliced(ws, "ffn_gate_up", x, self.w_gate_up, self.dtype)
            if isinstance(gate_up, ops.Partials) and self.group % 8 == 0:
                return linear_sliced(ws, "ffn_out", ops.GatedRows(gate_up, self.group), self.w_down, self.dtype, add_to=add_to)
            act = ws.buffer("ffn_act", T, F, self.dtype)
            ops.silu_mul(act, gate_up, group=self.group)
            return linear_sliced(ws, "ffn_out", act, self.w_down, self.dtype, add_to=add_to)
        act = ws.buffer("ffn_act", T, F, self.dtype)
        gated = self.group == GATE_UP_GROUP and F % GATE_UP_GROUP == 0 and gated_product_usable(x, self.w_gate_up)
        if gated and CLUSTER_GATED and T <= ops.SKINNY_CLUSTER_MAX_ROWS and linear_module._SPLITK == "" \
                and min(ops.gemm_skinny_cluster_splits(T, 2 * F, H), 4) >= 2:
            # few rows: K is cut, the slices are added up inside a thread-block cluster and the activation
            # follows there, so neither the packed product nor a kernel for the activation is needed
            ops.gemm_skinny(act, x, self.w_gate_up, ops.SKINNY_CLUSTER_GATED,
                            splits=min(ops.gemm_skinny_cluster_splits(T, 2 * F, H), 4))
        elif gated and T <= ops.SKINNY_MAX_ROWS and ops.gemm_skinny_splits(T, 2 * F, H) == 1:
            ops.gemm_skinny(act, x, self.w_gate_up, ops.SKINNY_GATED)
        elif gated and T > ops.SKINNY_MAX_ROWS:
            ops.gemm_tc(act, x, self.w_gate_up, gated=True)
        else:
            gate_up = linear_sliced(ws, "ffn_gate_up", x, self.w_gate_up, self.dtype)
            ops.silu_mul(act, gate_up, group=self.group)
        return linear_sliced(ws, "ffn_out", act, self.w_down, self.dtype, add_to=add_to)


register_feed_forward("gated_mlp", GatedMLP)
