"""Dense gated feed-forward (SwiGLU for Qwen3)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward
from .linear import linear
from .registry import register_feed_forward
from .spec import GatedMLPSpec, WeightDecl


class GatedMLP(FeedForward):
    """down( silu(x Wg^T) * (x Wu^T) ).  Gate and up are packed row-wise into one [2F, H]
    matrix at load (values untouched) so that one product yields both, and the activation is
    one pass over the packed result.  The reference runs gate, up, silu and mul as four
    nodes, each rounded to bfloat16 (src/models/qwen3.zig:153-162); here act * up is rounded
    once."""

    @staticmethod
    def weight_decls(spec: GatedMLPSpec):
        return [WeightDecl(spec.gate_proj, (spec.intermediate_size, spec.hidden_size)),
                WeightDecl(spec.up_proj, (spec.intermediate_size, spec.hidden_size)),
                WeightDecl(spec.down_proj, (spec.hidden_size, spec.intermediate_size))]

    @staticmethod
    def kernel_modules(spec):
        return ("elementwise", "gemm_simt", "gemv")

    def __init__(self, spec: GatedMLPSpec, weights, dtype, device):
        if spec.activation != "silu":
            raise ValueError(f"gated feed-forward: activation {spec.activation!r} is not supported")
        self.spec = spec
        self.dtype = dtype
        self.w_gate_up = torch.cat([weights.host_tensor(spec.gate_proj), weights.host_tensor(spec.up_proj)], dim=0) \
            .to(device=device, dtype=dtype).contiguous()
        self.w_down = weights.device_tensor(spec.down_proj, dtype, device)

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        F, H = self.spec.intermediate_size, self.spec.hidden_size
        ws = ctx.workspace
        gate_up = linear(x, self.w_gate_up, ws.buffer("ffn_gate_up", T, 2 * F, self.dtype))
        act = ws.buffer("ffn_act", T, F, self.dtype)
        ops.silu_mul(act, gate_up)
        return linear(act, self.w_down, ws.buffer("ffn_out", T, H, self.dtype))


register_feed_forward("gated_mlp", GatedMLP)
