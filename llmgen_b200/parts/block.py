"""The arrangement of a layer's parts."""
from __future__ import annotations

import torch

from .base import LayerCache, Part
from .registry import (build_feed_forward, build_mixer, build_norm, feed_forward_class, mixer_class, norm_class,
                       register_block)
from .spec import PreNormBlockSpec


class PreNormBlock(Part):
    """x1 = x + mixer(norm(x)); x2 = x1 + ffn(norm(x1))  (src/models/qwen3.zig:224-236).

    The residual stream is float32 and lives in one buffer.  Each sum is folded into the norm
    that follows it: the block receives the previous block's output as `delta`, adds it in its
    first norm, adds the mixer's output in its second norm and returns the feed-forward's
    output as the next `delta` (an array or the float32 slices of a product cut along K, which the
    norm adds up: `kernels.ops.Partials`)."""

    @staticmethod
    def weight_decls(spec: PreNormBlockSpec):
        return (norm_class(spec.mixer_norm).weight_decls(spec.mixer_norm)
                + mixer_class(spec.mixer).weight_decls(spec.mixer)
                + norm_class(spec.ffn_norm).weight_decls(spec.ffn_norm)
                + feed_forward_class(spec.ffn).weight_decls(spec.ffn))

    @staticmethod
    def kernel_modules(spec: PreNormBlockSpec):
        return (tuple(norm_class(spec.mixer_norm).kernel_modules(spec.mixer_norm))
                + tuple(mixer_class(spec.mixer).kernel_modules(spec.mixer))
                + tuple(feed_forward_class(spec.ffn).kernel_modules(spec.ffn)))

    def __init__(self, spec: PreNormBlockSpec, weights, dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = build_norm(spec.mixer_norm, weights, dtype, device)
        self.mixer = build_mixer(spec.mixer, weights, dtype, device)
        self.ffn_norm = build_norm(spec.ffn_norm, weights, dtype, device)
        self.ffn = build_feed_forward(spec.ffn, weights, dtype, device)

    def workspace_bytes(self, tokens: int) -> int:
        """Bytes of activations a step of `tokens` rows keeps in the workspace for this layer: the normed
        input plus what the mixer and the feed-forward say they need (a part without `workspace_bytes`
        counts as nothing and must allocate before any graph is captured, like every part)."""
        elem = 2 if self.dtype == torch.bfloat16 else 4
        own = tokens * self.spec.mixer_norm.dim * elem
        parts = [getattr(p, "workspace_bytes", None) for p in (self.mixer, self.ffn)]
        return own + max([f(tokens) for f in parts if f is not None] or [0])

    def forward(self, ctx, resid: torch.Tensor, delta, cache: LayerCache):
        T, H = resid.shape
        x = self.mixer_norm.add_norm(resid, delta, ctx.workspace.buffer("block_normed", T, H, self.dtype))
        mixed = self.mixer.forward(ctx, x, cache)
        x = self.ffn_norm.add_norm(resid, mixed, ctx.workspace.buffer("block_normed", T, H, self.dtype))
        return self.ffn.forward(ctx, x)


register_block("prenorm", PreNormBlock)
