"""The arrangement of a layer's parts."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from . import linear as linear_module
from .base import LayerCache, Part
from .registry import (build_feed_forward, build_mixer, build_norm, feed_forward_class, mixer_class, norm_class,
                       register_block)
from .spec import PreNormBlockSpec


class PreNormBlock(Part):
    """x1 = x + mixer(norm(x)); x2 = x1 + ffn(norm(x1))  (src/models/qwen3.zig:224-236).

    The residual stream is float32 and lives in one buffer.  Each sum is folded into the norm
    that follows it: the block receives the previous block's output as `delta`, adds it in its
    first norm, adds the mixer's output in its second norm and returns the feed-forward's
    output as the next `delta`.  Parts that declare `fuses_neighbours` are offered the residual
    (`add_to`) and may add their output themselves; they then return `ops.RowSquares`, which says so
    and carries what the next norm needs, and that norm is handed to its consumer uncomputed."""

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

    def _normed(self, ctx, norm, consumer, resid, delta):
        """(the consumer's input norm(resid + delta), the array that holds the residual afterwards).

        When `delta` is an `ops.RowSquares` the sum is already in `resid`; a norm that can defer itself
        and a consumer that takes deferred operands then get an `ops.NormedRows` and no kernel runs here.
        When `delta` is the slices of a product (`ops.Partials`) and there are few rows, such a consumer
        gets an `ops.AddNormRows`: its product adds the slices, normalises and leaves the new residual in
        the other of the residual's two arrays."""
        fuses = getattr(consumer, "fuses_neighbours", False)
        if isinstance(delta, ops.RowSquares):
            if hasattr(norm, "deferred") and fuses:
                return norm.deferred(resid, delta), resid
            delta = None
        T, H = resid.shape
        if (isinstance(delta, ops.Partials) and fuses and hasattr(norm, "deferred_add") and linear_module.ADDNORM
                and self.dtype == torch.bfloat16 and T <= ops.ADDNORM_MAX_ROWS and resid.is_contiguous()):
            first = ctx.workspace.buffer("residual", T, H, torch.float32)
            other = ctx.workspace.buffer("residual_other", T, H, torch.float32) if resid.data_ptr() == first.data_ptr() else first
            return norm.deferred_add(resid, delta, other), other
        return norm.add_norm(resid, delta, ctx.workspace.buffer("block_normed", T, H, self.dtype)), resid

    def forward(self, ctx, resid: torch.Tensor, delta, cache: LayerCache):
        given = resid
        x, resid = self._normed(ctx, self.mixer_norm, self.mixer, resid, delta)
        if getattr(self.mixer, "fuses_neighbours", False):
            mixed = self.mixer.forward(ctx, x, cache, add_to=resid)
        else:
            mixed = self.mixer.forward(ctx, x, cache)
        x, resid = self._normed(ctx, self.ffn_norm, self.ffn, resid, mixed)
        if getattr(self.ffn, "fuses_neighbours", False):
            out = self.ffn.forward(ctx, x, add_to=resid)
        else:
            out = self.ffn.forward(ctx, x)
        return out if resid is given else ops.Moved(resid, out)


register_block("prenorm", PreNormBlock)
