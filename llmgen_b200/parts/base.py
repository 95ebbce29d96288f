"""What each kind of part must offer.  These classes are documentation with defaults; a part
need not inherit from them as long as it has the same methods.

All parts:
    weight_decls(spec) -> [WeightDecl]        static; tensors read from the model file
    kernel_modules(spec) -> (str, ...)        static; CUDA modules to build before first use
    __init__(spec, weights, dtype, device)    take tensors from the `WeightStore`

Norm:
    add_norm(resid, delta, out, rows=None)    resid(float32) += delta; out = norm(resid);
                                              with `rows`: output row r from source row rows[r],
                                              resid untouched.  `delta` is None, an array [T, H]
                                              of the compute dtype, or a `kernels.ops.Partials`
                                              (float32 slices to be added up), whichever the
                                              part before it returned
Position encoding:
    tables()                                  whatever its mixer's kernel needs (cos, sin)
Mixer:
    cache_request() -> KVRequest | None       pages it needs (group kind, kv heads, head width)
    state_request() -> StateRequest | None    fixed-size per-request state (shape, dtype)
    prepare_step(builder)                     optional: add int32 arrays to the step's metadata
    step_arrays_follow_shapes = True          optional class attribute: those arrays depend on the
                                              portions' lengths only (lets decode steps reuse them)
    replay_any_step = True                    optional class attribute: steps of every kind may be replayed from
                                              a graph captured for their shape.  The mixer then promises that
                                              `forward` launches the same kernels with the same arguments for
                                              every step of one (token rows, sequences) pair: it reads lengths,
                                              positions and tables from the step's device arrays only; arrays it
                                              adds in `prepare_step` have sizes that follow from
                                              `builder.token_bound` and `builder.n_seqs` (padded if need be);
                                              token rows beyond the sequences' own (slot -1, in no sequence) and
                                              sequences of length 0 are harmless to it.  Without it such steps
                                              are launched kernel by kernel
    step_arrays_key()                         optional: mixers with equal keys add the same arrays,
                                              and only one of them is asked each step
    forward(ctx, x, cache) -> [T, H]          x is the normed input; `cache` is this run
                                              item's `LayerCache`; returns an array or a
                                              `Partials` (see `parts.linear.linear_sliced`)
Feed-forward:
    forward(ctx, x) -> [T, H]                 an array or a `Partials`
Any part, optional:
    capturable = False                        class attribute of a part whose `forward` (or `add_norm`) cannot be
                                              recorded into a CUDA graph: it reads a result back on the host, or
                                              what it launches depends on the data.  A model with such a part
                                              runs every step kernel by kernel
Mixer, feed-forward and block, optional:
    workspace_bytes(tokens) -> int            bytes of activations a step of `tokens` rows keeps in
                                              the workspace for this part; the engine leaves that
                                              much device memory beside the cache pages
Block:
    mixer                                     the block's mixer (the engine asks it for cache)
    forward(ctx, resid, delta, cache) -> delta_out
                                              `delta` is the previous block's output not yet
                                              added to the residual (None for the first block);
                                              the block adds it inside its first norm
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class KVRequest:
    """Paged keys and values: which group's pages, and the geometry of one token's entry."""
    group_kind: str          # cache.manager.FULL or WINDOW
    window: int              # 0 for FULL
    num_kv_heads: int
    head_dim: int
    v_head_dim: int = 0      # width of a value where it differs from a key's (0: the same)

    @property
    def value_dim(self) -> int:
        return self.v_head_dim or self.head_dim


@dataclass(frozen=True)
class StateRequest:
    """One array of `shape` and `dtype` per request, zero when the request starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """What a run item hands to its mixer."""
    k: Optional[torch.Tensor] = None        # [pages, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor] = None        # the same with the values' width (KVRequest.v_head_dim)
    group: int = 0                          # index into ctx.groups
    page_size: int = 0
    writes: bool = True                     # False: read what another run item wrote
    state: Optional[torch.Tensor] = None    # [slots, *shape]


class Part:
    @staticmethod
    def weight_decls(spec):
        return []

    @staticmethod
    def kernel_modules(spec):
        return ()


class Mixer(Part):
    def cache_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def prepare_step(self, builder) -> None:
        pass

    def forward(self, ctx, x, cache: LayerCache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x):
        raise NotImplementedError
