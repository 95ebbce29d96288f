"""Causal grouped-query attention over the paged cache, as a mixer."""
from __future__ import annotations

import torch

from ..cache.manager import FULL, WINDOW
from ..kernels import ops
from .base import KVRequest, LayerCache, Mixer
from .linear import GEMM_MODULES, linear, linear_sliced
from .registry import build_position, norm_class, register_mixer
from .spec import INIT_ONE_PLUS_NORMAL, VECTOR, AttentionSpec, WeightDecl


class GQAAttention(Mixer):
    """q, k, v projections (packed into one [(nq + 2 nkv) hd, H] matrix at load) -> per-head
    RMSNorm of q and k, rotary encoding, cache write (one kernel) -> attention over the block
    table -> output projection.

    Attention kernels: in bfloat16 a step of single decoded tokens runs the bandwidth-shaped
    flash-decoding kernel (csrc/attention_decode.cu), any other step the tensor-core kernel
    (csrc/attention_tc.cu); float32, and sizes those two refuse, run the general CUDA-core kernel
    (csrc/attention.cu).

    Order and formulas: src/models/qwen3.zig:192-207 (q/k norm before RoPE, norm weights
    shared by all heads), src/module/attention.zig:85-92, src/backend/cpu/attention.zig:64-118.
    A run item with `writes=False` projects q only and reads the cache another item wrote."""

    # what `prepare_step` adds depends on the lengths of the step's portions only, not on their
    # positions or requests: the engine may keep it across decode steps of one batch size
    step_arrays_follow_shapes = True
    # its launches follow from a step's shape (token rows, sequences) alone, its lists of tiles have the length
    # that the shape bounds, and token rows that belong to no sequence pass through untouched: any step may be
    # replayed from the graph of its shape
    replay_any_step = True

    @staticmethod
    def weight_decls(spec: AttentionSpec):
        qd, kd = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        decls = [WeightDecl(spec.q_proj, (qd, spec.hidden_size)), WeightDecl(spec.k_proj, (kd, spec.hidden_size)),
                 WeightDecl(spec.v_proj, (kd, spec.hidden_size)), WeightDecl(spec.o_proj, (spec.hidden_size, qd))]
        for n in (spec.q_norm, spec.k_norm):
            if n is not None:
                decls += norm_class(n).weight_decls(n)
        return decls

    @staticmethod
    def kernel_modules(spec):
        return ("attn_prep", "attention", "attention_decode", "attention_tc") + GEMM_MODULES

    def __init__(self, spec: AttentionSpec, weights, dtype, device):
        if spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError(f"attention: {spec.num_heads} heads are not a multiple of {spec.num_kv_heads} kv heads")
        if spec.head_dim % 8 != 0 or spec.head_dim > 512:
            raise ValueError(f"attention: head_dim {spec.head_dim} must be a multiple of 8, at most 512")
        for n in (spec.q_norm, spec.k_norm):
            if n is not None and (n.kind not in ops.HEAD_NORMS or n.dim != spec.head_dim):
                raise ValueError(f"attention: per-head norms must run over head_dim and be one of {sorted(ops.HEAD_NORMS)}")
        self.spec = spec
        self.dtype = dtype
        self.nq, self.nkv, self.hd = spec.num_heads, spec.num_kv_heads, spec.head_dim
        # packed on the device: each matrix goes up through the loader's pinned stage as the file holds it
        self.w_qkv = torch.cat([weights.device_tensor(n, dtype, device, keep=False) for n in (spec.q_proj, spec.k_proj, spec.v_proj)],
                               dim=0).contiguous()
        self.w_q = self.w_qkv[: self.nq * self.hd]
        self.w_o = weights.device_tensor(spec.o_proj, dtype, device)
        self.q_gain = weights.device_tensor(spec.q_norm.weight, dtype, device) if spec.q_norm else None
        self.k_gain = weights.device_tensor(spec.k_norm.weight, dtype, device) if spec.k_norm else None
        self.norm_eps = float((spec.q_norm or spec.k_norm).eps) if (spec.q_norm or spec.k_norm) else 0.0
        if spec.q_norm and spec.k_norm and spec.q_norm.eps != spec.k_norm.eps:
            raise ValueError("attention: q and k norms must share eps")
        self.q_off = float(spec.q_norm.weight_offset) if spec.q_norm else 0.0
        self.k_off = float(spec.k_norm.weight_offset) if spec.k_norm else 0.0
        self.position = build_position(spec.position, weights, dtype, device) if spec.position is not None else None
        # which values of a head the position encoding turns together, and the kind of the per-head norms: the
        # kernels are told and refuse what they do not implement
        self.pairing = getattr(self.position, "pairing", "half") if self.position is not None else "half"
        self.head_norm = (spec.q_norm or spec.k_norm).kind if (spec.q_norm or spec.k_norm) else "rmsnorm"
        self.sm_count = ops.sm_count(device)
        self.window = int(spec.window or 0)
        self.bq = ops.attention_tile_queries(self.nq, self.nkv)
        self.tiles_name = f"attention_tiles_bq{self.bq}"
        self._tc_bq = {}       # page size -> queries per tile of the tensor-core kernel (0: not taken)

    # -- what the engine asks
    def cache_request(self) -> KVRequest:
        return KVRequest(WINDOW if self.window else FULL, self.window, self.nkv, self.hd)

    def max_positions(self):
        return self.position.max_positions if self.position is not None else None

    def _tiles(self, builder, bq: int, heaviest_first: bool = False) -> None:
        """(sequence, first query) of every tile of `bq` queries.  `heaviest_first`: in the order of
        the keys a tile has to read, most first; the blocks of a launch start in the order of the
        list, and a prompt's last tiles read the whole prompt while its first read one tile of keys."""
        name = f"attention_tiles_bq{bq}"
        if builder.has(name + "_seq"):
            return
        tiles = []
        bound = getattr(builder, "token_bound", 0)
        for s, n in enumerate(builder.q_lens):
            if bound and n == 0:
                continue
            for start in range(0, max(n, 1), bq):
                keys = builder.starts[s] + min(start + bq, max(n, 1))
                tiles.append((min(keys, self.window + bq) if self.window else keys, s, start))
        if heaviest_first:
            tiles.sort(key=lambda t: -t[0])
        if bound:
            # a list of fixed length for the step's shape: no more tiles than this exist for `bound` tokens in
            # `n_seqs` sequences; the rest is padding (sequence -1), which the kernels skip
            most = bound // bq + builder.n_seqs
            tiles += [(0, -1, 0)] * (most - len(tiles))
        builder.add(name + "_seq", [t[1] for t in tiles])
        builder.add(name + "_q0", [t[2] for t in tiles])

    def tc_tile_queries(self, page_size: int) -> int:
        if self.dtype != torch.bfloat16:
            return 0
        if page_size not in self._tc_bq:
            self._tc_bq[page_size] = ops.attention_tc_tile_queries(self.nq, self.nkv, self.hd, page_size)
        return self._tc_bq[page_size]

    def step_arrays_key(self):
        """Mixers with equal keys add the same arrays in `prepare_step`: the engine asks one of them."""
        return ("attention_tiles", self.bq, self.nq, self.nkv, self.hd, self.window, str(self.dtype))

    def prepare_step(self, builder) -> None:
        """Tiles of queries, (sequence, first query of the tile) pairs, for the kernel this step will
        run: the tensor-core kernel's where it takes the step, else the CUDA-core kernel's."""
        page_size = getattr(builder, "page_size", 0)
        tc_bq = self.tc_tile_queries(page_size) if page_size and not builder.pure_decode else 0
        if tc_bq:
            self._tiles(builder, tc_bq, heaviest_first=True)
        else:
            self._tiles(builder, self.bq)

    def _split(self, ctx):
        """(num_parts, part_size) for flash-decoding; only pure-decode steps are split."""
        if not ctx.pure_decode:
            return 1, 0
        G = self.nq // self.nkv
        chunks = (G + 15) // 16
        blocks = max(1, ctx.n_seqs * self.nkv * chunks)
        longest = ctx.max_ctx_bound if ctx.fixed_shapes else ctx.max_ctx
        if self.window:
            longest = min(longest, self.window)
        by_sms = (2 * self.sm_count + blocks - 1) // blocks
        by_len = max(1, longest // 128)
        parts = max(1, min(by_sms, by_len, 64))
        if self.window:
            # parts are ranges of absolute key positions: a window far into a long context
            # would leave most of an even split empty, so windowed layers are not split
            return 1, 0
        return parts, 0

    def workspace_bytes(self, tokens: int) -> int:
        """Bytes of activations this part keeps in the step's workspace for `tokens` rows: the packed projection
        (and the float32 slices of two products cut along K), q, the attention's output and the output projection."""
        elem = 2 if self.dtype == torch.bfloat16 else 4
        packed = (self.nq + 2 * self.nkv) * self.hd
        return tokens * (packed + 2 * self.nq * self.hd + self.spec.hidden_size) * elem + 2 * ops.SLICED_PRODUCT_BYTES

    def forward(self, ctx, x, cache: LayerCache):
        T = ctx.n_tokens
        ws = ctx.workspace
        group = ctx.groups[cache.group]
        nk = self.nkv if cache.writes else 0
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        rot = self.position.rotary_dim if self.position is not None else 0
        decode = (self.dtype == torch.bfloat16 and ctx.pure_decode
                  and ops.attention_decode_usable(self.nq, self.nkv, self.hd, cache.page_size))
        fused = decode and ops.attention_decode_fuses_prep(self.hd, rot)
        w = self.w_qkv if cache.writes else self.w_q
        name = "attn_qkv" if cache.writes else "attn_q_only"
        if fused or T <= ops.SKINNY_BEST_ROWS or self.dtype != torch.bfloat16:
            packed = linear_sliced(ws, name, x, w, self.dtype)
        else:
            # the preparation kernel's fast path wants finished rows: with hundreds of them a product cut along K
            # would save less than adding its slices up there costs
            packed = linear(x, w, ws.buffer(name, T, w.shape[0], self.dtype))
        o = ws.buffer("attn_o", T, self.nq * self.hd, self.dtype)
        scale = float(self.spec.scale)
        if fused:
            # single decoded tokens: the attention kernel normalises, rotates and stores q, k and v itself
            self._decode(ctx, o, None, cache, group, scale,
                         prep=dict(packed=packed, nk=nk, rot=rot, positions=ctx.positions, slots=group.slots, cos=cos,
                                   sin=sin, q_gain=self.q_gain, k_gain=self.k_gain, eps=self.norm_eps,
                                   q_offset=self.q_off, k_offset=self.k_off, pairing=self.pairing,
                                   head_norm=self.head_norm))
            return linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)
        q = ws.buffer("attn_q", T, self.nq * self.hd, self.dtype) if isinstance(packed, ops.Partials) else packed
        ops.attn_prep(packed, cache.k, cache.v, ctx.positions, group.slots, cos, sin, self.q_gain, self.k_gain,
                      self.nq, nk, self.hd, rot, cache.page_size, self.norm_eps, self.q_off, self.k_off, q_out=q,
                      pairing=self.pairing, head_norm=self.head_norm)
        packed = q
        if decode:
            self._decode(ctx, o, packed, cache, group, scale)
            return linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)
        tc_bq = 0 if ctx.pure_decode else self.tc_tile_queries(cache.page_size)
        if tc_bq and ctx.has_array(f"attention_tiles_bq{tc_bq}_seq"):
            tile_seq = ctx.array(f"attention_tiles_bq{tc_bq}_seq")
            tile_q0 = ctx.array(f"attention_tiles_bq{tc_bq}_q0")
            ops.attention_tc(o, packed, packed.stride(0), cache.k, cache.v, group.block_tables, group.max_blocks,
                             ctx.ctx_len, ctx.cu_q, tile_seq, tile_q0, tile_seq.numel(), T, self.nq, self.nkv,
                             self.hd, cache.page_size, self.window, scale)
            return linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)
        tile_seq = ctx.array(self.tiles_name + "_seq")
        tile_q0 = ctx.array(self.tiles_name + "_q0")
        parts, part_size = self._split(ctx)
        scratch = None
        if parts > 1:
            scratch = ws.flat("attn_split", ops.attention_scratch_floats(T, self.nq, self.hd, parts), torch.float32)
        ops.paged_attention(o, packed, packed.stride(0), cache.k, cache.v, group.block_tables, group.max_blocks,
                            ctx.ctx_len, ctx.cu_q, tile_seq, tile_q0, tile_seq.numel(), T, self.nq, self.nkv,
                            self.hd, cache.page_size, self.window, float(self.spec.scale), parts, part_size, scratch)
        return linear_sliced(ws, "mixer_out", o, self.w_o, self.dtype)

    def _decode(self, ctx, o, q, cache, group, scale, prep=None) -> None:
        """Single decoded tokens: as many key parts as fill the SMs, at least 128 keys a part; the
        bound of the step's context class decides, not the lengths."""
        ws = ctx.workspace
        S = ctx.n_seqs
        G = self.nq // self.nkv
        chunks = (G + 7) // 8
        # the bound of the step's context class, for eager steps too: a step then cuts its keys the
        # same way whether it is replayed from a graph or launched directly, and gives the same bits
        bound = max(ctx.max_ctx_bound, ctx.max_ctx, 1)
        visible = min(bound, self.window) if self.window else bound
        blocks = max(1, S * self.nkv * chunks)
        # Key parts: at least 128 keys each, at most 64.  A block an SM where that still cuts every sequence's keys
        # into 4 parts or more (up to 4 sequences on 8 kv heads): two blocks an SM (the most that are resident) leave
        # the kernels after this one no room to start, and to ask for their weights, under it (a step of 4 sequences
        # of 640 keys: 0.898 ms with 8 parts, 0.798 with 4; of 1,500 keys: 0.994 with 9, 0.888 with 4).  Two blocks
        # an SM otherwise: with 8 sequences 2 parts are too few (0.935 against 0.907 ms with 4; at 1,500 keys 1.095
        # against 1.022).
        one_each = self.sm_count // blocks
        target = one_each if one_each >= 4 else (2 * self.sm_count) // blocks
        parts = max(1, min(target, visible // 128, 64))
        scratch = counters = None
        if parts > 1:
            scratch = ws.flat("attn_decode_split", ops.attention_decode_scratch_floats(S, self.nq, self.hd, parts),
                              torch.float32)
            counters = ws.flat("attn_decode_counters", ops.attention_decode_counters(max(ctx.max_seqs_bound, S), self.nq, self.nkv),
                               torch.int32, zero=True)
        ops.attention_decode(o, q, q.stride(0) if q is not None else 0, cache.k, cache.v, group.block_tables,
                             group.max_blocks, ctx.ctx_len, ctx.cu_q, S, self.nq, self.nkv, self.hd, cache.page_size,
                             self.window, scale, parts, bound, scratch, counters, **(prep or {}))


register_mixer("attention", GQAAttention)
