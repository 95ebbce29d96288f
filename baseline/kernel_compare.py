"""This engine's kernels beside the reference's own, recompiled for sm_100a, on the same GPU.

Used by `bench.py --kernels`.  Shapes are those of the Qwen3-0.6B layer (hidden 1,024, 16 query heads on 8 kv
heads of 128, intermediate 3,072, vocabulary 151,936).  Both arms run on one stream (the reference's), are
timed with CUDA events around the replay of a CUDA graph of `iters` back-to-back launches (after warm-up
launches and one untimed replay), and rotate over enough copies of their operands that a launch never finds its
weights or its cache in L2 (the copies together exceed twice the 126 MB).  What "ours" launches is what the engine launches for that shape: the few-rows product cut
along K hands float32 slices to its consumer, so its time is the product's alone, as is the reference's.
"""
import math

import torch

from llmgen_b200.kernels import ops
from llmgen_b200.parts.mlp import interleave_gate_up

from . import reference_kernels as ref

H, NQ, NKV, HD, F, V = 1024, 16, 8, 128, 3072, 151936
PAGE = 16
L2_BYTES = 126 << 20


def _copies(nbytes: int) -> int:
    return max(2, math.ceil(2.2 * L2_BYTES / max(nbytes, 1)))


def time_us(fn, copies: int, iters: int = 40) -> float:
    """Mean microseconds of fn(i % copies) over `iters` launches recorded into one CUDA graph on the
    reference's stream and replayed: device time of back-to-back launches, without the host's launch cost
    (about 8 us a call from Python, more than most of these kernels take)."""
    s = ref.stream()
    # The reference's stream does not wait for torch's default stream (it is created non-blocking): whatever
    # filled the operands, on whichever stream, has to be finished before a launch here reads them.
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        for i in range(2):
            fn(i % copies)                      # loads modules, sets attributes: nothing of that inside the capture
        s.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        for i in range(iters):
            fn(i % copies)
    with torch.cuda.stream(s):
        graph.replay()
        s.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        s.synchronize()
    ops.check_tc_errors(torch.device("cuda:0"))
    ref.check("timed loop")
    return start.elapsed_time(end) * 1e3 / iters


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


# ------------------------------------------------------------------------------ products
def products(rows=(1, 8, 64, 256, 512, 2048)):
    out = []
    shapes = [("qkv", (NQ + 2 * NKV) * HD, H), ("o_proj", H, NQ * HD), ("down", H, F), ("lm_head", V, H)]
    for name, N, K in shapes:
        n = _copies(N * K * 2) if name != "lm_head" else 2
        ws = [_bf(N, K, scale=0.05) for _ in range(n)]
        for M in rows:
            if name == "lm_head" and M > 64:
                continue
            x = _bf(M, K)
            y_ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            t_ref = time_us(lambda i: ref.linear(y_ref, x, ws[i]), n)
            # the choice parts/linear.py makes: W straight into mma.sync up to ROWS8_BEST_ROWS, the few-rows tcgen05
            # product up to SKINNY_BEST_ROWS, the tiled one above, each cut along K (float32 slices for the consumer)
            # where that fills the SMs
            few = M <= ops.SKINNY_BEST_ROWS
            splits = ops.gemm_skinny_splits(M, N, K) if few else ops.gemm_tc_splits(M, N, K)
            if name == "lm_head":
                splits = 1                                   # float32 logits, never cut
            if name != "lm_head" and M <= ops.ROWS8_BEST_ROWS and ops.gemm_rows8_usable(x, ws[0]):
                slices = ops.gemm_rows8_slices(N, K)
                part8 = torch.empty(slices, M, N, dtype=torch.float32, device="cuda")
                ours = lambda i: ops.gemm_rows8(part8, x, ws[i])
                what = f"gemm_rows8 (mma.sync from global memory), {slices} slices of K"
            elif splits > 1:
                part = torch.empty(splits, M, N, dtype=torch.float32, device="cuda")
                if few:
                    ours = lambda i: ops.gemm_skinny(part, x, ws[i], ops.SKINNY_PARTIAL)
                else:
                    ours = lambda i: ops.gemm_tc_sliced(part, x, ws[i])
                what = f"{'gemm_skinny' if few else 'gemm_tc'}, {splits} slices of K"
            else:
                y = torch.empty(M, N, dtype=torch.float32 if name == "lm_head" else torch.bfloat16, device="cuda")
                if few:
                    ours = lambda i: ops.gemm_skinny(y, x, ws[i])
                else:
                    ours = lambda i: ops.gemm_tc(y, x, ws[i])
                what = "gemm_skinny" if few else "gemm_tc"
            t_ours = time_us(ours, n)
            out.append({"kernel": f"{name} [{N} x {K}]", "case": f"M = {M}", "ours": what,
                        "reference": "gemv_kernel" if M <= 2 else "cublasGemmEx", "ours_us": t_ours, "ref_us": t_ref,
                        "bytes": N * K * 2, "flops": 2 * M * N * K})
        del ws
    # gate and up with the activation: one kernel here, two products + silu + mul there
    n = _copies(2 * F * H * 2)
    wg, wu = [_bf(F, H, scale=0.05) for _ in range(n)], [_bf(F, H, scale=0.05) for _ in range(n)]
    packed = [interleave_gate_up(g, u).contiguous() for g, u in zip(wg, wu)]
    lib = ref.lib()
    from ctypes import c_size_t, c_void_p
    for M in rows:
        x = _bf(M, H)
        g, u, a = (torch.empty(M, F, dtype=torch.bfloat16, device="cuda") for _ in range(3))

        def theirs(i):
            ref.linear(g, x, wg[i])
            ref.linear(u, x, wu[i])
            lib.cuda_silu(c_void_p(g.data_ptr()), c_void_p(g.data_ptr()), c_size_t(g.numel()))
            lib.cuda_mul(c_void_p(a.data_ptr()), c_void_p(g.data_ptr()), c_void_p(u.data_ptr()), c_size_t(g.numel()))
        act = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
        if M <= ops.ROWS8_GATED_BEST_ROWS and ops.gemm_rows8_gated_usable(x, packed[0]):
            ours = lambda i: ops.gemm_rows8_gated(act, x, packed[i])
            what = "gemm_rows8 (mma.sync from global memory), gated"
        elif M <= ops.SKINNY_CLUSTER_MAX_ROWS:
            cl = min(ops.gemm_skinny_cluster_splits(M, 2 * F, H), 4)
            ours = lambda i: ops.gemm_skinny(act, x, packed[i], ops.SKINNY_CLUSTER_GATED, splits=cl)
            what = f"gemm_skinny, cluster of {cl}, gated"
        else:
            ours = lambda i: ops.gemm_tc(act, x, packed[i], gated=True)
            what = "gemm_tc, gated epilogue"
        out.append({"kernel": f"gate_up + silu*up [2 x {F} x {H}]", "case": f"M = {M}", "ours": what,
                    "reference": "2 products + silu + mul", "ours_us": time_us(ours, n), "ref_us": time_us(theirs, n),
                    "bytes": 2 * F * H * 2, "flops": 4 * M * F * H})
    return out


# ------------------------------------------------------------------------------ attention
def _cache(n_seqs, ctx, copies):
    """`copies` caches of [pages, nkv, PAGE, hd] with shuffled block tables for n_seqs sequences of ctx keys."""
    blocks = (ctx + PAGE - 1) // PAGE
    pages = n_seqs * blocks
    kcs = [_bf(pages, NKV, PAGE, HD) for _ in range(copies)]
    vcs = [_bf(pages, NKV, PAGE, HD) for _ in range(copies)]
    perm = torch.randperm(pages, device="cuda").to(torch.int32)
    bt = perm.view(n_seqs, blocks).contiguous()
    return kcs, vcs, bt, blocks


def decode_attention(cases=((1, 4096), (8, 640), (64, 640), (64, 2048))):
    out = []
    scale = 1.0 / math.sqrt(HD)
    sms = ops.sm_count()
    for S, ctx in cases:
        nbytes = S * ctx * NKV * HD * 2 * 2
        n = _copies(nbytes)
        kcs, vcs, bt, blocks = _cache(S, ctx, n)
        q = _bf(S, NQ * HD)
        ctx_len = torch.full((S,), ctx, dtype=torch.int32, device="cuda")
        cu_q = torch.arange(S + 1, dtype=torch.int32, device="cuda")
        o = torch.empty(S, NQ * HD, dtype=torch.bfloat16, device="cuda")
        # ours: the cut the engine makes (parts/attention.py: two resident blocks per SM, at least 128 keys a part)
        bound = 512
        while bound < ctx:
            bound *= 2
        parts = max(1, min((2 * sms) // max(1, S * NKV), bound // 128, 64))
        scratch = torch.empty(max(ops.attention_decode_scratch_floats(S, NQ, HD, parts), 1), dtype=torch.float32, device="cuda")
        counters = torch.zeros(max(ops.attention_decode_counters(S, NQ, NKV), 1), dtype=torch.int32, device="cuda")
        ours = lambda i: ops.attention_decode(o, q, NQ * HD, kcs[i], vcs[i], bt, blocks, ctx_len, cu_q, S, NQ, NKV, HD, PAGE, 0,
                                              scale, parts, bound, scratch, counters)
        psize = ref.part_size(S)
        max_parts = (4096 + psize - 1) // psize
        part_o = torch.empty(S * NQ * max_parts * HD, dtype=torch.float32, device="cuda")
        part_ml = torch.empty(S * NQ * max_parts * 2, dtype=torch.float32, device="cuda")
        o_ref = torch.empty_like(o)
        theirs = lambda i: ref.attn_decode(o_ref, q, kcs[i], vcs[i], bt, ctx_len, S, NQ, NKV, HD, blocks, PAGE, scale, part_o,
                                           part_ml, psize, max_parts)
        t_ours, t_ref = time_us(ours, n), time_us(theirs, n)
        agree = float((o.float() - o_ref.float()).abs().max())          # both ran on the last copy
        out.append({"kernel": "decode attention", "case": f"{S} x {ctx} keys", "ours": f"attention_decode, {parts} parts",
                    "reference": f"attn_decode_kernel<2> + reduce, parts of {psize}", "ours_us": t_ours, "ref_us": t_ref,
                    "bytes": nbytes, "flops": 4 * S * NQ * HD * ctx, "max_abs_diff": agree})
        del kcs, vcs
    return out


def prefill_attention(lengths=(1024, 2048, 4096)):
    out = []
    scale = 1.0 / math.sqrt(HD)
    for T in lengths:
        kcs, vcs, bt, blocks = _cache(1, T, 2)
        q = _bf(T, NQ * HD)
        ctx_len = torch.tensor([T], dtype=torch.int32, device="cuda")
        cu_q = torch.tensor([0, T], dtype=torch.int32, device="cuda")
        o, o_ref = (torch.empty(T, NQ * HD, dtype=torch.bfloat16, device="cuda") for _ in range(2))
        bq = ops.attention_tc_tile_queries(NQ, NKV, HD, PAGE)
        q0 = list(range(0, T, bq))[::-1]                       # heaviest tiles first, as the engine lists them
        tile_seq = torch.zeros(len(q0), dtype=torch.int32, device="cuda")
        tile_q0 = torch.tensor(q0, dtype=torch.int32, device="cuda")
        ours = lambda i: ops.attention_tc(o, q, NQ * HD, kcs[i], vcs[i], bt, blocks, ctx_len, cu_q, tile_seq, tile_q0, len(q0), T,
                                          NQ, NKV, HD, PAGE, 0, scale)
        tile = ref.attn_prefill_tile()
        r0 = list(range(0, T, tile))
        rseq = torch.zeros(len(r0), dtype=torch.int32, device="cuda")
        rq0 = torch.tensor(r0, dtype=torch.int32, device="cuda")
        theirs = lambda i: ref.attn_prefill(o_ref, q, kcs[i], vcs[i], bt, ctx_len, cu_q, rseq, rq0, len(r0), NQ, NKV, HD, blocks,
                                            PAGE, scale)
        t_ours, t_ref = time_us(ours, 2, 20), time_us(theirs, 2, 20)
        out.append({"kernel": "prompt attention", "case": f"{T} tokens", "ours": f"attention_tc (tcgen05), tiles of {bq}",
                    "reference": f"attn_prefill_tc_kernel<2> (mma.sync), tiles of {tile}", "ours_us": t_ours, "ref_us": t_ref,
                    "bytes": T * (NQ + 2 * NKV) * HD * 2, "flops": 4 * NQ * HD * T * (T + 1) // 2,
                    "max_abs_diff": float((o.float() - o_ref.float()).abs().max())})
    return out


# ------------------------------------------------------------------------------ the small kernels
def prep_and_norm(rows=(8, 2048)):
    out = []
    eps = 1e-6
    half = HD // 2
    inv = 1.0 / torch.pow(torch.tensor(1e6, dtype=torch.float64), torch.arange(0, half, dtype=torch.float64) * 2.0 / HD)
    ang = torch.arange(4096, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().float().cuda().contiguous(), ang.sin().float().cuda().contiguous()
    cos2, sin2 = torch.cat([cos, cos], 1).contiguous(), torch.cat([sin, sin], 1).contiguous()     # the reference's tables
    qg, kg = (1 + 0.1 * torch.randn(HD, device="cuda")), (1 + 0.1 * torch.randn(HD, device="cuda"))
    for T in rows:
        packed = _bf(T, (NQ + 2 * NKV) * HD)
        pages = (T + PAGE - 1) // PAGE + 1
        kc, vc = _bf(pages, NKV, PAGE, HD), _bf(pages, NKV, PAGE, HD)
        pos = torch.arange(T, dtype=torch.int32, device="cuda")
        slots = torch.arange(T, dtype=torch.int32, device="cuda")
        work = packed.clone()

        def ours(i):
            ops.attn_prep(work, kc, vc, pos, slots, cos, sin, qg, kg, NQ, NKV, HD, HD, PAGE, eps)
        q, k, v = (_bf(T, n * HD) for n in (NQ, NKV, NKV))
        qn, kn, qr, kr = torch.empty_like(q), torch.empty_like(k), torch.empty_like(q), torch.empty_like(k)

        def theirs(i):
            ref.rmsnorm(qn.view(-1, HD), q.view(-1, HD), qg, eps)
            ref.rmsnorm(kn.view(-1, HD), k.view(-1, HD), kg, eps)
            ref.rope(qr, qn, cos2, sin2, pos, NQ, HD)
            ref.rope(kr, kn, cos2, sin2, pos, NKV, HD)
            ref.store_kv(kr, v, slots, kc, vc, NKV, HD, PAGE)
        out.append({"kernel": "q/k norm + rotary + cache write", "case": f"{T} tokens", "ours": "attn_prep (one kernel)",
                    "reference": "rmsnorm_head x2 + rope x2 + store_kv", "ours_us": time_us(ours, 1), "ref_us": time_us(theirs, 1),
                    "bytes": 2 * T * (NQ + 2 * NKV) * HD * 2, "flops": 0})
        # residual add + RMSNorm over the hidden width
        resid = torch.randn(T, H, device="cuda")
        delta = _bf(T, H)
        gain = 1 + 0.1 * torch.randn(H, device="cuda")
        y = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
        xr, yr = _bf(T, H), torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
        lib = ref.lib()
        from ctypes import c_size_t, c_void_p

        def theirs_norm(i):
            lib.cuda_add(c_void_p(xr.data_ptr()), c_void_p(xr.data_ptr()), c_void_p(delta.data_ptr()), c_size_t(xr.numel()))
            ref.rmsnorm(yr, xr, gain, eps)
        out.append({"kernel": "residual add + RMSNorm", "case": f"{T} rows of {H}", "ours": "add_rmsnorm (one kernel, float32 residual)",
                    "reference": "add + rmsnorm_row (bfloat16 residual)",
                    "ours_us": time_us(lambda i: ops.add_rmsnorm(resid, delta, gain, y, eps), 1), "ref_us": time_us(theirs_norm, 1),
                    "bytes": T * H * (4 + 4 + 2 + 2), "flops": 0})
    return out


def run_all():
    torch.manual_seed(0)
    rows = []
    # operands are made on the stream that the launches use
    with torch.cuda.stream(ref.stream()):
        for part in (products, decode_attention, prefill_attention, prep_and_norm):
            rows += part()
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
    return rows


def as_markdown(rows) -> str:
    lines = ["| kernel | case | ours | µs | reference (sm_100a build) | µs | ours / reference speed | ours GB/s | ours TFLOP/s |",
             "|---|---|---|---:|---|---:|---:|---:|---:|"]
    for r in rows:
        gbs = r["bytes"] / r["ours_us"] / 1e3
        tf = r["flops"] / r["ours_us"] / 1e6
        lines.append(f"| {r['kernel']} | {r['case']} | {r['ours']} | {r['ours_us']:.1f} | {r['reference']} | {r['ref_us']:.1f} | "
                     f"{r['ref_us'] / r['ours_us']:.2f}x | {gbs:,.0f} | {tf:,.1f} |")
    return "\n".join(lines)
