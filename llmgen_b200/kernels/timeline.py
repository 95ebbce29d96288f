"""Phase timelines of the tensor-core kernels, from builds with their timeline macros.

    python -m llmgen_b200.kernels.timeline gemm_tc M N K [gated] [pairs]
    python -m llmgen_b200.kernels.timeline skinny_chain ROWS
    python -m llmgen_b200.kernels.timeline products
    python -m llmgen_b200.kernels.timeline attention_tc [TOKENS]

`gemm_tc`, `gemm_skinny` and `attention_tc` can be compiled with `-DLLMK_GEMM_TIMELINE`,
`-DLLMK_SKINNY_TIMELINE`, `-DLLMK_ATTN_TIMELINE`: a few blocks then stamp the global timer at their
phases into a device array that an extra entry point copies out.  This module builds such a
library beside the normal one (in the system's temporary folder), runs the workload a few times
and prints the stamps in nanoseconds since the block started.  It is a measuring aid: nothing in
the engine imports it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

from . import build, ops


def _timeline_library(module: str, macro: str) -> ctypes.CDLL:
    out = os.path.join(tempfile.gettempdir(), f"llmgen_b200_{module}_timeline_{os.getuid()}.so")
    cmd = [build.find_nvcc()] + build.ARCH_FLAGS + [f for f in build.NVCC_FLAGS if f != "-lineinfo"] + \
          [f"-D{macro}", "-I", build.CSRC_DIR, "-o", out, os.path.join(build.CSRC_DIR, module + ".cu")]
    subprocess.check_call(cmd)
    lib = ctypes.CDLL(out)
    lib.llmk_last_error.restype = ctypes.c_char_p
    build._loaded[module] = lib          # the bindings in `ops` now call the timeline build
    return lib


def _weights(n: int, k: int) -> torch.Tensor:
    return (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)


def gemm_tc(M: int, N: int, K: int, gated: bool = False, pairs: bool = False) -> None:
    """Stamps of blocks 0 and 1 of `gemm_tc` on an [M, K] x [N, K]^T product: when each 64-wide slice
    of K was in shared memory, when each tile's accumulator was complete and when it was stored."""
    lib = _timeline_library("gemm_tc", "LLMK_GEMM_TIMELINE")
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    ws = [_weights(N, K) for _ in range(4)]
    out = torch.empty(M, N // 2 if gated else N, dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc_set_pair_mode(2 if pairs else 0)
    for i in range(6):
        ops.gemm_tc(out, a, ws[i % 4], gated=gated)
    torch.cuda.synchronize()
    ops.check_tc_errors(out.device)
    stamps = np.zeros(8 * 64, dtype=np.uint64)
    assert lib.llmk_gemm_tc_timeline(stamps.ctypes.data_as(ctypes.c_void_p)) == 0
    stamps = stamps.reshape(8, 64).astype(np.int64)
    print(f"gemm_tc {M} x {N} x {K}{' gated' if gated else ''}{' pairs of blocks' if pairs else ''} (ns since the block started)")
    for b in (0, 1):
        r = stamps[b]
        t0 = r[0]
        slices = [int(r[8 + i] - t0) for i in range(40) if r[8 + i] > t0]
        tiles = [(int(r[48 + 2 * i] - t0), int(r[49 + 2 * i] - t0)) for i in range(4) if r[48 + 2 * i] > t0]
        print(f"block {b}: producer starts {r[1] - t0}, waited for the kernel before {r[2] - t0}, block ends {r[3] - t0}")
        print(f"   slices of K in shared memory at: {slices}")
        print(f"   tiles (accumulator complete, stored): {tiles}")


def skinny_chain(rows: int) -> None:
    """Stamps of the fused few-rows products of a decoder layer's chain at `rows` rows (Qwen3-0.6B
    sizes): o_proj adding to the residual, gate_up normalising its rows itself, down_proj applying
    the activation itself and adding to the residual, qkv normalising its rows itself."""
    lib = _timeline_library("gemm_skinny", "LLMK_SKINNY_TIMELINE")
    H, F, NQ, NKV, HD = 1024, 3072, 16, 8, 128
    nqkv = (NQ + 2 * NKV) * HD
    layers = [dict(qkv=_weights(nqkv, H), o=_weights(H, NQ * HD), gu=_weights(2 * F, H), down=_weights(H, F)) for _ in range(6)]
    s_qkv, s_o = ops.gemm_skinny_splits(rows, nqkv, H), ops.gemm_skinny_splits(rows, H, NQ * HD)
    s_gu, s_dn = ops.gemm_skinny_splits(rows, 2 * F, H), ops.gemm_skinny_splits(rows, H, F)
    f32 = dict(dtype=torch.float32, device="cuda")
    p_qkv, p_o = torch.empty(s_qkv, rows, nqkv, **f32), torch.empty(s_o, rows, H, **f32)
    p_gu, p_dn = torch.empty(s_gu, rows, 2 * F, **f32), torch.empty(s_dn, rows, H, **f32)
    o = torch.randn(rows, NQ * HD, device="cuda").to(torch.bfloat16)
    resid = torch.randn(rows, H, device="cuda")
    gain = torch.ones(H, device="cuda")
    sq = [torch.ones(H // 128, rows, device="cuda") for _ in range(2)]
    tickets = [torch.zeros(H // 128, dtype=torch.int32, device="cuda") for _ in range(2)]

    def chain(i: int) -> None:
        w = layers[i % len(layers)]
        ops.gemm_skinny_fused(p_o, o, w["o"], add_to=resid, squares_out=sq[0], tickets=tickets[0])
        ops.gemm_skinny_fused(p_gu, ops.NormedRows(resid, ops.RowSquares(sq[0]), gain, 1e-6), w["gu"])
        ops.gemm_skinny_fused(p_dn, ops.GatedRows(ops.Partials(p_gu), 16), w["down"], add_to=resid, squares_out=sq[1],
                              tickets=tickets[1])
        ops.gemm_skinny_fused(p_qkv, ops.NormedRows(resid, ops.RowSquares(sq[1]), gain, 1e-6), w["qkv"])

    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        chain(0)
        chain(1)                  # 8 launches: timeline records 0..7
    torch.cuda.synchronize()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(4):        # 16 launches: the records of the last 8 stay
            chain(i)
    torch.cuda.synchronize()
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    ops.check_tc_errors(resid.device)
    stamps = np.zeros(8 * 32 * 16, dtype=np.uint64)
    assert lib.llmk_gemm_skinny_timeline(stamps.ctypes.data_as(ctypes.c_void_p)) == 0
    stamps = stamps.reshape(8, 32, 16).astype(np.int64)
    names = ["block starts", "waited for the kernel before", "operand built", "arrived", "MMA thread sees the operand",
             "MMAs issued", "accumulator complete", "slices stored", "fenced", "ticket taken", "sum added to the residual"]
    kinds = ["o_proj + residual", "norm + gate_up", "activation + down_proj + residual", "norm + qkv"] * 2
    splits = [s_o, s_gu, s_dn, s_qkv] * 2
    base = stamps[0, :splits[0], 0].min()
    print(f"fused chain at {rows} rows (ns; min and max over the blocks of the first tile)")
    for k in range(8):
        rec = stamps[k, :splits[k], :11]
        first = rec[:, 0].min()
        print(f"launch {k} {kinds[k]}: first block starts {first - base} ns after the chain's first")
        for j, name in enumerate(names):
            col = rec[:, j]
            col = col[col >= first]          # blocks that did not run this phase keep the stamp of an earlier launch
            if col.size:
                print(f"   {name:32s} {col.min() - first:7d} .. {col.max() - first:7d}")


def products() -> None:
    """CUDA-event times of `gemm_tc` on the products of a prompt (Qwen3-0.6B sizes) and on larger ones:
    lone blocks, pairs of blocks with 256 x 256 tiles, what the launcher chooses, and the library
    product (cuBLAS through torch.matmul, ungated) for comparison.  Weights of 12 layers in turn."""
    def best_of(fn, rep=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(rep):
                fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1000 / rep)
        return best

    shapes = [("qkv, 2,048 tokens", 2048, 4096, 1024, False), ("o_proj", 2048, 1024, 2048, False),
              ("gate_up (gated)", 2048, 6144, 1024, True), ("down_proj", 2048, 1024, 3072, False),
              ("qkv, 8,192 tokens", 8192, 4096, 1024, False), ("down_proj, 8,192 tokens", 8192, 1024, 3072, False),
              ("4096 x 4096 x 4096", 4096, 4096, 4096, False)]
    print(f"{'product':26s} {'lone':>9s} {'pairs':>9s} {'chosen':>9s} {'library':>9s}   (us; TFLOP/s of the chosen one)")
    for name, M, N, K, gated in shapes:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        ws = [_weights(N, K) for _ in range(12)]
        out = torch.empty(M, N // 2 if gated else N, dtype=torch.bfloat16, device="cuda")
        full = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        turn = [0]

        def ours():
            turn[0] = (turn[0] + 1) % len(ws)
            ops.gemm_tc(out, a, ws[turn[0]], gated=gated)

        def library():
            turn[0] = (turn[0] + 1) % len(ws)
            torch.matmul(a, ws[turn[0]].t(), out=full)

        times = []
        for mode in (0, 2, 1):
            ops.gemm_tc_set_pair_mode(mode)
            times.append(best_of(ours))
        ops.gemm_tc_set_pair_mode(1)
        times.append(best_of(library))
        tflops = 2.0 * M * N * K / (times[2] * 1e-6) / 1e12
        print(f"{name:26s} " + " ".join(f"{t:9.2f}" for t in times) + f"   {tflops:7.0f}")
    ops.check_tc_errors(torch.device("cuda"))


def attention_tc(tokens: int = 2048) -> None:
    """Stamps (SM clock cycles) of the first softmax warp of the heaviest block of `attention_tc` on one
    prompt of `tokens` tokens (16 query heads on 8 kv heads of 128, pages of 16), tile by tile: when the
    loop came round, when S was there, after the row maximum, after the exchange of maxima, after the
    decision on the reference maximum, after P was handed over, at the tile's end."""
    import ctypes as C
    import math
    lib = _timeline_library("attention_tc", "LLMK_ATTN_TIMELINE")
    nq, nkv, hd, page, T = 16, 8, 128, 16, tokens
    n_pages = (T + page - 1) // page
    kc = torch.randn(n_pages, nkv, page, hd, device="cuda").to(torch.bfloat16)
    vc = torch.randn(n_pages, nkv, page, hd, device="cuda").to(torch.bfloat16)
    q = torch.randn(T, nq * hd, device="cuda").to(torch.bfloat16)
    out = torch.empty(T, nq * hd, device="cuda", dtype=torch.bfloat16)
    bt = torch.arange(n_pages, dtype=torch.int32, device="cuda")
    ctx = torch.tensor([T], dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    bq = ops.attention_tc_tile_queries(nq, nkv, hd, page)
    q0 = torch.arange(0, T, bq, dtype=torch.int32, device="cuda").flip(0).contiguous()      # heaviest tile first: block 0
    seq = torch.zeros_like(q0)
    stamps = torch.zeros(16 * 8, dtype=torch.int64, device="cuda")
    ptr = lambda t: C.c_void_p(t.data_ptr())
    for _ in range(3):
        rc = lib.llmk_attention_tc(ptr(out), C.c_longlong(nq * hd), ptr(q), C.c_longlong(nq * hd), C.c_int(T), ptr(kc), ptr(vc),
                                   C.c_longlong(n_pages), ptr(bt), C.c_int(n_pages), ptr(ctx), ptr(cu), ptr(seq), ptr(q0),
                                   C.c_int(q0.numel()), C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page), C.c_int(0),
                                   C.c_float(1 / math.sqrt(hd)), ptr(ops.tc_error_flag(q.device)), C.c_uint(0), C.c_uint(0),
                                   ops._stream(), ptr(stamps))
        if rc != 0:
            raise ops.KernelError(lib.llmk_last_error().decode())
        torch.cuda.synchronize()
    ops.check_tc_errors(q.device)
    t = stamps.cpu().view(16, 8)
    tiles = min(16, (T + 127) // 128)
    print(f"attention_tc, {T} tokens: cycles per key tile of the heaviest block's first softmax warp")
    print("tile   wait for S   pass 1   exchange   reference   pass 2   rest   whole tile")
    for j in range(tiles - 1):
        d = [int(t[j, 1] - t[j, 0]), int(t[j, 2] - t[j, 1]), int(t[j, 3] - t[j, 2]), int(t[j, 4] - t[j, 3]),
             int(t[j, 5] - t[j, 4]), int(t[j, 7] - t[j, 5]), int(t[j + 1, 0] - t[j, 0])]
        print(f"{j:4d} " + " ".join(f"{v:10d}" for v in d))


def main(argv) -> int:
    if argv[:1] == ["attention_tc"] and len(argv) <= 2:
        attention_tc(int(argv[1]) if len(argv) == 2 else 2048)
        return 0
    if argv == ["products"]:
        products()
        return 0
    if len(argv) >= 4 and argv[0] == "gemm_tc":
        gemm_tc(int(argv[1]), int(argv[2]), int(argv[3]), "gated" in argv[4:], "pairs" in argv[4:])
        return 0
    if len(argv) == 2 and argv[0] == "skinny_chain":
        skinny_chain(int(argv[1]))
        return 0
    print(__doc__)
    return 2


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
