"""ctypes bindings of the reference's CUDA kernels compiled for sm_100a (baseline/build_reference_kernels.py).

Only comparisons use this: `bench.py --kernels` (timings on the same B200, same inputs, same loop) and
tests/golden/make_reference_kernel_fixtures.py (outputs that anchor the plain implementation).  The reference
launches on a stream of its own (`global_cuda_stream`, src/backend/cuda/cuda_context.cu:5); `stream()` wraps
it so that both arms of a comparison run and are timed on that one stream.

Entry points and argument orders: src/backend/cuda/linear/linear.cu:74, norm/norm_final.cu:47,
rope/rope_v1.cu:47, attention/attention.cu:35 (store_kv), :209 (decode), :470 (prefill), sample/sample.cu:79.
Part sizes of the split decode by batch size: src/backend/cuda/attention/attention_v1.zig:51-57.
"""
import ctypes
import os
from ctypes import c_float, c_int, c_long, c_size_t, c_void_p

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libllmgen_ref_kernels.so")

_lib = None
_stream = None


def available() -> bool:
    return os.path.isfile(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError(f"{LIB_PATH} is not built: run baseline/build_reference_kernels.py --src <reference checkout>")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.cuda_init.restype = c_int
        _lib.cuda_last_error.restype = c_int
        _lib.cuda_attn_prefill_tile.restype = c_int
        _lib.cuda_sample_scratch_bytes.restype = c_size_t
        rc = _lib.cuda_init(c_size_t(32 << 20))        # the workspace size the reference gives cuBLAS
        if rc != 0:
            raise RuntimeError(f"the reference's cuda_init failed ({rc})")
    return _lib


def stream() -> torch.cuda.Stream:
    """The reference's global stream as a torch stream."""
    global _stream
    if _stream is None:
        handle = c_void_p.in_dll(lib(), "global_cuda_stream").value
        _stream = torch.cuda.ExternalStream(handle)
    return _stream


def _p(t):
    return c_void_p(0 if t is None else t.data_ptr())


def check(what: str) -> None:
    rc = lib().cuda_last_error()
    if rc != 0:
        raise RuntimeError(f"reference kernel {what}: CUDA error {rc}")


def part_size(n_seqs: int) -> int:
    return 512 if n_seqs >= 64 else 256 if n_seqs >= 16 else 128 if n_seqs >= 4 else 64


def linear(y, x, w):
    """y[M, N] (bfloat16 or float32) = x[M, K] w[N, K]^T: its GEMV for M <= 2 (SV_GEMV_MAX_M), cublasGemmEx above."""
    M, K = x.shape
    lib().cuda_linear(_p(y), c_int(1 if y.dtype == torch.float32 else 0), _p(x), _p(w), c_int(M), c_int(w.shape[0]), c_int(K))


def rmsnorm(out, x, w, eps):
    rows = x.numel() // x.shape[-1]
    lib().cuda_rmsnorm(_p(out), _p(x), _p(w), c_long(rows), c_int(x.shape[-1]), c_float(eps))


def rope(out, x, cos_tab, sin_tab, positions, n_head, hd):
    """x, out [T, n_head, 128]; cos / sin tables [positions, 128] float32 whose two halves hold the same angles."""
    lib().cuda_rope(_p(out), _p(x), _p(cos_tab), _p(sin_tab), _p(positions), c_int(x.shape[0]), c_int(n_head), c_int(hd))


def store_kv(k, v, slots, kc, vc, nkv, hd, block_size):
    lib().cuda_store_kv(_p(k), _p(v), _p(slots), _p(kc), _p(vc), c_int(k.shape[0]), c_int(nkv), c_int(hd), c_int(block_size))


def attn_decode(out, q, kc, vc, block_tables, ctx_lens, n_seqs, nq, nkv, hd, max_blocks, block_size, scale, part_o, part_ml,
                psize, max_parts):
    lib().cuda_attn_decode(_p(out), _p(q), _p(kc), _p(vc), _p(block_tables), _p(ctx_lens), c_int(n_seqs), c_int(nq), c_int(nkv),
                           c_int(hd), c_int(max_blocks), c_int(block_size), c_float(scale), _p(part_o), _p(part_ml),
                           c_int(psize), c_int(max_parts))


def attn_prefill_tile() -> int:
    return int(lib().cuda_attn_prefill_tile())


def attn_prefill(out, q, kc, vc, block_tables, ctx_lens, cu_q, tile_seq, tile_q0, n_tiles, nq, nkv, hd, max_blocks, block_size, scale):
    lib().cuda_attn_prefill(_p(out), _p(q), _p(kc), _p(vc), _p(block_tables), _p(ctx_lens), _p(cu_q), _p(tile_seq), _p(tile_q0),
                            c_int(n_tiles), c_int(nq), c_int(nkv), c_int(hd), c_int(max_blocks), c_int(block_size), c_float(scale))


def sample(out_ids, logits_bf16, temps, seed, scratch):
    S, V = logits_bf16.shape
    lib().cuda_sample(_p(out_ids), _p(logits_bf16), _p(temps), _p(seed), c_int(S), c_int(V), _p(scratch))


def sample_scratch_bytes(max_rows: int) -> int:
    return int(lib().cuda_sample_scratch_bytes(c_int(max_rows)))
