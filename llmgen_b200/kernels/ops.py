"""Python bindings of the CUDA kernels: thin functions from torch tensors to the C ABI.

torch is used as the allocator and for stream handles only; every function launches on
`torch.cuda.current_stream()`, allocates nothing and never synchronises, so a sequence of
calls can be captured into a CUDA graph.  There is no CPU path: a tensor that is not on a
CUDA device raises `KernelError`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, Optional, Tuple

import torch

from . import build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 storage, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernel arguments must live on a CUDA device (there is no CPU path)")
    return c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> c_void_p:
    """The current stream's handle.  Asked of torch's C layer directly where it offers that: the
    `torch.cuda.current_stream()` object costs several microseconds, more than a launch."""
    if _raw_stream is not None and _raw_device is not None:
        return c_void_p(_raw_stream(_raw_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class _Counter:
    """How many kernels of this package were launched (a claim for benchmarks' records)."""
    launches = 0


def launches() -> int:
    return _Counter.launches


def _check(lib, rc: int, n_kernels: int = 1) -> None:
    if rc != 0:
        raise KernelError(lib.llmk_last_error().decode("utf-8", "replace"))
    _Counter.launches += n_kernels


def _row_stride(t: torch.Tensor) -> int:
    if t.dim() < 2:
        return t.shape[-1] if t.dim() == 1 else 1
    if t.stride(-1) != 1:
        raise KernelError("kernel operands must be contiguous in their last dimension")
    return t.stride(-2)


class Partials:
    """The result of a matrix product cut along K: float32 slices [splits, rows, cols] whose sum, in
    slice order, is the product.  The kernels that consume a product (`add_rmsnorm`, `attn_prep`,
    `attention_decode`, `silu_mul`) take a `Partials` in place of the finished array and do the sum themselves."""

    def __init__(self, tensor: torch.Tensor):
        if tensor.dim() != 3 or tensor.dtype != torch.float32 or not tensor.is_contiguous():
            raise KernelError("partial sums are a contiguous float32 [splits, rows, cols] array")
        self.tensor = tensor
        self.splits, self.rows, self.cols = tensor.shape

    @property
    def split_stride(self) -> int:
        return self.rows * self.cols

    def sum(self) -> torch.Tensor:
        """The finished product (float32), for callers that have no kernel taking slices."""
        return self.tensor.sum(dim=0)


# ---------------------------------------------------------------------------- elementwise
def embed_rows(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, bad_flag: Optional[torch.Tensor] = None,
               ids_from: Optional[torch.Tensor] = None, sampled: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """out[t] (float32 [n, H]) = table[ids[t]] * scale; ids int32 on the device.  With `ids_from` and
    `sampled` (int32, device) a row whose ids_from[t] >= 0 takes the id sampled[ids_from[t]]."""
    lib = build.load("elementwise")
    n, H = out.shape
    _check(lib, lib.llmk_embed_rows(_ptr(out), _ptr(table), _ptr(ids), _ptr(ids_from), _ptr(sampled), c_int(n), c_int(H),
                                    c_int(table.shape[0]), _ptr(bad_flag), c_int(dtype_code(table.dtype)), c_float(scale),
                                    _stream()))


def logit_cap(logits: torch.Tensor, cap: float) -> None:
    """logits (float32, contiguous) = cap * tanh(logits / cap), in place."""
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("logit_cap: logits must be contiguous float32")
    lib = build.load("elementwise")
    _check(lib, lib.llmk_logit_cap(_ptr(logits), c_longlong(logits.numel()), c_float(cap), _stream()))


def add_rmsnorm(resid: torch.Tensor, delta, weight: torch.Tensor, out: torch.Tensor,
                eps: float, weight_offset: float = 0.0, rows: Optional[torch.Tensor] = None,
                write_resid: bool = True) -> None:
    """resid (float32 [n, H]) += delta; out = rmsnorm(resid) * (weight + offset).  `delta` is an
    array of the output's dtype, a `Partials`, or None.

    With `rows` (int32 [m]) output row r is computed from source row rows[r] and the
    residual is left untouched."""
    lib = build.load("elementwise")
    H = resid.shape[-1]
    n_rows = out.shape[0]
    if resid.dtype != torch.float32 or weight.dtype != torch.float32:
        raise KernelError("add_rmsnorm: residual and gain must be float32")
    splits, split_stride = 0, 0
    if isinstance(delta, Partials):
        if delta.cols != H or delta.rows != resid.shape[0]:
            raise KernelError("add_rmsnorm: partial sums do not have the residual's shape")
        splits, split_stride, delta = delta.splits, delta.split_stride, delta.tensor
    elif delta is not None and (delta.dtype != out.dtype or not delta.is_contiguous()):
        raise KernelError("add_rmsnorm: delta must be contiguous and of the output's dtype")
    if rows is not None:
        write_resid = False
    _check(lib, lib.llmk_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), c_int(n_rows),
                                     c_int(H), c_float(eps), c_float(weight_offset), c_int(1 if write_resid else 0),
                                     c_int(splits), c_longlong(split_stride), c_int(dtype_code(out.dtype)), _stream()))


def silu_mul(out: torch.Tensor, gate_up, group: int = 0) -> None:
    """out[n, F] = silu(gate) * up, where gate_up[n, 2F] (an array or a `Partials`) alternates `group`
    gate columns and `group` up columns (group 0 or F: gate in columns [0, F), up in [F, 2F))."""
    lib = build.load("elementwise")
    n, F = out.shape
    splits, split_stride = 0, 0
    if isinstance(gate_up, Partials):
        splits, split_stride, ld = gate_up.splits, gate_up.split_stride, gate_up.cols
        gate_up = gate_up.tensor
    else:
        ld = _row_stride(gate_up)
    _check(lib, lib.llmk_silu_mul(_ptr(out), _ptr(gate_up), c_int(n), c_int(F), c_int(ld),
                                  c_int(group if group else F), c_int(splits), c_longlong(split_stride),
                                  c_int(dtype_code(out.dtype)), _stream()))


def widen(out: torch.Tensor, src: torch.Tensor) -> None:
    """out (float32) = src, element by element (both contiguous)."""
    lib = build.load("elementwise")
    _check(lib, lib.llmk_widen(_ptr(out), _ptr(src), c_longlong(src.numel()), c_int(dtype_code(src.dtype)), _stream()))


# ------------------------------------------------------------------------------ attn_prep
# Codes of the C ABI (csrc/common.cuh).  "half": pairs (i, i + rot / 2), the reference's pairing
# (src/backend/cpu/rope.zig:13-45); "interleaved": pairs (2i, 2i + 1), which no kernel here implements yet:
# a position encoding that names it is refused by the kernel with a message, not rotated wrongly.
ROTARY_PAIRINGS = {"half": 0, "interleaved": 1}
HEAD_NORMS = {"rmsnorm": 0}


def pairing_code(pairing: str) -> int:
    try:
        return ROTARY_PAIRINGS[pairing]
    except KeyError:
        raise KernelError(f"unknown rotary pairing {pairing!r} (known: {', '.join(ROTARY_PAIRINGS)})") from None


def head_norm_code(kind: str) -> int:
    try:
        return HEAD_NORMS[kind]
    except KeyError:
        raise KernelError(f"no kernel normalises heads with {kind!r} (known: {', '.join(HEAD_NORMS)})") from None


def attn_prep_set_by_token(on: bool) -> None:
    """Which 16-byte variant `attn_prep` runs on prompts: a warp on several heads of one token at a
    time (the default) or a row at a time (for comparisons and tests)."""
    build.load("attn_prep").llmk_attn_prep_set_by_token(c_int(1 if on else 0))


def attn_prep(qkv, kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
              positions: Optional[torch.Tensor], slots: Optional[torch.Tensor], cos: Optional[torch.Tensor],
              sin: Optional[torch.Tensor], q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor],
              nq: int, nk: int, hd: int, rot: int, page_size: int, eps: float,
              q_offset: float = 0.0, k_offset: float = 0.0, q_out: Optional[torch.Tensor] = None,
              pairing: str = "half", head_norm: str = "rmsnorm") -> None:
    """Per-head norm and rotary encoding of q and k, and the cache write of k, v.  `qkv` holds the
    packed rows [n, (nq + 2 nk) hd] as an array (q is then rewritten in place unless `q_out` is
    given) or as a `Partials` (q goes to `q_out`, which gives the storage dtype).  `pairing` says which
    values of a head the rotary encoding turns together and `head_norm` which norm runs over a head
    (see `ROTARY_PAIRINGS`, `HEAD_NORMS`); the kernel refuses the ones it does not implement."""
    lib = build.load("attn_prep")
    nkv_cache = kcache.shape[1] if kcache is not None else 0
    splits, split_stride = 0, 0
    if isinstance(qkv, Partials):
        if q_out is None:
            raise KernelError("attn_prep: partial sums need a place for q")
        n, stride, src = qkv.rows, qkv.cols, qkv.tensor
        splits, split_stride = qkv.splits, qkv.split_stride
        dtype = q_out.dtype
    else:
        n, stride, src = qkv.shape[0], _row_stride(qkv), qkv
        dtype = qkv.dtype
        if q_out is None:
            q_out = qkv
    if q_out.dtype != dtype:
        raise KernelError("attn_prep: q_out must have the storage dtype")
    _check(lib, lib.llmk_attn_prep(_ptr(src), c_longlong(stride), c_int(splits), c_longlong(split_stride),
                                   _ptr(q_out), c_longlong(_row_stride(q_out)), _ptr(kcache), _ptr(vcache),
                                   _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin), _ptr(q_gain), _ptr(k_gain),
                                   c_int(n), c_int(nq), c_int(nk), c_int(nkv_cache), c_int(hd), c_int(rot),
                                   c_int(page_size), c_float(eps), c_float(q_offset), c_float(k_offset),
                                   c_int(pairing_code(pairing)), c_int(head_norm_code(head_norm)),
                                   c_int(dtype_code(dtype)), _stream()))


# ------------------------------------------------------------------------- matrix products
def gemm_simt(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, accumulate: bool = False) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on the CUDA cores (float32 multiply-add, fixed k order)."""
    lib = build.load("gemm_simt")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm: shapes a{list(a.shape)} w{list(w.shape)} out{list(out.shape)} do not fit")
    if a.dtype != w.dtype:
        raise KernelError("gemm: a and w must share a dtype")
    _check(lib, lib.llmk_gemm_simt(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K),
                                   c_longlong(_row_stride(a)), c_longlong(_row_stride(w)), c_longlong(_row_stride(out)),
                                   c_int(1 if accumulate else 0), c_int(dtype_code(a.dtype)),
                                   c_int(dtype_code(out.dtype)), _stream()))


GEMV_MAX_ROWS = 4


def gemv_bf16(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, accumulate: bool = False) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T for M <= 4 in bfloat16, float32 accumulation."""
    lib = build.load("gemv")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemv: shapes a{list(a.shape)} w{list(w.shape)} out{list(out.shape)} do not fit")
    _check(lib, lib.llmk_gemv_bf16(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K),
                                   c_longlong(_row_stride(a)), c_longlong(_row_stride(w)), c_longlong(_row_stride(out)),
                                   c_int(1 if accumulate else 0), c_int(dtype_code(out.dtype)), _stream()))


def gemv_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[0] <= GEMV_MAX_ROWS and a.shape[1] % 8 == 0
            and _row_stride(a) % 8 == 0 and _row_stride(w) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_tc_plans = {}


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """Into how many slices of K the tiled product is best cut when its tiles are too few for the SMs (1: not cut)."""
    key = (M, N, K)
    v = _tc_plans.get(key)
    if v is None:
        v = int(build.load("gemm_tc").llmk_gemm_tc_splits(c_int(M), c_int(N), c_int(K)))
        _tc_plans[key] = v
    return v


def gemm_tc_sliced(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """The tiled tensor-core product cut along K: out is float32 [splits, M, N] and receives the sums
    of `splits` slices of K, for a consumer that adds them up (`Partials`)."""
    lib = build.load("gemm_tc")
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError(f"gemm_tc: operands a{list(a.shape)} {a.dtype} w{list(w.shape)} {w.dtype} do not fit")
    if out.dim() != 3 or out.shape[1] != M or out.shape[2] != N or out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("gemm_tc: the slices go to a contiguous float32 [splits, M, N] array")
    _check(lib, lib.llmk_gemm_tc_sliced(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K), c_longlong(_row_stride(a)),
                                        c_longlong(_row_stride(w)), c_longlong(N), c_int(out.shape[0]),
                                        _ptr(tc_error_flag(a.device)), c_int(1), _stream()))


def gemm_tc_set_pair_mode(mode: int) -> None:
    """How `gemm_tc` uses pairs of blocks on 256-row tiles (`tcgen05.mma.cta_group::2`): 0 never,
    1 where the product has the rows for it (the default), 2 / 3 always, with tiles 256 / 128 columns
    wide (for measurements and tests)."""
    build.load("gemm_tc").llmk_gemm_tc_set_pair_mode(c_int(mode))


def gemm_tc_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    """True when the tensor-core product takes these operands: bfloat16, rows starting on 16-byte
    boundaries (what its TMA loads need)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and _row_stride(a) % 8 == 0 and _row_stride(w) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_status = {}      # device (object or its string) -> (both flags, view of [0], view of [1])


def _status_of(device):
    entry = _status.get(device)
    if entry is None:
        entry = _status.get(str(device))
        if entry is None:
            flags = torch.zeros(2, dtype=torch.int32, device=device)
            entry = (flags, flags[0:1], flags[1:2])
            _status[str(device)] = entry
        _status[device] = entry              # the device object itself as a second key: no string per launch
    return entry


def status_flags(device) -> torch.Tensor:
    """Two device ints that kernels raise and the engine reads with a step's results: [0] a kernel's error
    (1: a bounded wait ran out; 2: a sequence longer than its attention launch was sized for), [1] a token
    id outside the vocabulary met by the embedding kernel."""
    return _status_of(device)[0]


def tc_error_flag(device) -> torch.Tensor:
    """Device int that a kernel raises when one of its bounded waits gave up or an input broke its bounds."""
    return _status_of(device)[1]


def bad_token_flag(device) -> torch.Tensor:
    """Device int that `embed_rows` raises when it meets an id outside the table."""
    return _status_of(device)[2]


def status_message(kernel_error: int, bad_token: int) -> Optional[str]:
    """What the two flags say, or None when both are clear."""
    if kernel_error == 2:
        return "a sequence was longer than the bound its attention launch was sized for (results of that step are invalid)"
    if kernel_error != 0:
        return "a kernel gave up waiting on a barrier (results of that step are invalid)"
    if bad_token != 0:
        return "a token id outside the vocabulary reached the embedding (its row was read as zeros)"
    return None


def check_tc_errors(device) -> None:
    """Raise if a kernel reported a wait that ran out or an input beyond its launch's bounds (synchronises)."""
    entry = _status.get(str(device))
    code = int(entry[1].item()) if entry is not None else 0
    if code != 0:
        entry[1].zero_()
        raise KernelError(status_message(code, 0))


_sm_counts: Dict[str, int] = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (launch plans are made from it, not from a constant)."""
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    key = str(dev)
    if key not in _sm_counts:
        _sm_counts[key] = int(torch.cuda.get_device_properties(dev).multi_processor_count)
    return _sm_counts[key]


def gemm_tc(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, gated: bool = False, pdl: bool = True) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on the tensor cores (tcgen05), bfloat16 operands, float32
    accumulation; `out` is bfloat16 or float32.  With `gated`, w interleaves gate and up rows in
    groups of 16 and out[M, N/2] = silu(gate) * up.  `pdl`: launched as a programmatic dependent of the
    kernel before it, like every other kernel here (its set-up then runs under that kernel's tail; a
    2,048-token prompt took 4.85 ms without and 4.45 ms with it)."""
    lib = build.load("gemm_tc")
    M, K = a.shape
    N = w.shape[0]
    n_out = N // 2 if gated else N
    if w.shape[1] != K or out.shape[0] != M or out.shape[1] != n_out:
        raise KernelError(f"gemm_tc: shapes a{list(a.shape)} w{list(w.shape)} out{list(out.shape)} do not fit")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: operands must be bfloat16")
    _check(lib, lib.llmk_gemm_tc(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K),
                                 c_longlong(_row_stride(a)), c_longlong(_row_stride(w)), c_longlong(_row_stride(out)),
                                 c_int(1 if gated else 0), c_int(dtype_code(out.dtype)), _ptr(tc_error_flag(a.device)),
                                 c_int(1 if pdl else 0), _stream()))


ROWS8_MAX_ROWS = 8           # what the kernel takes
ROWS8_BEST_ROWS = 4          # up to here the engine uses it (decode steps of 1 / 2 / 4 / 8 sequences: +2.3 / +5.5 / +0.7 / -1.0 %)
ROWS8_GATED_BEST_ROWS = 1    # and its gated form (a step of one sequence 0.780 -> 0.767 ms; of 2 and 4: 0.773 -> 0.817, 0.898 -> 1.015)
_rows8_plans = {}


def gemm_rows8_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the product for up to 8 rows that loads W straight from global memory into `mma.sync`
    (csrc/gemm_rows8.cu) takes these operands."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.shape[0] > ROWS8_MAX_ROWS:
        return False
    lib = build.load("gemm_rows8")
    M, K = a.shape
    return bool(lib.llmk_gemm_rows8_usable(_ptr(a), _ptr(w), c_int(M), c_int(w.shape[0]), c_int(K), c_longlong(_row_stride(a)),
                                           c_longlong(_row_stride(w))))


def gemm_rows8_slices(N: int, K: int) -> int:
    """Into how many slices of K that product cuts [M, K] x [N, K]^T."""
    v = _rows8_plans.get((N, K))
    if v is None:
        v = int(build.load("gemm_rows8").llmk_gemm_rows8_slices(c_int(N), c_int(K)))
        _rows8_plans[(N, K)] = v
    return v


def gemm_rows8(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[slices, M, N] (float32, contiguous; slices = gemm_rows8_slices(N, K)) = the partial sums of a[M, K] @ w[N, K]^T
    over the slices of K, M <= 8."""
    lib = build.load("gemm_rows8")
    M, K = a.shape
    N = w.shape[0]
    if out.dtype != torch.float32 or not out.is_contiguous() or tuple(out.shape) != (gemm_rows8_slices(N, K), M, N) or w.shape[1] != K:
        raise KernelError(f"gemm_rows8: a{list(a.shape)} w{list(w.shape)} need contiguous float32 slices "
                          f"[{gemm_rows8_slices(N, K)}, {M}, {N}], got {list(out.shape)} {out.dtype}")
    _check(lib, lib.llmk_gemm_rows8(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K), c_longlong(_row_stride(a)),
                                    c_longlong(_row_stride(w)), _stream()))


def gemm_rows8_gated_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the gated form of that product (w interleaving 16 gate and 16 up rows) takes these operands."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.shape[0] > ROWS8_MAX_ROWS:
        return False
    lib = build.load("gemm_rows8")
    M, K = a.shape
    return bool(lib.llmk_gemm_rows8_gated_usable(_ptr(a), _ptr(w), c_int(M), c_int(w.shape[0]), c_int(K), c_longlong(_row_stride(a)),
                                                 c_longlong(_row_stride(w))))


def gemm_rows8_gated(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[M, N/2] (bfloat16) = silu(gate) * up of a[M, K] @ w[N, K]^T, w interleaving gate and up rows in groups of 16, M <= 8."""
    lib = build.load("gemm_rows8")
    M, K = a.shape
    N = w.shape[0]
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N // 2) or w.shape[1] != K:
        raise KernelError(f"gemm_rows8_gated: a{list(a.shape)} w{list(w.shape)} need a bfloat16 result [{M}, {N // 2}], got {list(out.shape)} {out.dtype}")
    _check(lib, lib.llmk_gemm_rows8_gated(_ptr(out), c_longlong(_row_stride(out)), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K),
                                          c_longlong(_row_stride(a)), c_longlong(_row_stride(w)), _stream()))


SKINNY_MAX_ROWS = 256        # what the kernel takes
SKINNY_BEST_ROWS = 32        # up to here it is the faster product (measured at 16, 32, 48 and 64 rows against the tiled product cut along K)
# most bytes of float32 slices one cut product leaves: about one 128 x 128 item per SM for the tiled product,
# 8 slices of 64 rows by the widest matrix for the few-rows one
SLICED_PRODUCT_BYTES = 16 << 20
SKINNY_DIRECT, SKINNY_PARTIAL, SKINNY_GATED = 0, 1, 2
SKINNY_CLUSTER_GATED = 5     # slices of K added up inside a cluster (2 or 4), then silu(gate) * up: out[M, N/2]
SKINNY_CLUSTER_MAX_ROWS = 64
_cluster_plans = {}
_skinny_plans = {}


def gemm_skinny_splits(M: int, N: int, K: int) -> int:
    """Into how many slices of K the few-rows product cuts [M, K] x [N, K]^T (1: no cut)."""
    key = (M, N, K)
    v = _skinny_plans.get(key)
    if v is None:
        v = int(build.load("gemm_skinny").llmk_gemm_skinny_splits(c_int(M), c_int(N), c_int(K)))
        _skinny_plans[key] = v
    return v


def gemm_skinny_cluster_splits(M: int, N: int, K: int) -> int:
    """Into how many slices of K the product is cut when a thread-block cluster adds them up
    (1: it is not cut)."""
    key = (M, N, K)
    v = _cluster_plans.get(key)
    if v is None:
        v = int(build.load("gemm_skinny").llmk_gemm_skinny_cluster_splits(c_int(M), c_int(N), c_int(K)))
        _cluster_plans[key] = v
    return v


def gemm_skinny(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, mode: int = SKINNY_DIRECT, splits: int = 1) -> None:
    """The weight-streaming tensor-core product for M <= 256 rows (csrc/gemm_skinny.cu).
    SKINNY_DIRECT: out[M, N]; SKINNY_GATED: out[M, N/2] = silu(gate) * up; SKINNY_PARTIAL: out is
    float32 [splits, M, N] and receives the partial sums of `splits` slices of K;
    SKINNY_CLUSTER_GATED: out[M, N/2] = silu(gate) * up from `splits` slices of K (2 or 4) added up
    inside a thread-block cluster (M <= 64)."""
    lib = build.load("gemm_skinny")
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError(f"gemm_skinny: operands a{list(a.shape)} {a.dtype} w{list(w.shape)} {w.dtype} do not fit")
    if mode == SKINNY_PARTIAL:
        if out.dim() != 3 or out.shape[1] != M or out.shape[2] != N or out.dtype != torch.float32 or not out.is_contiguous():
            raise KernelError("gemm_skinny: partial sums go to a contiguous float32 [splits, M, N] array")
        splits, ldc = out.shape[0], N
    else:
        n_out = N // 2 if mode in (SKINNY_GATED, SKINNY_CLUSTER_GATED) else N
        if out.shape[0] != M or out.shape[1] != n_out:
            raise KernelError(f"gemm_skinny: out{list(out.shape)} does not fit [{M}, {n_out}]")
        splits, ldc = (splits if mode == SKINNY_CLUSTER_GATED else 1), _row_stride(out)
    _check(lib, lib.llmk_gemm_skinny(_ptr(out), _ptr(a), _ptr(w), c_int(M), c_int(N), c_int(K),
                                     c_longlong(_row_stride(a)), c_longlong(_row_stride(w)), c_longlong(ldc),
                                     c_int(splits), c_int(mode), c_int(dtype_code(out.dtype)),
                                     _ptr(tc_error_flag(a.device)), _stream()))


def gemm_skinny_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    return a.shape[0] <= SKINNY_MAX_ROWS and gemm_tc_usable(a, w)


# ------------------------------------------------------------------------------ attention
def attention_tile_queries(nq: int, nkv: int) -> int:
    """Queries per tile of `paged_attention` for this group size."""
    lib = build.load("attention")
    return int(lib.llmk_attention_tile_queries(c_int(nq), c_int(nkv)))


def attention_scratch_floats(n_tokens: int, nq: int, hd: int, num_parts: int) -> int:
    return 0 if num_parts <= 1 else n_tokens * nq * num_parts * (hd + 2)


def paged_attention(out: torch.Tensor, q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                    block_tables: torch.Tensor, max_blocks: int, ctx_len: torch.Tensor, cu_q: torch.Tensor,
                    tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, n_tokens: int, nq: int, nkv: int,
                    hd: int, page_size: int, window: int, scale: float, num_parts: int = 1, part_size: int = 0,
                    scratch: Optional[torch.Tensor] = None) -> None:
    """out[t, nq*hd] = causal GQA of q[t] over the paged cache (see csrc/attention.cu)."""
    lib = build.load("attention")
    if num_parts > 1:
        need = attention_scratch_floats(n_tokens, nq, hd, num_parts)
        if scratch is None or scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"paged_attention: split into {num_parts} parts needs {need} float32 of scratch")
    _check(lib, lib.llmk_paged_attention(_ptr(out), c_longlong(_row_stride(out)), _ptr(q), c_longlong(q_stride),
                                         _ptr(kcache), _ptr(vcache), _ptr(block_tables), c_int(max_blocks),
                                         _ptr(ctx_len), _ptr(cu_q), _ptr(tile_seq), _ptr(tile_q0), c_int(n_tiles),
                                         c_int(n_tokens), c_int(nq), c_int(nkv), c_int(hd), c_int(page_size),
                                         c_int(window), c_float(scale), c_int(num_parts), c_int(part_size),
                                         _ptr(scratch), c_int(dtype_code(q.dtype)), _stream()),
           2 if num_parts > 1 else 1)


def attention_decode_set_cluster_merge(on: bool) -> None:
    """Whether `attention_decode` merges up to 8 key parts through the shared memory of a thread-block
    cluster (the default) or through global memory and a ticket (for measurements and tests)."""
    build.load("attention_decode").llmk_attention_decode_set_cluster_merge(c_int(1 if on else 0))


def attention_decode_usable(nq: int, nkv: int, hd: int, page_size: int) -> bool:
    return bool(build.load("attention_decode").llmk_attention_decode_usable(c_int(nq), c_int(nkv), c_int(hd), c_int(page_size)))


def attention_decode_scratch_floats(n_seqs: int, nq: int, hd: int, parts: int) -> int:
    return 0 if parts <= 1 else n_seqs * nq * parts * (hd + 2)


def attention_decode_counters(n_seqs: int, nq: int, nkv: int) -> int:
    lib = build.load("attention_decode")
    lib.llmk_attention_decode_counters.restype = c_longlong
    return int(lib.llmk_attention_decode_counters(c_int(n_seqs), c_int(nq), c_int(nkv)))


def attention_decode_fuses_prep(hd: int, rot: int) -> bool:
    return bool(build.load("attention_decode").llmk_attention_decode_fuses_prep(c_int(hd), c_int(rot)))


def attention_decode(out: torch.Tensor, q: Optional[torch.Tensor], q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                     block_tables: torch.Tensor, max_blocks: int, ctx_len: torch.Tensor, cu_q: torch.Tensor,
                     n_seqs: int, nq: int, nkv: int, hd: int, page_size: int, window: int, scale: float,
                     parts: int, max_ctx: int, scratch: Optional[torch.Tensor], counters: Optional[torch.Tensor],
                     packed=None, nk: int = 0, rot: int = 0, positions: Optional[torch.Tensor] = None,
                     slots: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
                     sin: Optional[torch.Tensor] = None, q_gain: Optional[torch.Tensor] = None,
                     k_gain: Optional[torch.Tensor] = None, eps: float = 0.0, q_offset: float = 0.0,
                     k_offset: float = 0.0, pairing: str = "half", head_norm: str = "rmsnorm") -> None:
    """out[t] = attention of the single token of each sequence over the paged cache, bfloat16
    (csrc/attention_decode.cu).  `counters` (int32) must be zero before the first call.  With
    `packed` (the q/k/v projection rows as an array or a `Partials`) the kernel also normalises and
    rotates q and k and writes k and v to the cache, and `q` is not read.  `max_ctx` must bound every
    sequence's length: a longer one is skipped and raises the device error flag (`check_tc_errors`)."""
    lib = build.load("attention_decode")
    if kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or (q is not None and q.dtype != torch.bfloat16):
        raise KernelError("attention_decode: bfloat16 only")
    if parts > 1:
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < attention_decode_scratch_floats(n_seqs, nq, hd, parts):
            raise KernelError("attention_decode: scratch too small")
        if counters is None or counters.dtype != torch.int32 or counters.numel() < attention_decode_counters(n_seqs, nq, nkv):
            raise KernelError("attention_decode: counters too small")
    splits, split_stride, packed_stride, src = 0, 0, 0, None
    if isinstance(packed, Partials):
        src, splits, split_stride, packed_stride = packed.tensor, packed.splits, packed.split_stride, packed.cols
    elif packed is not None:
        if packed.dtype != torch.bfloat16:
            raise KernelError("attention_decode: packed rows must be bfloat16 or partial sums")
        src, packed_stride = packed, _row_stride(packed)
    _check(lib, lib.llmk_attention_decode(_ptr(out), c_longlong(_row_stride(out)), _ptr(q), c_longlong(q_stride),
                                          _ptr(kcache), _ptr(vcache), _ptr(block_tables), c_int(max_blocks),
                                          _ptr(ctx_len), _ptr(cu_q), c_int(n_seqs), c_int(nq), c_int(nkv), c_int(hd),
                                          c_int(page_size), c_int(window), c_float(scale), c_int(parts), c_int(max_ctx),
                                          _ptr(scratch), _ptr(counters), _ptr(src), c_longlong(packed_stride),
                                          c_int(splits), c_longlong(split_stride), c_int(nk), c_int(rot),
                                          _ptr(positions), _ptr(slots), _ptr(cos), _ptr(sin), _ptr(q_gain), _ptr(k_gain),
                                          c_float(eps), c_float(q_offset), c_float(k_offset),
                                          c_int(pairing_code(pairing)), c_int(head_norm_code(head_norm)),
                                          _ptr(tc_error_flag(out.device)), _stream()))


def attention_tc_tile_queries(nq: int, nkv: int, hd: int, page_size: int) -> int:
    """Queries per tile of the tensor-core attention; 0 when it does not take these sizes."""
    return int(build.load("attention_tc").llmk_attention_tc_tile_queries(c_int(nq), c_int(nkv), c_int(hd), c_int(page_size)))


def attention_tc(out: torch.Tensor, q: torch.Tensor, q_stride: int, kcache: torch.Tensor, vcache: torch.Tensor,
                 block_tables: torch.Tensor, max_blocks: int, ctx_len: torch.Tensor, cu_q: torch.Tensor,
                 tile_seq: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int, n_tokens: int, nq: int, nkv: int,
                 hd: int, page_size: int, window: int, scale: float, v_lbo: int = 0, v_sbo: int = 0) -> None:
    """out[t, nq*hd] = causal GQA of q[t] over the paged cache on the tensor cores, bfloat16
    (csrc/attention_tc.cu).  q is [n_tokens, >= nq*hd] with row stride q_stride."""
    lib = build.load("attention_tc")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_tc: bfloat16 only")
    _check(lib, lib.llmk_attention_tc(_ptr(out), c_longlong(_row_stride(out)), _ptr(q), c_longlong(q_stride),
                                      c_int(n_tokens), _ptr(kcache), _ptr(vcache), c_longlong(kcache.shape[0]),
                                      _ptr(block_tables), c_int(max_blocks), _ptr(ctx_len), _ptr(cu_q),
                                      _ptr(tile_seq), _ptr(tile_q0), c_int(n_tiles), c_int(nq), c_int(nkv), c_int(hd),
                                      c_int(page_size), c_int(window), c_float(scale), _ptr(tc_error_flag(q.device)),
                                      ctypes.c_uint(v_lbo), ctypes.c_uint(v_sbo), _stream()))


# ------------------------------------------------------------------------------- sampling
SAMPLE_SPLIT = 32
_SAMPLE_ROW_BYTES = SAMPLE_SPLIT * 8 + 4        # a row's candidates and its ticket counter


def sample_scratch_bytes(max_rows: int) -> int:
    return max_rows * _SAMPLE_ROW_BYTES


def sample_scratch(max_rows: int, device) -> torch.Tensor:
    """Scratch for `sample` with up to `max_rows` rows: zeroed, because the ticket counters in it must start
    at zero (every launch leaves them at zero)."""
    return torch.zeros(sample_scratch_bytes(max_rows) // 4, dtype=torch.int32, device=device)


def sample(out_ids: torch.Tensor, logits: torch.Tensor, temps: torch.Tensor, seed: Optional[torch.Tensor],
           scratch: torch.Tensor, row_keys: Optional[torch.Tensor] = None) -> None:
    """out_ids[s] (int32) = argmax or Gumbel-max draw of logits[s] (float32 [n, V]); `scratch` from
    `sample_scratch`.  The random numbers of row s come from `seed` (one 64-bit value) and s, or, with
    `row_keys` (64 bits a row, as int64 or pairs of int32), from that row's key alone."""
    lib = build.load("sampling")
    n, V = logits.shape
    if logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32")
    rows = scratch.numel() * scratch.element_size() // _SAMPLE_ROW_BYTES
    if rows < n:
        raise KernelError("sample: scratch too small")
    if row_keys is not None and row_keys.numel() * row_keys.element_size() < 8 * n:
        raise KernelError("sample: one 64-bit key per row is required")
    _check(lib, lib.llmk_sample(_ptr(out_ids), _ptr(logits), c_longlong(_row_stride(logits)), _ptr(temps),
                                _ptr(seed), _ptr(row_keys), c_int(n), c_int(V), _ptr(scratch), c_int(rows), _stream()))
