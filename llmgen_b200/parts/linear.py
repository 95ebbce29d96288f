"""y = x W^T: the one place that chooses a matrix-product kernel.

    float32 engine   CUDA-core kernel with a fixed summation order (csrc/gemm_simt.cu)
    bfloat16 engine  up to 256 rows: the weight-streaming tensor-core kernel with swapped operands
                     (csrc/gemm_skinny.cu), cut along K so that every SM streams a share of W; the
                     float32 slices come back as an `ops.Partials`, which the consuming kernel adds
                     up (LLMGEN_SPLITK=cluster adds them up inside a thread-block cluster instead);
                     more rows: the tiled tensor-core kernel (csrc/gemm_tc.cu: TMA, tcgen05.mma,
                     tensor memory); operands TMA refuses (rows not on 16-byte boundaries): the
                     CUDA-core weight-streaming kernel for up to 4 rows (csrc/gemv.cu), else the
                     CUDA-core product.

The reference uses its own GEMV for M <= 2 and `cublasGemmEx` above
(src/backend/cuda/linear/linear.cu:53-96).  Setting LLMGEN_GEMM=lib swaps the tensor-core kernel
for the library product (cuBLAS through torch.matmul), for comparisons; LLMGEN_GEMM=simt forces the
CUDA-core kernel everywhere.

Weight layout [out, in] row-major, no bias (src/module/linear.zig:48-82).
"""
from __future__ import annotations

import os

import torch

from ..kernels import ops

_FORCE = os.environ.get("LLMGEN_GEMM", "")
_SPLITK = os.environ.get("LLMGEN_SPLITK", "")      # "cluster": add the slices of K up inside a thread-block cluster
# "chain": at up to 16 rows the few-rows products of a layer build their operands themselves (norm,
# gated activation) and add their results to the residual.  Measured slower than the separate
# kernels (the same dependent memory round trips, now inside the products): not the default.
FUSE_CHAIN = os.environ.get("LLMGEN_FUSE", "") == "chain"
# "1": the tiled product of many rows and few columns is cut along K too (float32 slices for the norm to
# add).  Measured on a 2,048-token prompt: the products win what the norms lose (5.02 against 5.04 ms
# a step), so it is not the default.
_TC_SPLITK = os.environ.get("LLMGEN_TC_SPLITK", "0") == "1"
FUSE_CHAIN_MAX_ROWS = 16
# "fused": at up to 16 rows the residual add and the norm before a few-rows product are done by the product
# itself (the slices of K of a tile, a cluster, exchange their shares of the sums of squares).  Every tile's
# cluster then reads the slices and the residual again, 32 to 48 times the same lines at once: measured
# 1.150 ms a decode step against 0.916 ms with the norm as a kernel of its own.  Not the default.
ADDNORM = os.environ.get("LLMGEN_ADDNORM", "") == "fused"

GEMM_MODULES = ("gemm_simt", "gemv", "gemm_tc", "gemm_skinny")


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T; `out` may be float32 for a bfloat16 product."""
    if x.shape[0] == 0:
        return out
    if x.dtype == torch.float32 or _FORCE == "simt":
        ops.gemm_simt(out, x, w)
    elif _FORCE == "" and ops.gemm_skinny_usable(x, w):
        ops.gemm_skinny(out, x, w)
    elif ops.gemv_usable(x, w):
        ops.gemv_bf16(out, x, w)
    elif _FORCE == "lib" and out.dtype == x.dtype:
        torch.matmul(x, w.t(), out=out)
    elif ops.gemm_tc_usable(x, w):
        ops.gemm_tc(out, x, w)
    else:
        ops.gemm_simt(out, x, w)
    return out


def _fused(ws, name: str, x, w: torch.Tensor, add_to):
    """The few-rows product with its neighbours folded in, when it can take these operands: the
    slices as `ops.Partials`, or, with `add_to`, `ops.RowSquares` after the sum went into `add_to`.
    None: it cannot."""
    if _FORCE != "" or _SPLITK != "" or w.dtype != torch.bfloat16:
        return None
    M, K = x.shape
    N = w.shape[0]
    if not (0 < M <= min(FUSE_CHAIN_MAX_ROWS, ops.SKINNY_FUSED_MAX_ROWS)):
        return None
    splits = ops.gemm_skinny_splits(M, N, K)
    if not ops.gemm_skinny_fused_usable(x, w, splits, add_to=add_to):
        return None
    part = ws.flat(name + "_slices", splits * M * N, torch.float32).view(splits, M, N)
    if add_to is None:
        ops.gemm_skinny_fused(part, x, w)
        return ops.Partials(part)
    tiles = (N + 127) // 128
    squares = ws.flat(name + "_squares", tiles * M, torch.float32).view(tiles, M)
    tickets = ws.flat(name + "_tickets", tiles, torch.int32, zero=True)
    ops.gemm_skinny_fused(part, x, w, add_to=add_to, squares_out=squares, tickets=tickets)
    return ops.RowSquares(squares)


def linear_sliced(ws, name: str, x, w: torch.Tensor, out_dtype: torch.dtype, add_to: torch.Tensor = None):
    """x W^T into the workspace buffer `name`: the finished [M, N] array, or, when the few-rows
    kernel cuts the product along K, an `ops.Partials` for a consumer that adds the slices.

    `x` may be an operand that is not computed yet (`ops.NormedRows`, `ops.GatedRows`): the few-rows
    kernel builds it block by block, otherwise it is computed here first.  With `add_to` (the
    float32 residual) the kernel may add the product to it and return `ops.RowSquares`; whatever
    else comes back has not been added."""
    if isinstance(x, ops.AddNormRows):
        M, N = x.shape[0], w.shape[0]
        splits = ops.gemm_skinny_addnorm_splits(x, w, False) if (_FORCE == "" and _SPLITK == "") else 0
        if splits >= 2:
            part = ws.flat(name + "_slices", splits * M * N, torch.float32).view(splits, M, N)
            ops.gemm_skinny_addnorm(part, x, w, splits)
            return ops.Partials(part)
        x = x.materialize(ws.buffer(name + "_x", M, x.shape[1], out_dtype))
    lazy = not isinstance(x, torch.Tensor)
    if lazy or (add_to is not None and FUSE_CHAIN):
        done = _fused(ws, name, x, w, add_to)
        if done is None and add_to is not None and lazy:
            done = _fused(ws, name, x, w, None)          # the operand at least
        if done is not None:
            return done
        if lazy:
            x = x.materialize(ws.buffer(name + "_x", x.shape[0], x.shape[1], out_dtype))
    M, N = x.shape[0], w.shape[0]
    if M > 0 and x.dtype == torch.bfloat16 and _FORCE == "" and ops.gemm_skinny_usable(x, w):
        if M <= ops.SKINNY_CLUSTER_MAX_ROWS and _SPLITK == "cluster":
            # the slices are added up inside a thread-block cluster: one float32 array comes back.
            # Measured at the benchmark's sizes this costs 1-1.7 us more per product than writing the
            # slices, and saves 1.2 us in the kernel that adds them: not the default.
            splits = ops.gemm_skinny_cluster_splits(M, N, x.shape[1])
            if splits > 1:
                total = ws.flat(name + "_sum", M * N, torch.float32).view(1, M, N)
                ops.gemm_skinny(total[0], x, w, ops.SKINNY_CLUSTER, splits=splits)
                return ops.Partials(total)
        splits = ops.gemm_skinny_splits(M, N, x.shape[1])
        if splits > 1:
            part = ws.flat(name + "_slices", splits * M * N, torch.float32).view(splits, M, N)
            ops.gemm_skinny(part, x, w, ops.SKINNY_PARTIAL)
            return ops.Partials(part)
    if (M > ops.SKINNY_MAX_ROWS and x.dtype == torch.bfloat16 and _FORCE == "" and _TC_SPLITK and ops.gemm_tc_usable(x, w)):
        # many rows but few columns: too few 128 x 256 tiles for the SMs, so K is cut here too
        splits = ops.gemm_tc_splits(M, N, x.shape[1])
        if splits > 1:
            part = ws.flat(name + "_slices", splits * M * N, torch.float32).view(splits, M, N)
            ops.gemm_tc_sliced(part, x, w)
            return ops.Partials(part)
    return linear(x, w, ws.buffer(name, M, N, out_dtype))


def gated_product_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True when a tensor-core product with the gated epilogue runs for these operands."""
    return (x.dtype == torch.bfloat16 and _FORCE == "" and ops.gemm_tc_usable(x, w) and w.shape[0] % 32 == 0)
