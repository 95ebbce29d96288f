"""y = x W^T: the one place that chooses a matrix-product kernel.

    float32 engine   CUDA-core kernel with a fixed summation order (csrc/gemm_simt.cu)
    bfloat16 engine  up to 4 rows, products that leave slices (qkv, o_proj, down_proj of a decode step): W straight
                     from global memory into `mma.sync`, all of it asked for before the wait for the kernel that
                     makes x (csrc/gemm_rows8.cu);
                     up to 64 rows: the weight-streaming tensor-core kernel with swapped operands
                     (csrc/gemm_skinny.cu), cut along K so that every SM streams a share of W; more rows: the
                     tiled tensor-core kernel (csrc/gemm_tc.cu: TMA, tcgen05.mma, tensor memory), cut along K
                     too while its tiles are too few for the SMs (a few hundred rows).  Either way the float32
                     slices of a cut product come back as an `ops.Partials`, which the consuming kernel adds up.
                     Operands TMA refuses (rows not on 16-byte boundaries): the CUDA-core weight-streaming kernel
                     for up to 4 rows (csrc/gemv.cu), else the CUDA-core product.

The reference uses its own GEMV for M <= 2 and `cublasGemmEx` above
(src/backend/cuda/linear/linear.cu:53-96).

Weight layout [out, in] row-major, no bias (src/module/linear.zig:48-82).
"""
from __future__ import annotations

import torch

from ..kernels import ops

GEMM_MODULES = ("gemm_simt", "gemv", "gemm_tc", "gemm_skinny", "gemm_rows8")


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T; `out` may be float32 for a bfloat16 product."""
    if x.shape[0] == 0:
        return out
    if x.dtype == torch.float32:
        ops.gemm_simt(out, x, w)
    elif x.shape[0] <= ops.SKINNY_BEST_ROWS and ops.gemm_skinny_usable(x, w):
        ops.gemm_skinny(out, x, w)
    elif ops.gemv_usable(x, w):
        ops.gemv_bf16(out, x, w)
    elif ops.gemm_tc_usable(x, w):
        ops.gemm_tc(out, x, w)
    else:
        ops.gemm_simt(out, x, w)
    return out


def linear_sliced(ws, name: str, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype):
    """x W^T into the workspace buffer `name`: the finished [M, N] array, or, when the product is cut
    along K, an `ops.Partials` for a consumer that adds the slices."""
    M, N, K = x.shape[0], w.shape[0], x.shape[1]
    if 0 < M <= ops.ROWS8_BEST_ROWS and ops.gemm_rows8_usable(x, w):
        # a few rows: W straight from global memory into mma.sync, the fewest dependent steps (csrc/gemm_rows8.cu)
        slices = ops.gemm_rows8_slices(N, K)
        part = ws.flat(name + "_slices", slices * M * N, torch.float32).view(slices, M, N)
        ops.gemm_rows8(part, x, w)
        return ops.Partials(part)
    if M > 0 and x.dtype == torch.bfloat16 and ops.gemm_tc_usable(x, w):
        few = M <= ops.SKINNY_BEST_ROWS
        splits = ops.gemm_skinny_splits(M, N, K) if few else ops.gemm_tc_splits(M, N, K)
        if splits > 1:
            part = ws.flat(name + "_slices", splits * M * N, torch.float32).view(splits, M, N)
            if few:
                ops.gemm_skinny(part, x, w, ops.SKINNY_PARTIAL)
            else:
                ops.gemm_tc_sliced(part, x, w)
            return ops.Partials(part)
    return linear(x, w, ws.buffer(name, M, N, out_dtype))


def gated_product_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True when a tensor-core product with the gated epilogue runs for these operands."""
    return x.dtype == torch.bfloat16 and ops.gemm_tc_usable(x, w) and w.shape[0] % 32 == 0
