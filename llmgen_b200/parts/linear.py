"""y = x W^T: the one place that chooses a matrix-product kernel.

    float32 engine   CUDA-core kernel with a fixed summation order (csrc/gemm_simt.cu)
    bfloat16 engine  up to 4 rows: weight-streaming kernel (csrc/gemv.cu);
                     otherwise the tensor-core kernel (csrc/gemm_tc.cu: TMA, tcgen05.mma, tensor
                     memory); operands it refuses (rows not on 16-byte boundaries) go to the
                     CUDA-core kernel.

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

GEMM_MODULES = ("gemm_simt", "gemv", "gemm_tc")


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T; `out` may be float32 for a bfloat16 product."""
    if x.shape[0] == 0:
        return out
    if x.dtype == torch.float32 or _FORCE == "simt":
        ops.gemm_simt(out, x, w)
    elif ops.gemv_usable(x, w):
        ops.gemv_bf16(out, x, w)
    elif _FORCE == "lib" and out.dtype == x.dtype:
        torch.matmul(x, w.t(), out=out)
    elif ops.gemm_tc_usable(x, w):
        ops.gemm_tc(out, x, w)
    else:
        ops.gemm_simt(out, x, w)
    return out


def gated_product_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """True when the tensor-core product with the gated epilogue runs for these operands (the same
    choice `linear` makes for a plain product)."""
    return (x.dtype == torch.bfloat16 and _FORCE == "" and not ops.gemv_usable(x, w)
            and ops.gemm_tc_usable(x, w) and w.shape[0] % 32 == 0)
