"""y = x W^T: the one place that chooses a matrix-product kernel.

    float32 engine   CUDA-core kernel with a fixed summation order (csrc/gemm_simt.cu)
    bfloat16 engine  up to 4 rows: weight-streaming kernel (csrc/gemv.cu);
                     otherwise the library product (cuBLAS through torch.matmul), as in the
                     reference, which uses its own GEMV for M <= 2 and `cublasGemmEx` above
                     (src/backend/cuda/linear/linear.cu:53-96); shapes the library path cannot
                     take in place go to the CUDA-core kernel.

Weight layout [out, in] row-major, no bias (src/module/linear.zig:48-82).
"""
from __future__ import annotations

import os

import torch

from ..kernels import ops

# "simt" forces the hand-written CUDA-core product everywhere (no library call).
_FORCE = os.environ.get("LLMGEN_GEMM", "")


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T; `out` may be float32 for a bfloat16 product."""
    if x.shape[0] == 0:
        return out
    if x.dtype == torch.float32:
        ops.gemm_simt(out, x, w)
    elif ops.gemv_usable(x, w):
        ops.gemv_bf16(out, x, w)
    elif _FORCE == "simt" or out.dtype != x.dtype:
        ops.gemm_simt(out, x, w)
    else:
        torch.matmul(x, w.t(), out=out)
    return out
