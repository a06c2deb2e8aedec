"""bfloat16 matrix product out[M, N] = a[M, K] @ w[N, K]^T with float32 accumulation.

The reference hands its matrix products to its tensor library's GEMM, and so
does this file for now: the library product (cuBLAS through torch) is the
stand-in until the engine's own tensor-core kernel takes a shape.
"""
from __future__ import annotations

import torch


def gemm_bf16(a, w, out):
    if out.dtype == torch.bfloat16:
        return torch.mm(a, w.t(), out=out)
    # float32 result from bfloat16 operands (the logits)
    return torch.mm(a, w.t(), out_dtype=torch.float32, out=out)
