"""bfloat16 matrix product out[M, N] = a[M, K] @ w[N, K]^T with float32 accumulation.

Few rows (a decode step) go to the engine's weight-streaming kernel, many rows (a prompt
portion of two thousand tokens or more; a thousand for the product that applies SwiGLU itself) to its tcgen05
kernels (one SM or a pair of SMs per tile).  What lies between goes to the library product (cuBLAS through torch), as the reference hands its matrix products to
its tensor library's GEMM.
"""
from __future__ import annotations

import torch

# The library product must add in float32 whatever the shape: with this switch left on (torch's default)
# cuBLAS may pick kernels that cut K among blocks and add the pieces in bfloat16, and a row's result
# could then depend on how many rows share its step.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


def fuses_swiglu(M, K) -> bool:
    """Whether the product for M rows runs in a kernel that can apply SwiGLU to its own tile."""
    from ..csrc import ops
    return ops.gemm_bf16_small_m_ok(M, K) or ops.gemm_bf16_tc5_ok(M, K, fused=True)


def gemm_bf16(a, w, out, err=None, swiglu=False):
    """swiglu (only where `fuses_swiglu`): w interleaves 8 gate rows with their 8 up rows and out is
    [M, N/2] = silu(gate) * up."""
    from ..csrc import ops
    M, K = a.shape
    if ops.gemm_bf16_small_m_ok(M, K):
        return ops.gemm_bf16_small_m(a, w, out, err, swiglu)
    if ops.gemm_bf16_tc5_ok(M, K, fused=swiglu):
        # Two SMs on a 256 x 256 tile halve the rows of w each SM copies; measured faster (3 to 7 %) when
        # there are tiles for every pair of SMs or K is long, slower (2 to 6 %) for the short, narrow products.
        N = w.shape[0]
        if -(-M // 256) * -(-N // 256) >= ops.sm_pairs() or K >= 8192:
            return ops.gemm_bf16_tc5_pair(a, w, out, err, swiglu)
        return ops.gemm_bf16_tc5(a, w, out, err, swiglu)
    if swiglu:
        raise ValueError("the library product has no fused activation; ask fuses_swiglu() first")
    if out.dtype == torch.bfloat16:
        return torch.mm(a, w.t(), out=out)
    return torch.mm(a, w.t(), out_dtype=torch.float32, out=out)      # float32 logits from bfloat16 operands
