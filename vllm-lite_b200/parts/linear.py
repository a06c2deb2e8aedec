"""y = x W^T (+ b) with the weight stored [out, in]; the model of this engine has no bias
(crates/model/src/components/attention/gqa/norm.rs:21-26 of the reference), a part that
has one passes `bias` and gives up the fusions with its neighbouring norms.

The product runs in the precision of the stored weight: a bfloat16 weight on
the tensor cores with float32 accumulation, a float32 weight through the true
float32 kernel (activations are widened for it and the result narrowed back).
"""
from __future__ import annotations

import torch

from .base import ScaledRows, StreamSink


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor = None):
        if weight.dim() != 2 or not weight.is_contiguous():
            raise ValueError("a linear weight is a contiguous [out, in] matrix")
        self.weight = weight
        self.out_features, self.in_features = weight.shape
        # a vector of out_features numbers: kept as float32 (exact from bfloat16) and added in float32
        self.bias = None if bias is None else bias.to(device=weight.device, dtype=torch.float32).contiguous()
        if self.bias is not None and tuple(self.bias.shape) != (self.out_features,):
            raise ValueError(f"a linear bias has out_features={self.out_features} entries, got {tuple(bias.shape)}")

    def factors_norms(self, M) -> bool:
        """Whether, for M rows, this layer's kernel can take an RMS norm's output in factored form
        (`ScaledRows`) and can add its result into the stream (`into_stream`)."""
        from ..csrc import ops
        return (self.bias is None and self.weight.dtype == torch.bfloat16
                and ops.gemm_bf16_small_m_ok(M, self.in_features))

    def into_stream(self, a, sink: StreamSink, step, tag) -> ScaledRows:
        """sink.x += a W^T; returns the next norm's output on the new stream, in factored form."""
        from ..csrc import ops
        M = a.shape[0]
        ws = step.workspace
        rows = ws.get(step.tag + tag + ".rows", (M, self.out_features), torch.bfloat16)
        partial = ws.get(step.tag + tag + ".ss", (ops.NORM_PARTIALS, 16), torch.float32)
        count = ops.gemm_bf16_small_m(a, self.weight, rows, step.err, sink=(sink.x, sink.weight, partial))
        return ScaledRows(rows, partial, count, sink.eps, sink.size)

    def swiglu(self, a, step, tag, group):
        """silu(gate) * up of y = a W^T, W holding gate and up rows (interleaved in blocks of `group`
        rows, or gate rows then up rows when group is 0): [M, out_features / 2].  The activation runs
        inside the product kernel when that kernel can, else in a kernel of its own."""
        from ..csrc import ops
        from . import matmul
        if self.bias is not None and group:
            raise ValueError("the fused gate/up layout has no bias; stack gate and up as plain halves (group 0)")
        if isinstance(a, ScaledRows):
            M = a.rows.shape[0]
            if group != ops.SWIGLU_GROUP or not self.factors_norms(M):
                raise TypeError("this layer cannot take a norm's output in factored form")
            out = step.workspace.get(step.tag + tag + ".act", (M, self.out_features // 2), a.rows.dtype)
            return ops.gemm_bf16_small_m(a.rows, self.weight, out, step.err, swiglu=True,
                                         scaled=(a.partial, a.count, a.eps, a.size))
        M = a.shape[0]
        ws = step.workspace
        out = ws.get(step.tag + tag + ".act", (M, self.out_features // 2), a.dtype)
        if (group == ops.SWIGLU_GROUP and self.bias is None and self.weight.dtype == torch.bfloat16
                and a.dtype == torch.bfloat16 and matmul.fuses_swiglu(M, self.in_features)):
            return matmul.gemm_bf16(a, self.weight, out, step.err, swiglu=True)
        return ops.silu_mul(self(a, step, tag), out, group)

    def __call__(self, a, step, tag, out_dtype=None):
        y = self._product(a, step, tag, out_dtype)
        if self.bias is not None:
            from ..csrc import ops
            ops.add_bias(y, self.bias)
        return y

    def _product(self, a, step, tag, out_dtype=None):
        from ..csrc import ops
        from . import matmul
        if isinstance(a, ScaledRows):
            M = a.rows.shape[0]
            if not self.factors_norms(M):
                raise TypeError("this layer cannot take a norm's output in factored form")
            out = step.workspace.get(step.tag + tag, (M, self.out_features), out_dtype or a.rows.dtype)
            return ops.gemm_bf16_small_m(a.rows, self.weight, out, step.err, scaled=(a.partial, a.count, a.eps, a.size))
        out_dtype = out_dtype or a.dtype
        M = a.shape[0]
        ws = step.workspace
        if self.weight.dtype == torch.float32:
            if a.dtype != torch.float32:
                a = ops.cast(a, ws.get(step.tag + tag + ".a32", a.shape, torch.float32))
            if out_dtype == torch.float32:
                return ops.gemm_f32(a, self.weight, ws.get(step.tag + tag, (M, self.out_features), torch.float32))
            y = ops.gemm_f32(a, self.weight, ws.get(step.tag + tag + ".y32", (M, self.out_features), torch.float32))
            return ops.cast(y, ws.get(step.tag + tag, (M, self.out_features), out_dtype))
        if a.dtype != self.weight.dtype:
            raise TypeError(f"activation {a.dtype} does not match weight {self.weight.dtype}")
        out = ws.get(step.tag + tag, (M, self.out_features), out_dtype)
        return matmul.gemm_bf16(a, self.weight, out, step.err)
