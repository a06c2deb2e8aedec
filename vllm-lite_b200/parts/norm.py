"""RMS norm: h = x / sqrt(mean(x^2) + eps) * w, in float32, with the pending
residual added into the stream by the same kernel
(crates/model/src/components/norm/rms_norm.rs:26-49 of the reference)."""
from __future__ import annotations

import torch

from .registry import NORMS
from .spec import NormSpec, TensorDecl


@NORMS.register("rms_norm")
class RmsNorm:
    factorable = True          # h = (x * weight) * scale(x): neighbours may fuse it (parts/base.py, ScaledRows)

    @staticmethod
    def declare(spec: NormSpec) -> dict:
        return {"weight": TensorDecl((spec.size,), init="norm")}

    def __init__(self, spec: NormSpec, weights: dict, ctx):
        self.spec = spec
        self.dtype = ctx.dtype
        # A vector of `size` numbers: kept as float32 on the device (exact from bfloat16).
        self.weight = weights["weight"].to(device=ctx.device, dtype=torch.float32).contiguous()

    def fused_rms(self):
        """(weight, eps): what a kernel that applies this norm itself needs (the attention mixer's
        kernel norms every head while it rotates it)."""
        return self.weight, self.spec.eps

    def __call__(self, x, delta, step, rows=None, tag="norm"):
        from ..csrc import ops
        R = x.shape[0] if rows is None else rows.shape[0]
        out = step.workspace.get(step.tag + tag, (R, self.spec.size), self.dtype)
        return ops.add_rmsnorm(x, delta, self.weight, self.spec.eps, out, rows=rows)
