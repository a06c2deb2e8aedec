"""Rotary position encoding: the table of inverse frequencies.

inv_freq[i] = theta^(-2i / rotary_dim) in float32
(crates/model/src/components/positional/rope.rs:498-503 of the reference).  The
rotation itself runs inside the kernel that also norms the heads and writes the
cache; this part owns the constants and hands them over through `fused_rotary`.
"""
from __future__ import annotations

import numpy as np
import torch

from .registry import POSITIONS
from .spec import RotarySpec


def inverse_frequencies(rotary_dim: int, theta: float) -> np.ndarray:
    i = np.arange(rotary_dim // 2, dtype=np.float32)
    exponent = (np.float32(-2.0) * i / np.float32(rotary_dim)).astype(np.float32)
    return np.power(np.float32(theta), exponent).astype(np.float32)


@POSITIONS.register("rotary")
class RotaryTable:
    @staticmethod
    def declare(spec: RotarySpec) -> dict:
        return {}

    def __init__(self, spec: RotarySpec, weights: dict, ctx):
        if spec.dim % 2 or spec.dim > spec.head_dim or spec.dim <= 0:
            raise ValueError(f"rotary_dim {spec.dim} must be even and at most head_dim {spec.head_dim}")
        self.spec = spec
        self.inv_freq = torch.from_numpy(inverse_frequencies(spec.dim, spec.theta)).to(ctx.device)

    def fused_rotary(self):
        return self.inv_freq, self.spec.dim
