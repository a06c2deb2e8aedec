"""Random weights from a plan's declarations and a seed.

Linear, embedding and head matrices are N(0, std); norm weights are
1 + N(0, norm_std).  Every element is a function of (seed, tensor name, element
index) alone: a 64-bit counter hash picks a point of the normal distribution's
inverse CDF from a table.  Only integer arithmetic and single, correctly rounded
float32 operations are used, so the same seed gives the same bits on the CPU and
on the GPU, whatever else is generated and in whatever order: `random_model`
(made on the device, no file) and a folder written by `write_model_dir` and read
back hold equal tensors.  `write_model_dir` makes a folder that the loader reads
like any checkpoint: config.json and model.safetensors, stored in bfloat16 unless
asked otherwise.

The reference has no random-weights mode (its `Qwen3Model::new` is all zeros,
crates/model/src/qwen3/model/construct.rs:44-58).
"""
from __future__ import annotations

import functools
import json
from pathlib import Path
from statistics import NormalDist

import torch

from ..parts.model import declare_model
from .safetensors_io import write_safetensors

_MASK64 = (1 << 64) - 1
_GOLDEN, _MIX1, _MIX2 = 0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
TABLE_BITS = 16                   # the inverse CDF is tabulated at 2^16 + 1 points, linear in between
FRACTION_BITS = 24                # bits that place an element between two points (exact in float32)
CHUNK = 1 << 24                   # elements made at a time (bounds the temporaries: a few hundred MB)


def _signed(v: int) -> int:
    """A 64-bit pattern as the int64 that holds it."""
    v &= _MASK64
    return v - (1 << 64) if v >> 63 else v


def _mix_python(z: int) -> int:
    z &= _MASK64
    z = ((z ^ (z >> 30)) * _MIX1) & _MASK64
    z = ((z ^ (z >> 27)) * _MIX2) & _MASK64
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """64 bits from the seed and the tensor's name (FNV-1a of the name, mixed with the seed)."""
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _MASK64
    return _mix_python(h ^ _mix_python(int(seed) & _MASK64))


@functools.lru_cache(maxsize=None)
def _inverse_cdf_table():
    """(points float32 [2^16 + 1], differences float32 [2^16]): the standard normal's inverse CDF at
    i / 2^16, its two ends taken a quarter step inside (about +-4.5), by the standard library's rational
    approximation in double precision, rounded once."""
    n = 1 << TABLE_BITS
    nd = NormalDist()
    q = [nd.inv_cdf(min(max(i, 0.25), n - 0.25) / n) for i in range(n + 1)]
    points = torch.tensor(q, dtype=torch.float64).to(torch.float32)
    return points, (points[1:] - points[:-1]).contiguous()


def _shift_right(z: torch.Tensor, s: int) -> torch.Tensor:
    """Logical right shift of 64-bit patterns held in int64."""
    return (z >> s) & ((1 << (64 - s)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _shift_right(z, 30)) * _signed(_MIX1)
    z = (z ^ _shift_right(z, 27)) * _signed(_MIX2)
    return z ^ _shift_right(z, 31)


def standard_normal(seed: int, name: str, numel: int, device="cpu") -> torch.Tensor:
    """float32 [numel]: element i depends on (seed, name, i) only."""
    device = torch.device(device)
    points, diffs = (t.to(device) for t in _inverse_cdf_table())
    key = tensor_key(seed, name)
    out = torch.empty(numel, dtype=torch.float32, device=device)
    for lo in range(0, numel, CHUNK):
        hi = min(numel, lo + CHUNK)
        idx = torch.arange(lo + 1, hi + 1, dtype=torch.int64, device=device)
        z = _mix(idx * _signed(_GOLDEN) + _signed(key))            # int64 arithmetic wraps: mod 2^64
        cell = _shift_right(z, 64 - TABLE_BITS)
        frac = (_shift_right(z, 64 - TABLE_BITS - FRACTION_BITS) & ((1 << FRACTION_BITS) - 1)).to(torch.float32)
        frac = frac * (2.0 ** -FRACTION_BITS)                      # exact
        step = diffs[cell] * frac                                  # one rounding
        out[lo:hi] = points[cell] + step                           # one rounding
    return out


def random_tensors(declared: dict, seed: int, std: float = 0.02, norm_std: float = 0.1,
                   dtype=torch.bfloat16, device="cpu") -> dict:
    out = {}
    for name in sorted(declared):
        decl = declared[name]
        n = 1
        for s in decl.shape:
            n *= int(s)
        t = standard_normal(seed, name, n, device).view(decl.shape)
        if decl.init == "norm":
            t = t.mul_(norm_std).add_(1.0)
        elif decl.init == "linear":
            t = t.mul_(std)
        else:
            raise ValueError(f"unknown init {decl.init!r} for {name}")
        out[name] = t.to(torch.float32 if decl.store == "float32" else dtype)
    return out


def write_model_dir(model_dir, config, seed: int, std=None, norm_std=None, dtype=torch.bfloat16):
    """`config`: a typed configuration (with `to_dict`) or a config.json dict."""
    from ..config import plan_from_config_json
    cfg_json = config.to_dict() if hasattr(config, "to_dict") else dict(config)
    _, plan = plan_from_config_json(cfg_json)
    tensors = random_tensors(declare_model(plan), seed,
                             plan.init_std if std is None else std,
                             plan.norm_init_std if norm_std is None else norm_std, dtype=dtype)
    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    (d / "config.json").write_text(json.dumps(cfg_json, indent=2) + "\n")
    write_safetensors(d / "model.safetensors", tensors, metadata={"format": "pt", "seed": seed})
    return d
