"""Random weights from a plan's declarations and a seed.

Linear, embedding and head matrices are N(0, std); norm weights are
1 + N(0, norm_std).  Tensors are drawn in the order of their names from one
generator, so (plan, seed, std) fixes every value.  `write_model_dir` makes a
folder that the loader reads like any checkpoint: config.json and
model.safetensors, stored in bfloat16 unless asked otherwise.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..parts.model import declare_model
from .safetensors_io import write_safetensors


def random_tensors(declared: dict, seed: int, std: float = 0.02, norm_std: float = 0.1,
                   dtype=torch.bfloat16, device="cpu") -> dict:
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for name in sorted(declared):
        decl = declared[name]
        t = torch.randn(decl.shape, generator=gen, device=device, dtype=torch.float32)
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
