"""From a model folder to a plan and its tensors on the device.

config.json picks the architecture through the registry, the architecture's
plan declares the tensors, the loader binds them by name
(crates/model/src/loader/builder.rs:276-330 of the reference walks the same
steps: detect -> config -> weights -> create model)."""
from __future__ import annotations

import torch

from ..config import plan_from_config_json, read_config_json
from ..parts.model import declare_model
from ..weights import load_weights, random_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype):
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


def load_model_dir(model_dir, dtype, device):
    """(typed configuration, plan, {name: device tensor})."""
    dtype = parse_dtype(dtype)
    cfg, plan = plan_from_config_json(read_config_json(model_dir))
    weights = load_weights(model_dir, declare_model(plan), dtype, device)
    return cfg, plan, weights


def random_model(config_json: dict, seed: int, dtype, device, std=None, store_dtype=torch.bfloat16):
    """The model that `write_model_dir(folder, config_json, seed, std, dtype=store_dtype)` would write and
    `load_model_dir(folder, dtype, device)` would read back, made on the device without a folder: every
    element is a function of (seed, tensor name, index) alone (weights/random_init.py), so the tensors
    are equal bit for bit."""
    dtype = parse_dtype(dtype)
    cfg, plan = plan_from_config_json(config_json)
    tensors = random_tensors(declare_model(plan), seed, plan.init_std if std is None else std,
                             plan.norm_init_std, dtype=store_dtype, device=device)
    # what the loader does with a stored tensor: widened for a float32 engine, else kept as stored
    from ..weights.loader import resident_dtype
    return cfg, plan, {k: v.to(resident_dtype(v.dtype, dtype)) for k, v in tensors.items()}
