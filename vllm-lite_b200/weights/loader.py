"""Binds the tensors of a model folder to the names a plan declares.

Files: `model.safetensors`, else the shards an index file names, else every
`model-*.safetensors` in sorted order (crates/model/src/loader/io.rs:51-80 of
the reference).  Names of a vision tower are skipped as the reference does
(crates/model/src/loader/checkpoint.rs:62-64).  Everything else must match the
declaration exactly: one `WeightError` lists every missing tensor, every
unexpected tensor, every wrong shape and every unusable dtype.

Precision: in the bfloat16 mode a tensor stored in 16 bits is kept as bfloat16
and a tensor stored as float32 stays float32; in the float32 mode everything is
widened to float32 (exact).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile

_SKIPPED = ("visual.", "vision_", "img_")
_FLOATS = ("F32", "BF16", "F16")


class WeightError(ValueError):
    def __init__(self, model_dir, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=(), other=()):
        self.missing, self.unexpected = sorted(missing), sorted(unexpected)
        self.wrong_shape, self.wrong_dtype, self.other = list(wrong_shape), list(wrong_dtype), list(other)
        lines = [f"weights under {model_dir} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is {got}, expected one of {', '.join(_FLOATS)}")
        lines.extend(f"  {o}" for o in self.other)
        super().__init__("\n".join(lines))


def find_weight_files(model_dir):
    d = Path(model_dir)
    single = d / "model.safetensors"
    if single.is_file():
        return [single]
    index = d / "model.safetensors.index.json"
    if index.is_file():
        names = sorted(set(json.loads(index.read_text()).get("weight_map", {}).values()))
        return [d / n for n in names]
    shards = sorted(list(d.glob("model-*.safetensors")) + list(d.glob("model.safetensors-*")))
    if not shards:
        raise WeightError(model_dir, other=[f"no model.safetensors (or shards of it) in {d}"])
    return shards


def load_weights(model_dir, declared: dict, dtype: torch.dtype, device) -> dict:
    """{name: device tensor} for every declared tensor; raises WeightError otherwise."""
    files, where, other = [], {}, []
    for path in find_weight_files(model_dir):
        try:
            f = SafetensorsFile(path)
        except (OSError, SafetensorsError) as e:
            raise WeightError(model_dir, other=[str(e)]) from e
        files.append(f)
        for name in f.names():
            if any(s in name for s in _SKIPPED):
                continue
            if name in where:
                other.append(f"duplicate tensor {name} in {where[name].path.name} and {f.path.name}")
            where[name] = f
    missing = [n for n in declared if n not in where]
    unexpected = [n for n in where if n not in declared]
    wrong_shape, wrong_dtype = [], []
    for name, decl in declared.items():
        if name not in where:
            continue
        st_dtype, shape = where[name].info(name)
        if tuple(shape) != tuple(decl.shape):
            wrong_shape.append((name, shape, decl.shape))
        if st_dtype not in _FLOATS:
            wrong_dtype.append((name, st_dtype))
    if missing or unexpected or wrong_shape or wrong_dtype or other:
        for f in files:
            f.close()
        raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype, other)
    out = {}
    try:
        for name in declared:
            t = where[name].read(name)
            out[name] = t.to(device=device, dtype=resident_dtype(t.dtype, dtype)).contiguous()
    except SafetensorsError as e:
        raise WeightError(model_dir, other=[str(e)]) from e
    finally:
        for f in files:
            f.close()
    return out


def resident_dtype(stored: torch.dtype, model_dtype: torch.dtype) -> torch.dtype:
    if model_dtype == torch.float32 or stored == torch.float32:
        return torch.float32
    return torch.bfloat16
