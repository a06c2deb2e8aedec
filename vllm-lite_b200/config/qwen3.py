"""Typed configuration of the Qwen3 dense decoder, read from config.json keys.

Keys and alternates follow the reference's reader
(crates/model/src/config/model_config.rs:251-325): `num_key_value_heads`
(alt `num_local_heads`) defaults to the number of query heads, `head_dim`
defaults to hidden_size / heads and need not multiply back to the hidden size,
`rope_theta` (alt `rotary_base`), `rms_norm_eps` (alt `layer_norm_eps`),
`tie_word_embeddings` (default false).  Unlike the reference, sizes have no
defaults: a missing size is an error.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Optional

from .errors import ConfigError, InvalidField, MissingField

ARCHITECTURE = "Qwen3ForCausalLM"


def _get(d, names, default=None, required=False):
    for n in names:
        if n in d and d[n] is not None:
            return d[n]
    if required:
        raise MissingField(names[0])
    return default


def _pos_int(d, names, default=None, required=True):
    v = _get(d, names, default, required and default is None)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise InvalidField(names[0], f"expected a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float
    rms_norm_eps: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    # eps of the per-head q/k norm.  The architecture uses its rms_norm_eps; the
    # reference hard-codes 1e-6 (crates/model/src/components/attention/gqa/mod.rs:77,82)
    # and the non-standard key `qk_norm_eps` selects another value.
    qk_norm_eps: Optional[float] = None
    architecture: str = ARCHITECTURE

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def head_norm_eps(self) -> float:
        return self.rms_norm_eps if self.qk_norm_eps is None else self.qk_norm_eps

    def validate(self) -> "Qwen3Config":
        if self.num_attention_heads % self.num_key_value_heads:
            raise InvalidField("num_key_value_heads",
                               f"{self.num_key_value_heads} does not divide num_attention_heads={self.num_attention_heads}")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise InvalidField("head_dim", f"{self.head_dim}: the attention kernels take multiples of 16 from 16 to 256 "
                                           f"(the rotation pairs x[i] with x[i + head_dim/2])")
        if not (self.rms_norm_eps > 0):
            raise InvalidField("rms_norm_eps", f"must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise InvalidField("rope_theta", f"must be positive, got {self.rope_theta}")
        return self

    # ---- config.json ----------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        if not isinstance(d, dict):
            raise ConfigError("config.json must hold a JSON object")
        heads = _pos_int(d, ["num_attention_heads"])
        hidden = _pos_int(d, ["hidden_size"])
        eps = _get(d, ["rms_norm_eps", "layer_norm_eps"], required=True)
        theta = _get(d, ["rope_theta", "rotary_base"], 10000.0)
        for key, val in (("rms_norm_eps", eps), ("rope_theta", theta)):
            if isinstance(val, bool) or not isinstance(val, (int, float)):
                raise InvalidField(key, f"expected a number, got {val!r}")
        if d.get("attention_bias"):
            raise InvalidField("attention_bias", "projections with bias are not part of this architecture's engine")
        if d.get("hidden_act", "silu") != "silu":
            raise InvalidField("hidden_act", f"only 'silu' is built, got {d['hidden_act']!r}")
        if d.get("rope_scaling") is not None:
            raise InvalidField("rope_scaling", "scaled rotary frequencies are not built; remove the key or set it to null")
        if d.get("use_sliding_window"):
            # The reference parses sliding_window and drops it for this
            # architecture (crates/model/src/config/hyperparams.rs:153).
            raise InvalidField("use_sliding_window", "the Qwen3 dense path has no windowed layers")
        qk_eps = d.get("qk_norm_eps")
        cfg = cls(
            vocab_size=_pos_int(d, ["vocab_size"]),
            hidden_size=hidden,
            num_hidden_layers=_pos_int(d, ["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=_pos_int(d, ["num_key_value_heads", "num_local_heads"], default=heads),
            head_dim=_pos_int(d, ["head_dim"], default=max(hidden // heads, 1)),
            intermediate_size=_pos_int(d, ["intermediate_size"]),
            rope_theta=float(theta),
            rms_norm_eps=float(eps),
            max_position_embeddings=_pos_int(d, ["max_position_embeddings"]),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            qk_norm_eps=None if qk_eps is None else float(qk_eps),
        )
        return cfg.validate()

    def to_dict(self) -> dict:
        d = asdict(self)
        arch = d.pop("architecture")
        if d["qk_norm_eps"] is None:
            d.pop("qk_norm_eps")
        out = {"architectures": [arch], "model_type": "qwen3", "hidden_act": "silu",
               "attention_bias": False, "torch_dtype": "bfloat16"}
        out.update(d)
        return out


def read_config_json(model_dir) -> dict:
    path = Path(model_dir) / "config.json"
    try:
        text = path.read_text()
    except OSError as e:
        raise ConfigError(f"io error reading {path}: {e}") from e
    try:
        return json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"json parse error in {path}: {e}") from e
