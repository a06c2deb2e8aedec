"""Per-request sampling options, with the reference's names, meanings and defaults
(crates/traits/src/sampling.rs:83-257).  The reference's `beam_width`,
`length_penalty`, `max_retries` and `top_logprobs` are declared there but are not
part of what its sampler draws with, and have no counterpart here."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional


@dataclass
class SamplingParams:
    temperature: float = 0.0            # 0 selects greedy argmax
    top_k: int = 0                      # 0 disables
    top_p: float = 1.0                  # 1 disables
    repeat_penalty: float = 1.0         # 1 disables; once per distinct generated token
    presence_penalty: float = 0.0       # 0 disables; once per distinct generated token
    logit_bias: Optional[Dict[int, float]] = None
    seed: Optional[int] = None          # per-request stream, indexed by the step
    stop_token_sequences: Optional[List[List[int]]] = None

    def validate(self) -> "SamplingParams":
        if self.temperature < 0 or self.temperature != self.temperature:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must lie in (0, 1], got {self.top_p}")
        if self.repeat_penalty <= 0:
            raise ValueError(f"repeat_penalty must be positive, got {self.repeat_penalty}")
        return self

    @property
    def needs_penalties(self) -> bool:
        return self.repeat_penalty != 1.0 or self.presence_penalty != 0.0 or bool(self.logit_bias)


_MASK = (1 << 64) - 1


def splitmix64(x: int) -> int:
    """The fixed bijection that the reference mixes the step index with
    (crates/core/src/sampling.rs:38-43)."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def seeded_uniform(seed: int, step: int) -> float:
    """One number in [0, 1) for (seed, step): same pair, same draw; other step, other
    draw.  The reference seeds a generator of its runtime with seed ^ splitmix64(step)
    (crates/core/src/sampling.rs:63-70); this engine takes 24 bits of one more
    splitmix64 round of that word, so streams are reproducible here but are not the
    reference's numbers."""
    word = splitmix64((int(seed) & _MASK) ^ splitmix64(int(step) & _MASK))
    return (word >> 40) / float(1 << 24)
