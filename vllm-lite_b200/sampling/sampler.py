"""Draws one token per logits row on the device.

Rows that are all greedy need no upload at all.  Otherwise the options of all rows
(temperature, top-p, the uniform number of the draw; top-k) go up as two small arrays;
penalties and biases go as ragged lists (each distinct generated id once,
as the reference's set does, crates/core/src/sampling.rs:670-688); the kernels of
csrc/sampling.cu do the rest and only the chosen ids come back to the host."""
from __future__ import annotations

import random
from typing import Optional, Sequence

import numpy as np
import torch

from .params import SamplingParams, seeded_uniform


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._rng = random.Random()
        self._tokens = None
        self._logprobs = None

    def _buffers(self, rows):
        if self._tokens is None or self._tokens.numel() < rows:
            n = max(rows, 64)
            self._tokens = torch.empty(n, dtype=torch.int32, device=self.device)
            self._logprobs = torch.empty(n, dtype=torch.float32, device=self.device)
        return self._tokens[:rows], self._logprobs[:rows]

    def uniform_for(self, params: SamplingParams, step: int) -> float:
        if params.seed is None:
            return self._rng.random()
        return seeded_uniform(params.seed, step)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], generated: Sequence[Sequence[int]],
               want_logprobs: bool = False, steps: Optional[Sequence[int]] = None):
        """logits float32 [R, V] (modified in place when penalties apply); `generated[r]`
        are the tokens row r's request has produced so far (their count is the step of
        its random stream, unless `steps` gives the counts).  Returns (tokens int32 [R] on the
        device, logprobs or None); both are views of buffers that the next call writes again."""
        from ..csrc import ops
        R = logits.shape[0]
        out_tok, out_lp = self._buffers(R)
        if all(p.temperature <= 0 and not p.needs_penalties for p in params):
            ops.sample(logits, None, None, None, None, out_tok, out_lp if want_logprobs else None)
            return out_tok, (out_lp if want_logprobs else None)
        if any(p.needs_penalties for p in params):
            self._penalties(logits, params, generated)
        f = np.zeros((3, R), dtype=np.float32)
        k = np.zeros(R, dtype=np.int32)
        for r, p in enumerate(params):
            f[0, r], f[1, r] = p.temperature, p.top_p
            f[2, r] = self.uniform_for(p, steps[r] if steps is not None else len(generated[r])) if p.temperature > 0 else 0.0
            k[r] = p.top_k
        fd = torch.from_numpy(f).to(self.device, non_blocking=True)
        kd = torch.from_numpy(k).to(self.device, non_blocking=True)
        ops.sample(logits, fd[0], kd, fd[1], fd[2], out_tok, out_lp if want_logprobs else None)
        return out_tok, (out_lp if want_logprobs else None)

    def _penalties(self, logits, params, generated):
        from ..csrc import ops
        R = logits.shape[0]
        seen_off, seen_ids = [0], []
        bias_off, bias_ids, bias_vals = [0], [], []
        rep = np.ones(R, dtype=np.float32)
        pres = np.zeros(R, dtype=np.float32)
        for r, p in enumerate(params):
            if p.repeat_penalty != 1.0 or p.presence_penalty != 0.0:
                rep[r], pres[r] = p.repeat_penalty, p.presence_penalty
                seen_ids.extend(sorted(set(int(t) for t in generated[r])))
            seen_off.append(len(seen_ids))
            if p.logit_bias:
                for t, b in p.logit_bias.items():
                    bias_ids.append(int(t))
                    bias_vals.append(float(b))
            bias_off.append(len(bias_ids))
        dev = self.device
        i32 = lambda a: torch.tensor(a if len(a) else [0], dtype=torch.int32, device=dev)
        ops.apply_penalties(
            logits, i32(seen_off), i32(seen_ids), torch.from_numpy(rep).to(dev), torch.from_numpy(pres).to(dev),
            i32(bias_off), i32(bias_ids),
            torch.tensor(bias_vals if bias_vals else [0.0], dtype=torch.float32, device=dev))
