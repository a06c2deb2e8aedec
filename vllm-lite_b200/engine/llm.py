"""The Python entry point: requests in, tokens out.

`LLMEngine.add_request` and `LLMEngine.step` mirror the reference's in-process API
(`Engine::add_request`, crates/core/src/engine/lifecycle.rs:174-200, and
`Engine::step`, crates/core/src/scheduler/batch.rs:275-297): a request is a list of
prompt token ids, a cap on generated tokens and sampling options; a step schedules
one batch, runs it, samples, and reports the new token of every request that
reached its end.  `generate` runs requests to completion.  Token ids are host
integers on both sides; the engine has no tokenizer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence as Seq

import torch

from ..cache.manager import OutOfPages
from ..sampling import Sampler, SamplingParams
from .loading import load_model_dir, parse_dtype
from .runner import ModelRunner, StepEntry
from .scheduler import Scheduler, SchedulerConfig, Sequence


@dataclass
class StepOutput:
    seq_id: int
    token: int
    finished: bool
    finish_reason: Optional[str] = None
    logprob: Optional[float] = None


class LLMEngine:
    def __init__(self, model=None, *, dtype="bfloat16", device="cuda:0", kv_blocks: int = 1024, block_size: int = 16,
                 max_batch_size: int = 256, max_num_batched_tokens: int = 4096, prefill_chunk_size: int = 512,
                 max_model_len: Optional[int] = None, plan=None, weights=None, logprobs: bool = False):
        """`model`: a folder with config.json and safetensors (never downloaded).  `kv_blocks`
        and `max_batch_size` carry the reference's names and defaults
        (crates/server/src/cli/args.rs:155-186); `block_size` is its BLOCK_SIZE constant
        (crates/traits/src/types.rs:13) made an option.  Alternatively pass `plan` and
        `weights` of a model that is already on the device."""
        self.dtype = parse_dtype(dtype)
        if plan is None:
            if model is None:
                raise ValueError("give a model folder (or plan and weights)")
            _, plan, weights = load_model_dir(model, self.dtype, device)
        if max_model_len is None:
            max_model_len = plan.max_position_embeddings
        self.runner = ModelRunner(plan, weights, dtype=self.dtype, device=device, page_size=block_size,
                                  num_pages=kv_blocks, max_requests=max_batch_size, max_context=max_model_len)
        self.scheduler = Scheduler(self.runner.cache, SchedulerConfig(
            max_num_seqs=max_batch_size, max_num_batched_tokens=max_num_batched_tokens,
            prefill_chunk_size=prefill_chunk_size, max_model_len=max_model_len))
        self.sampler = Sampler(device)
        self.want_logprobs = logprobs
        self.sequences: Dict[int, Sequence] = {}

    # ---- requests -----------------------------------------------------------
    def add_request(self, prompt: Seq[int], max_tokens: int, sampling_params: SamplingParams = None) -> int:
        vocab = self.runner.plan.vocab_size
        for t in prompt:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token id {t} lies outside the vocabulary of {vocab}")
        seq = self.scheduler.add_request(prompt, max_tokens, sampling_params)
        self.sequences[seq.seq_id] = seq
        return seq.seq_id

    def cancel_request(self, seq_id: int) -> bool:
        return self.scheduler.cancel(seq_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    # ---- one step -------------------------------------------------------------
    def step(self) -> List[StepOutput]:
        plan = self.scheduler.schedule()
        if not plan.entries:
            return []
        entries = [StepEntry(e.seq.seq_id, e.seq.tokens[e.start:e.start + e.count],
                             [e.count - 1] if e.samples else []) for e in plan.entries]
        logits = self.runner.step(entries)
        sampling = [e for e in plan.entries if e.samples]
        sampled: List[Optional[int]] = [None] * len(plan.entries)
        logprobs = None
        if sampling:
            tok, lp = self.sampler.sample(logits, [e.seq.params for e in sampling],
                                          [e.seq.generated for e in sampling], self.want_logprobs)
            host = tok.cpu().tolist()                         # the step's only read-back
            logprobs = lp.cpu().tolist() if lp is not None else None
            it = iter(host)
            sampled = [next(it) if e.samples else None for e in plan.entries]
        finished = self.scheduler.update(plan, sampled)
        out, k = [], 0
        for e, t in zip(plan.entries, sampled):
            if t is None:
                continue
            out.append(StepOutput(e.seq.seq_id, t, e.seq.status == "finished", e.seq.finish_reason,
                                  logprobs[k] if logprobs else None))
            k += 1
        return out

    # ---- whole requests ---------------------------------------------------------
    def generate(self, prompts: Seq[Seq[int]], max_tokens: int = 16, sampling_params=None) -> List[List[int]]:
        """Generated token ids for every prompt, in the order given."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        ids = [self.add_request(p, max_tokens, sp) for p, sp in zip(prompts, sampling_params)]
        while self.has_unfinished():
            self.step()
        self.runner.check_device_errors()
        out = [list(self.sequences[i].generated) for i in ids]
        for i in ids:
            self.sequences.pop(i, None)
        return out

    def stats(self) -> dict:
        s = dict(self.scheduler.stats)
        s["free_pages"] = self.runner.cache.free_pages()
        s["running"] = len(self.scheduler.running)
        s["waiting"] = len(self.scheduler.waiting)
        return s
