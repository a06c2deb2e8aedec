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

import time
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence as Seq

import torch

from ..sampling import Sampler, SamplingParams
from .loading import load_model_dir, parse_dtype
from .runner import ModelRunner, StepEntry
from .scheduler import Scheduler, SchedulerConfig, Sequence


@contextmanager
def _span(name: str):
    """A named range on the profiler's timeline (NVTX), as the reference wraps the phases of a step in
    tracing spans (crates/core/src/scheduler/engine/state/batch.rs:23-28).  Costs nothing when no
    profiler listens."""
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


class StepTimes:
    """Host time of every `step()` by kind, and device time of every N-th step (events on the stream;
    read only once they have completed, so that steps launched ahead are never waited for)."""
    KINDS = ("prompt", "mixed", "decode")

    def __init__(self, device_every: int = 16, keep: int = 4096):
        self.device_every, self.keep = int(device_every), int(keep)
        self.host_ms = {k: [] for k in self.KINDS}
        self.device_ms = {k: [] for k in self.KINDS}
        self.count = {k: 0 for k in self.KINDS}
        self._pending = []

    @staticmethod
    def kind_of(plan) -> str:
        prompt = any(e.count > 1 or not e.samples for e in plan.entries)
        single = any(e.count == 1 and e.samples for e in plan.entries)
        return "mixed" if prompt and single else "prompt" if prompt else "decode"

    def host(self, kind: str, ms: float):
        self.count[kind] += 1
        self._add(self.host_ms[kind], ms)

    def _add(self, where, ms):
        where.append(ms)
        if len(where) > self.keep:
            del where[:len(where) - self.keep]

    def wants_device_time(self) -> bool:
        return self.device_every > 0 and sum(self.count.values()) % self.device_every == 0

    def device(self, kind, start, end):
        self._pending.append((kind, start, end))
        if len(self._pending) > 8:                       # read those that have completed; none is waited for
            self.harvest()
            del self._pending[:-64]                      # (a stream that never completes must not grow the list)

    def harvest(self):
        still = []
        for kind, start, end in self._pending:
            if end.query():
                self._add(self.device_ms[kind], start.elapsed_time(end))
            else:
                still.append((kind, start, end))
        self._pending = still

    @staticmethod
    def _quantile(values, q):
        v = sorted(values)
        return round(v[min(len(v) - 1, int(q * len(v)))], 4) if v else None

    def summary(self) -> dict:
        self.harvest()
        out = {}
        for k in self.KINDS:
            out[k] = {"steps": self.count[k],
                      "host_ms_p50": self._quantile(self.host_ms[k], 0.5), "host_ms_p90": self._quantile(self.host_ms[k], 0.9),
                      "device_ms_p50": self._quantile(self.device_ms[k], 0.5),
                      "device_ms_p90": self._quantile(self.device_ms[k], 0.9), "device_samples": len(self.device_ms[k])}
        return out


class _InFlight:
    """A launched step whose tokens the host has not read yet."""
    def __init__(self, plan, sampling):
        self.plan, self.sampling, self.kind = plan, sampling, "decode"
        self.event = self.tokens_device = self.host_tokens = self.host_logprobs = None


@dataclass
class StepOutput:
    seq_id: int
    token: int
    finished: bool
    finish_reason: Optional[str] = None
    logprob: Optional[float] = None


class LLMEngine:
    def __init__(self, model=None, *, dtype="bfloat16", device="cuda:0", kv_blocks: Optional[int] = None,
                 block_size: int = 64, max_batch_size: int = 256, max_num_batched_tokens: int = 4096,
                 prefill_chunk_size: int = 512, max_model_len: Optional[int] = None, plan=None, weights=None,
                 logprobs: bool = False, lookahead: bool = True, gpu_memory_fraction: float = 0.9):
        """`model`: a folder with config.json and safetensors (never downloaded).  `kv_blocks`
        and `max_batch_size` carry the reference's names (crates/server/src/cli/args.rs:155-186);
        `block_size` is its BLOCK_SIZE constant (crates/traits/src/types.rs:13: 16) made an option; the
        default here is 64 positions a page, which one TMA box brings whole (measured at Qwen3-8B sizes against
        pages of 16: 64 requests decode 8.6 % faster, a 2,048-token prompt 6 %, 8 requests alike).
        `kv_blocks=None` (the default here; the reference's is 1,024) sizes the cache from the GPU:
        `gpu_memory_fraction` of the memory that is free once the weights are resident, less a
        reserve for activations (cache/sizing.py).  Alternatively pass `plan` and `weights` of a
        model that is already on the device; the engine takes the dict over and empties it.
        `lookahead`: see `step`."""
        self.dtype = parse_dtype(dtype)
        if plan is None:
            if model is None:
                raise ValueError("give a model folder (or plan and weights)")
            _, plan, weights = load_model_dir(model, self.dtype, device)
        if max_model_len is None:
            max_model_len = plan.max_position_embeddings
        self.runner = ModelRunner(plan, weights, dtype=self.dtype, device=device, page_size=block_size,
                                  num_pages=kv_blocks, max_requests=max_batch_size, max_context=max_model_len,
                                  memory_fraction=gpu_memory_fraction, max_step_tokens=max_num_batched_tokens,
                                  own_weights=True)
        del weights
        self.scheduler = Scheduler(self.runner.cache, SchedulerConfig(
            max_num_seqs=max_batch_size, max_num_batched_tokens=max_num_batched_tokens,
            prefill_chunk_size=prefill_chunk_size, max_model_len=max_model_len))
        self.sampler = Sampler(device)
        self.want_logprobs = logprobs
        self.sequences: Dict[int, Sequence] = {}
        self.lookahead = bool(lookahead)
        self._ahead = None                      # a step that is launched but not yet reported
        self._slot = 0
        self._host_tok = [None, None]           # pinned read-back buffers of the two steps that can be in flight
        self._host_lp = [None, None]
        self.times = StepTimes()

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
        self.sequences.pop(seq_id, None)
        return self.scheduler.cancel(seq_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work() or (self._ahead is not None and self._ahead_is_live())

    def _ahead_is_live(self) -> bool:
        return any(e.seq.status != "finished" for e in self._ahead.plan.entries)

    # ---- one step -------------------------------------------------------------
    def step(self) -> List[StepOutput]:
        """Outputs of one step: the new token of every request whose portion reached its end.

        With `lookahead` (the default) the step after the one being reported is launched before the
        host has read this one's tokens, whenever that step can be foretold: every request of this
        step yields a token and goes on (none reaches max_tokens), nobody waits for admission, no
        option needs the token on the host (penalties, biases).  Its input tokens then stay on the
        device.  A request that turns out to have ended (stop sequence, cancel) has cost one token
        of work that is thrown away."""
        t0 = time.perf_counter()
        if self._ahead is None:
            with _span("schedule"):
                plan = self.scheduler.schedule()
            if not plan.entries:
                return []
            self._ahead = self._launch(plan)
        current, self._ahead = self._ahead, None
        if self.lookahead:
            with _span("launch ahead"):
                self._ahead = self._launch_following(current)
        with _span("collect"):
            out = self._collect(current)
        self.times.host(current.kind, (time.perf_counter() - t0) * 1e3)
        return out

    def _launch(self, plan) -> "_InFlight":
        entries = [StepEntry(e.seq.seq_id, e.seq.tokens[e.start:e.start + e.count],
                             [e.count - 1] if e.samples else []) for e in plan.entries]
        kind = StepTimes.kind_of(plan)
        timed = self.times.wants_device_time()
        if timed:
            start = torch.cuda.Event(enable_timing=True)
            start.record()
        with _span("pack and launch " + kind):
            logits = self.runner.step(entries)
        sampling = [e for e in plan.entries if e.samples]
        with _span("sample"):
            flight = self._sample(plan, sampling, logits, [len(e.seq.generated) for e in sampling])
        flight.kind = kind
        if timed:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.times.device(kind, start, end)
        return flight

    def _sample(self, plan, sampling, logits, steps) -> "_InFlight":
        """Queues sampling and the copy of the tokens to pinned host memory; nothing waits here."""
        flight = _InFlight(plan, sampling)
        if sampling:
            tok, lp = self.sampler.sample(logits, [e.seq.params for e in sampling], [e.seq.generated for e in sampling],
                                          self.want_logprobs, steps=steps)
            k = self._slot
            self._slot ^= 1
            n = len(sampling)
            if self._host_tok[k] is None or self._host_tok[k].numel() < n:
                self._host_tok[k] = torch.empty(max(n, 64), dtype=torch.int32).pin_memory()
                self._host_lp[k] = torch.empty(max(n, 64), dtype=torch.float32).pin_memory()
            self._host_tok[k][:n].copy_(tok, non_blocking=True)              # the step's only read-back
            if lp is not None:
                self._host_lp[k][:n].copy_(lp, non_blocking=True)
            flight.event = torch.cuda.Event()
            flight.event.record()
            flight.tokens_device, flight.host_tokens = tok, self._host_tok[k][:n]
            flight.host_logprobs = self._host_lp[k][:n] if lp is not None else None
        return flight

    def _launch_following(self, current: "_InFlight"):
        """The decode step that follows `current`, launched with its tokens still on the device, or
        None when it cannot be foretold."""
        entries = current.plan.entries
        if not entries or len(current.sampling) != len(entries) or self.scheduler.waiting:
            return None
        steps = []
        for e in entries:
            seq = e.seq
            produced = len(seq.tokens) - seq.prompt_len + 1            # once the token in flight has arrived
            if seq.status != "running" or seq.params.needs_penalties or produced >= seq.max_tokens:
                return None
            steps.append(produced)
        longest = max(e.start + e.count for e in entries) + 1
        timed = self.times.wants_device_time()
        if timed:
            start = torch.cuda.Event(enable_timing=True)
            start.record()
        logits = self.runner.step_ahead([e.seq.seq_id for e in entries], current.tokens_device, longest)
        if logits is None:
            return None
        from .scheduler import Scheduled, StepPlan
        plan = StepPlan()
        plan.entries = [Scheduled(e.seq, e.start + e.count, 1, True) for e in entries]
        flight = self._sample(plan, plan.entries, logits, steps)
        if timed:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.times.device("decode", start, end)
        return flight

    def _collect(self, flight: "_InFlight") -> List[StepOutput]:
        plan = flight.plan
        sampled: List[Optional[int]] = [None] * len(plan.entries)
        logprobs = None
        if flight.sampling:
            flight.event.synchronize()
            host = flight.host_tokens.tolist()
            logprobs = flight.host_logprobs.tolist() if flight.host_logprobs is not None else None
            it = iter(host)
            sampled = [next(it) if e.samples else None for e in plan.entries]
        live = [e.seq.status != "finished" for e in plan.entries]     # a step launched ahead may hold ended requests
        self.scheduler.update(plan, sampled)
        out, k = [], 0
        for e, t, alive in zip(plan.entries, sampled, live):
            if t is None:
                continue
            if alive:
                out.append(StepOutput(e.seq.seq_id, t, e.seq.status == "finished", e.seq.finish_reason,
                                      logprobs[k] if logprobs else None))
                if e.seq.status == "finished":                       # reported: the engine keeps it no longer
                    self.sequences.pop(e.seq.seq_id, None)
            k += 1
        return out

    # ---- whole requests ---------------------------------------------------------
    def generate(self, prompts: Seq[Seq[int]], max_tokens: int = 16, sampling_params=None) -> List[List[int]]:
        """Generated token ids for every prompt, in the order given."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        seqs = [self.sequences[self.add_request(p, max_tokens, sp)] for p, sp in zip(prompts, sampling_params)]
        while self.has_unfinished():
            self.step()
        self._ahead = None                      # at most a step launched ahead for requests that have ended since
        self.runner.check_device_errors()
        return [list(seq.generated) for seq in seqs]

    def stats(self) -> dict:
        """Counters of the scheduler, the state of the pools and queues, and step times by kind of step
        (`prompt`: portions only, `decode`: single tokens only, `mixed`): how many, the median and the
        90th percentile of the host time of `step()` and, for every 16th step, of the time on the device."""
        s = dict(self.scheduler.stats)
        s["free_pages"] = self.runner.cache.free_pages()
        s["running"] = len(self.scheduler.running)
        s["waiting"] = len(self.scheduler.waiting)
        s["step_times"] = self.times.summary()
        return s
