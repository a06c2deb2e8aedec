"""Continuous batching: admission, prompt portions under a token budget, decoding,
finishing and freeing, and what happens when pages run out.

Names and defaults of the limits follow the reference's `SchedulerConfig`
(crates/core/src/types/scheduler_config.rs:115-132: max_num_seqs 256,
max_num_batched_tokens 4096, prefill_chunk_size 512).  The policy is this
engine's own.  The reference alternates all-prefill and all-decode rounds
(crates/core/src/scheduler/phase_scheduler.rs:83-128); here every step holds the
next token of every decoding request and, beside them, as many prompt tokens as
the budget allows, first come first served by arrival.

When pages run out the most recently admitted running request is pre-empted: its
pages are given back and it returns to the head of the queue with its generated
tokens kept, to be recomputed as one longer prompt (the reference pre-empts by
recompute too, crates/core/src/scheduler/engine/memory.rs:46-162, with another
choice of victim).  Older requests therefore always make progress.

The scheduler is host logic only: it reads page counts from the cache manager and
decides; the step function takes the pages.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional

from ..cache.manager import OutOfPages
from ..sampling.params import SamplingParams


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 4096
    prefill_chunk_size: int = 512
    max_model_len: Optional[int] = None

    def validate(self):
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0 or self.prefill_chunk_size <= 0:
            raise ValueError("max_num_seqs, max_num_batched_tokens and prefill_chunk_size must be positive")
        return self


@dataclass
class Sequence:
    seq_id: int
    tokens: List[int]                   # prompt followed by generated tokens
    prompt_len: int
    max_tokens: int
    params: SamplingParams
    num_computed: int = 0               # tokens whose keys and values are in the cache
    status: str = "waiting"             # waiting | running | finished
    finish_reason: Optional[str] = None
    preemptions: int = 0
    arrival: int = 0

    @property
    def generated(self) -> List[int]:
        return self.tokens[self.prompt_len:]

    @property
    def remaining(self) -> int:
        return len(self.tokens) - self.num_computed


@dataclass
class Scheduled:
    seq: Sequence
    start: int
    count: int
    samples: bool                       # the portion reaches the sequence's last token


@dataclass
class StepPlan:
    entries: List[Scheduled] = field(default_factory=list)
    preempted: List[Sequence] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class AdmissionError(ValueError):
    pass


class Scheduler:
    def __init__(self, cache, config: SchedulerConfig = None, native: Optional[bool] = None):
        """`native`: take each step's decision in the C++ core (the cache manager must be the native
        one; default: whenever it is).  The Python policy below is the reference; both are run by
        the same tests and must decide alike."""
        self.cache = cache
        self.config = (config or SchedulerConfig()).validate()
        can = hasattr(cache, "schedule")
        if native and not can:
            raise ValueError("the native scheduler needs the native cache manager")
        self.native = can if native is None else bool(native)
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self._next_id = 1                 # ids start at 1, as the reference's do
        self._arrivals = 0
        self.stats = dict(steps=0, prefill_tokens=0, decode_tokens=0, preemptions=0, finished=0)

    # ---- admission ----------------------------------------------------------
    def add_request(self, prompt, max_tokens: int, params: SamplingParams = None) -> Sequence:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise AdmissionError("an empty prompt is rejected")   # crates/core/src/engine/lifecycle.rs:176-179
        if max_tokens <= 0:
            raise AdmissionError("max_tokens must be positive")
        total = len(prompt) + max_tokens
        if self.config.max_model_len is not None and total > self.config.max_model_len:
            raise AdmissionError(f"prompt ({len(prompt)}) + max_tokens ({max_tokens}) exceeds max_model_len "
                                 f"{self.config.max_model_len}")
        ps = self.cache.page_size
        for need, pool in zip(self.cache.layout.paged_groups, self.cache.pools):
            longest_step = max(self.config.prefill_chunk_size, self.config.max_num_batched_tokens)
            most = total if need.window is None else min(total, need.window + 2 * ps + longest_step)
            if -(-most // ps) > pool.size:
                raise AdmissionError(f"the request needs {-(-most // ps)} pages alone; the pool has {pool.size}")
        seq = Sequence(self._next_id, prompt, len(prompt), int(max_tokens), (params or SamplingParams()).validate(),
                       arrival=self._arrivals)
        self._next_id += 1
        self._arrivals += 1
        self.waiting.append(seq)
        return seq

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step -----------------------------------------------------------
    def schedule(self) -> StepPlan:
        if self.native:
            return self._schedule_native()
        plan = StepPlan()
        while True:
            entries, starved = self._compose()
            if starved is None:
                break
            victim = self.running[-1]                      # the most recently admitted
            self._preempt(victim)
            plan.preempted.append(victim)
        plan.entries = entries
        return plan

    def _schedule_native(self) -> StepPlan:
        """The same decision taken by the C++ core; what it answers is applied here."""
        cfg = self.config
        seqs = list(self.running) + list(self.waiting)
        if not seqs:
            return StepPlan()
        held = [s.seq_id if s.seq_id in self.cache.requests else None for s in seqs]
        try:
            entries, victims, admitted = self.cache.schedule(
                cfg.max_num_seqs, cfg.max_num_batched_tokens, cfg.prefill_chunk_size, len(self.running),
                [s.remaining for s in seqs], [s.num_computed for s in seqs], held, [s.arrival for s in seqs])
        except OutOfPages as e:
            raise RuntimeError("a sequence cannot get its pages although it runs alone") from e
        plan = StepPlan()
        for v in victims:
            self._preempt(seqs[v])
            plan.preempted.append(seqs[v])
        for a in admitted:
            seq = seqs[a]
            if not self.waiting or self.waiting[0] is not seq:
                raise RuntimeError("the native scheduler admitted a sequence that is not at the head of the queue")
            self.waiting.popleft()
            seq.status = "running"
            self.running.append(seq)
        if admitted:
            self.running.sort(key=lambda s: s.arrival)
        plan.entries = [Scheduled(seqs[i], seqs[i].num_computed, int(n), seqs[i].num_computed + int(n) == len(seqs[i].tokens))
                        for i, n in entries]
        return plan

    def _chunk(self, seq: Sequence, room: int, capped: bool = True) -> int:
        """Tokens of `seq` in this step.  `prefill_chunk_size` bounds a prompt's portion only in a step that
        also holds decoding requests (whose next tokens would wait behind a long portion); a step of prompts
        alone gives a prompt all the room the token budget leaves."""
        n = min(seq.remaining, room)
        if seq.remaining > 1 and capped:
            n = min(n, self.config.prefill_chunk_size)
        return n

    def _compose(self):
        """(entries, None) or (_, a running sequence that cannot get its pages)."""
        cfg = self.config
        free = list(self.cache.free_pages())
        free_slots = self.cache.slots.free_count
        room = cfg.max_num_batched_tokens
        entries: List[Scheduled] = []
        # decoding requests first, then running prompts, both in order of arrival
        order = [s for s in self.running if s.remaining == 1] + [s for s in self.running if s.remaining > 1]
        capped = any(s.remaining == 1 for s in self.running)     # someone decodes in this step
        for seq in order:
            n = self._chunk(seq, room, capped)
            if n <= 0:
                continue
            need = self._pages_needed(seq, n)
            if any(a > b for a, b in zip(need, free)):
                if len(self.running) == 1 and not entries:
                    raise RuntimeError(f"sequence {seq.seq_id} cannot get its pages although it runs alone")
                return entries, seq
            free = [b - a for a, b in zip(need, free)]
            room -= n
            entries.append(Scheduled(seq, seq.num_computed, n, seq.num_computed + n == len(seq.tokens)))
        # admit from the head of the queue while slots, pages and budget last
        while self.waiting and room > 0 and len(self.running) < cfg.max_num_seqs:
            seq = self.waiting[0]
            n = self._chunk(seq, room, capped)
            need = self._pages_needed(seq, n)
            if any(a > b for a, b in zip(need, free)) or (seq.seq_id not in self.cache.requests and free_slots < 1):
                break                                         # head-of-line: never admit what cannot get pages
            self.waiting.popleft()
            seq.status = "running"
            self.running.append(seq)
            self.running.sort(key=lambda s: s.arrival)
            if seq.seq_id not in self.cache.requests:
                free_slots -= 1
            free = [b - a for a, b in zip(need, free)]
            room -= n
            entries.append(Scheduled(seq, seq.num_computed, n, seq.num_computed + n == len(seq.tokens)))
        return entries, None

    def _pages_needed(self, seq: Sequence, n: int):
        """Pages that n more tokens take in every group: the blocks their positions open.  (A running
        sequence holds num_computed tokens in the cache; a window gives pages back but keeps the
        block table's length, so the count is the same for every group.)"""
        ps = self.cache.page_size
        held = seq.num_computed if seq.seq_id in self.cache.requests else 0
        return [-(-(held + n) // ps) - -(-held // ps)] * len(self.cache.pools)

    def _preempt(self, seq: Sequence):
        self.running.remove(seq)
        if seq.seq_id in self.cache.requests:
            self.cache.free(seq.seq_id)
        seq.num_computed = 0
        seq.status = "waiting"
        seq.preemptions += 1
        self.waiting.appendleft(seq)
        self.stats["preemptions"] += 1

    # ---- after the step -------------------------------------------------------
    def update(self, plan: StepPlan, sampled: List[Optional[int]]) -> List[Sequence]:
        """`sampled[i]` is the token drawn for plan.entries[i] (None when the portion did
        not reach the end of its sequence).  Returns the sequences that finished."""
        done = []
        self.stats["steps"] += 1
        for entry, token in zip(plan.entries, sampled):
            seq = entry.seq
            if seq.status == "finished":                   # ended (stop, cancel) while a step launched ahead held it
                continue
            seq.num_computed += entry.count
            self.stats["decode_tokens" if entry.count == 1 and entry.start >= seq.prompt_len else "prefill_tokens"] += entry.count
            if not entry.samples:
                continue
            if token is None:
                raise ValueError(f"sequence {seq.seq_id} reached its end but no token was sampled")
            seq.tokens.append(int(token))
            reason = self._finish_reason(seq)
            if reason:
                self._finish(seq, reason)
                done.append(seq)
        return done

    def _finish_reason(self, seq: Sequence) -> Optional[str]:
        gen = seq.generated
        stops = seq.params.stop_token_sequences
        if stops:
            for s in stops:                                # suffix match on generated ids
                if s and len(gen) >= len(s) and gen[-len(s):] == list(s):
                    return "stop"
        if len(gen) >= seq.max_tokens:                     # crates/core/src/scheduler/engine/update.rs:214-264
            return "length"
        return None

    def _finish(self, seq: Sequence, reason: str):
        seq.status, seq.finish_reason = "finished", reason
        if seq in self.running:
            self.running.remove(seq)
        if seq.seq_id in self.cache.requests:
            self.cache.free(seq.seq_id)
        self.stats["finished"] += 1

    def cancel(self, seq_id: int) -> bool:
        for seq in list(self.running) + list(self.waiting):
            if seq.seq_id == seq_id:
                if seq in self.waiting:
                    self.waiting.remove(seq)
                self._finish(seq, "cancelled")
                return True
        return False
