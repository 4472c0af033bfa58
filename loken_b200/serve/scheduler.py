"""Iteration-level scheduler of the continuous-batching engine.

Semantics follow the reference's `Scheduler` (`src/inference/serve/scheduler.rs:105-345`):
  1. running decodes grow first, oldest first; when the pool cannot give a sequence its next
     block, the NEWEST running sequence is preempted (its blocks are freed and it goes back
     to the head of the waiting queue; on readmission its prompt AND the tokens it already
     generated are recomputed);
  2. waiting requests are admitted first-come-first-served while fewer than `max_running`
     sequences run and the step's prefill tokens stay within `max_prefill_tokens` (the first
     prefill of a step is always admitted, so a long prompt cannot starve);
  3. admission goes through the prefix cache, so only the uncached suffix is prefilled;
  4. `trim` cuts a sequence back after a speculative reject;
  5. a request the pool can never hold (its prompt, or its prompt plus what it had generated before
     a preemption, needs more blocks than exist) is finished with reason "error" instead of waiting
     for ever at the head of the first-come-first-served queue.
A prompt longer than `max_prefill_tokens` is read in chunks over several steps.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

from .kv_manager import PagedKvAllocator
from .params import SamplingParams


@dataclass
class Sequence:
    seq_id: int
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    computed: int = 0            # tokens whose KV is in the cache
    cached_tokens: int = 0       # of which came from the prefix cache at (last) admission
    state: str = "waiting"       # waiting | running | finished
    finish_reason: Optional[str] = None
    arrival: float = 0.0
    first_token_time: Optional[float] = None
    preemptions: int = 0
    salt: int = 0
    draft_tokens: List[int] = field(default_factory=list)
    accepted_drafts: int = 0
    rejected_drafts: int = 0
    logprobs: List[tuple] = field(default_factory=list)   # per output token: (logprob, [(id, logprob)...])
    grammar: Optional[object] = None     # a text.grammar.GrammarSession while the request is constrained
    prompt_embeds: Optional[object] = None   # bf16 [len(prompt), hidden] on the device: the prompt as embedding rows
    # after a context shift: the tokens the cache still stands for, as of `kv_out0` output tokens (`prompt` and
    # `output` stay whole: they are what the client sent and what it was sent)
    kv_head: Optional[List[int]] = None
    kv_out0: int = 0
    shifts: int = 0

    @property
    def tokens(self) -> List[int]:
        """Token i is the token at cache position i."""
        if self.kv_head is None:
            return self.prompt + self.output
        return self.kv_head + self.output[self.kv_out0:]

    @property
    def total_len(self) -> int:
        if self.kv_head is None:
            return len(self.prompt) + len(self.output)
        return len(self.kv_head) + len(self.output) - self.kv_out0

    def drop_positions(self, n_keep: int, n_discard: int):
        toks = self.tokens
        self.kv_head = toks[:n_keep] + toks[n_keep + n_discard:]
        self.kv_out0 = len(self.output)
        self.shifts += 1


@dataclass
class PrefillItem:
    seq: Sequence
    start: int        # first position computed this step
    end: int          # one past the last
    is_last_chunk: bool


@dataclass
class StepPlan:
    prefills: List[PrefillItem] = field(default_factory=list)
    decodes: List[Sequence] = field(default_factory=list)
    preempted: List[Sequence] = field(default_factory=list)
    rejected: List[Sequence] = field(default_factory=list)   # finished with "error": the pool can never hold them

    @property
    def empty(self) -> bool:
        return not self.prefills and not self.decodes


class Scheduler:
    def __init__(self, alloc: PagedKvAllocator, max_running: int = 256, max_prefill_tokens: int = 8192,
                 lookahead: int = 0):
        self.alloc = alloc
        self.max_running = max_running
        self.max_prefill_tokens = max_prefill_tokens
        self.lookahead = lookahead          # extra slots a decode needs per step (speculative rows)
        self.on_finish = None               # callable(seq, cached positions), run before a finished sequence's blocks are freed
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []   # admission order: oldest first
        self.finished: List[Sequence] = []

    def fits_pool(self, seq: Sequence) -> bool:
        """Could the whole pool, with nothing else in it, hold this sequence and its next token?"""
        return self.alloc.blocks_needed(seq.total_len + 1 + self.lookahead) <= self.alloc.num_blocks

    def add_request(self, seq: Sequence):
        seq.state = "waiting"
        self.waiting.append(seq)
        if not self.fits_pool(seq):
            self.finish(seq, "error")

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _preempt(self, seq: Sequence):
        self.alloc.free(seq.seq_id)
        seq.computed = 0
        seq.state = "waiting"
        seq.preemptions += 1
        self.running.remove(seq)
        self.waiting.appendleft(seq)

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        # 1. decodes grow, oldest first; preempt the newest under pressure
        for seq in list(self.running):
            if seq.state != "running" or seq.computed < seq.total_len - 1:
                continue        # still prefilling (chunked) or already preempted this step
            need = 1 + self.lookahead
            grown = False
            while True:
                have = self.alloc.length(seq.seq_id)
                want = seq.total_len + self.lookahead
                if want <= have or self.alloc.append(seq.seq_id, want - have):
                    grown = True
                    break
                victim = next((s for s in reversed(self.running) if s is not seq and s.state == "running"), None)
                if victim is None:
                    break
                self._preempt(victim)
                plan.preempted.append(victim)
                if victim in plan.decodes:
                    plan.decodes.remove(victim)
            if grown:
                plan.decodes.append(seq)
            else:
                self._preempt(seq)
                plan.preempted.append(seq)
            del need
        # 2. chunked prefills in flight continue
        budget = self.max_prefill_tokens
        for seq in self.running:
            if seq.state == "running" and seq.computed < seq.total_len - 1 and seq not in plan.decodes:
                if seq.computed >= seq.total_len:
                    continue
                n = min(budget, seq.total_len - seq.computed) if plan.prefills else seq.total_len - seq.computed
                n = min(n, self.max_prefill_tokens)
                if n <= 0:
                    break
                end = seq.computed + n
                plan.prefills.append(PrefillItem(seq, seq.computed, end, end == seq.total_len))
                budget -= n
        # 3. admit waiting requests FCFS
        while self.waiting and len(self.running) < self.max_running:
            seq = self.waiting[0]
            if not self.fits_pool(seq):
                # grown past the pool while it ran (preempted with its output): it can never come back
                self.finish(seq, "error")
                plan.rejected.append(seq)
                continue
            toks = seq.tokens
            if plan.prefills and budget <= 0:
                break
            cached = self.alloc.allocate_with_prefix(seq.seq_id, toks, seq.salt)
            if cached is None:
                if not self.running and not plan.prefills and not plan.decodes:
                    # nothing runs, so nothing will ever free a block for it
                    self.finish(seq, "error")
                    plan.rejected.append(seq)
                    continue
                break
            uncached = len(toks) - cached
            if plan.prefills and uncached > budget and uncached <= self.max_prefill_tokens:
                self.alloc.free(seq.seq_id)     # does not fit this step's budget: wait a step
                break
            self.waiting.popleft()
            seq.state = "running"
            seq.computed = cached
            seq.cached_tokens = cached
            self.running.append(seq)
            n = min(uncached, self.max_prefill_tokens if not plan.prefills else max(budget, 0))
            n = max(n, 1)
            end = cached + n
            plan.prefills.append(PrefillItem(seq, cached, end, end == len(toks)))
            budget -= n
        return plan

    def on_step_done(self, plan: StepPlan):
        """Marks the planned work as computed and publishes finished prompts' full blocks."""
        for it in plan.prefills:
            it.seq.computed = it.end
            if it.is_last_chunk:
                self.alloc.commit_prefix(it.seq.seq_id, it.seq.tokens[:it.end], it.seq.salt)
        for seq in plan.decodes:
            seq.computed = seq.total_len

    def finish(self, seq: Sequence, reason: str):
        seq.state = "finished"
        seq.finish_reason = reason
        if seq in self.running:
            self.running.remove(seq)
        elif seq in self.waiting:
            self.waiting.remove(seq)
        if seq.seq_id in self.alloc.seqs:
            # generated tokens' full blocks are as reusable as the prompt's
            n = min(seq.computed, seq.total_len)
            self.alloc.seqs[seq.seq_id].length = min(self.alloc.seqs[seq.seq_id].length, max(n, 0))
            self.alloc.commit_prefix(seq.seq_id, seq.tokens[:n], seq.salt)
            if self.on_finish is not None and n > 0:
                self.on_finish(seq, n)          # the cache's disk tier reads the rows while the blocks are still owned
            self.alloc.free(seq.seq_id)
        self.finished.append(seq)

    def trim(self, seq: Sequence, new_len: int):
        """Cuts the sequence's cache back to `new_len` tokens (rows rejected by verification)."""
        self.alloc.trim(seq.seq_id, new_len)
        seq.computed = min(seq.computed, new_len)
