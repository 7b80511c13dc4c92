"""Continuous batching under a token budget, with chunked prefill.

Decisions, all taken from the reference's scheduler (engine/scheduler.py:26-173):

* A request whose prompt + max_tokens exceeds ``max_model_len``, or that could not be held
  by an empty pool, is refused at ``add`` with ValueError.
* Each step has ``max_num_batched_tokens`` tokens to give out: first to running requests
  that owe one token (decodes), then to running requests in the middle of their prompt,
  both in admission order, then to waiting requests from the head of the queue (no
  skipping) while the budget, ``max_num_seqs`` and the pages last.  A prompt is cut where
  the budget ends, or at ``long_prefill_token_threshold`` if that is set.
* When pages run out for a running request, the newest running request that is not yet
  part of this step (under ``priority``: the one with the worst (priority, arrival)) is
  preempted: it gives back all its pages and goes to the front of the waiting queue, to be
  recomputed later, prompt and generated tokens alike (much of it usually found again as
  prefix hits).  If the victim is the requester itself, scheduling of running requests
  stops there.  After a preemption nothing new is admitted in that step.
* Without chunked prefill: whole prompts are admitted first; decoding happens only in
  steps that admit nothing.
* ``postprocess`` advances the counters, hashes pages that filled, gives back pages that a
  window has passed, appends the sampled token and finishes a request on EOS (unless
  ``ignore_eos``) or at ``max_tokens``.
"""
from __future__ import annotations

from collections import deque
from typing import Optional, Sequence as Seq

from ..cache.manager import CacheManager
from .sequence import Sequence, SequenceStatus


class Scheduler:
    def __init__(self, config, cache: CacheManager):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.long_prefill_token_threshold = config.long_prefill_token_threshold
        self.enable_chunked_prefill = config.enable_chunked_prefill
        self.policy = config.scheduling_policy
        self.eos = config.eos
        self.max_model_len = config.max_model_len
        self.cache = cache
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.num_preemptions = 0

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    # ---- admission -------------------------------------------------------------------
    def add(self, seq: Sequence) -> None:
        total = seq.num_prompt_tokens + seq.sampling_params.max_tokens
        if total > self.max_model_len:
            raise ValueError(f"prompt+max_tokens={total} exceeds max_model_len={self.max_model_len}")
        portion = self.max_num_batched_tokens if self.enable_chunked_prefill else total
        if not self.cache.fits_at_all(total, portion):
            raise ValueError(f"a request of {total} tokens needs more pages than the cache pool has "
                             f"({[p.num_pages for p in self.cache.pools]} pages of {self.cache.page_size})")
        self._push_waiting(seq)

    @staticmethod
    def _key(seq: Sequence):
        return (seq.priority, seq.arrival_time)

    def _push_waiting(self, seq: Sequence, front: bool = False) -> None:
        if self.policy == "priority":
            i = 0
            while i < len(self.waiting) and self._key(self.waiting[i]) <= self._key(seq):
                i += 1
            self.waiting.insert(i, seq)
        elif front:
            self.waiting.appendleft(seq)
        else:
            self.waiting.append(seq)

    def _portion(self, owed: int, budget: int) -> int:
        n = owed
        if 0 < self.long_prefill_token_threshold < n:
            n = self.long_prefill_token_threshold
        return min(n, budget)

    # ---- when pages run out ----------------------------------------------------------
    def _pick_victim(self, scheduled: set[int]) -> Sequence:
        cands = [s for s in self.running if s.seq_id not in scheduled]
        if self.policy == "priority":
            return max(cands, key=self._key)
        return cands[-1]

    def _preempt(self, seq: Sequence) -> None:
        self.running.remove(seq)
        seq.status = SequenceStatus.WAITING
        seq.num_scheduled_tokens = 0
        self.cache.free(seq)
        self._push_waiting(seq, front=True)
        self.num_preemptions += 1

    def _allocate_or_preempt(self, seq: Sequence, n: int, scheduled: set[int]) -> bool:
        while not self.cache.allocate(seq, n):
            victim = self._pick_victim(scheduled)
            self._preempt(victim)
            if victim is seq:
                return False
        return True

    def _start(self, seq: Sequence, n: int, out: list[Sequence], ids: set[int]) -> None:
        self.waiting.popleft()
        seq.status = SequenceStatus.RUNNING
        seq.num_scheduled_tokens = n
        self.running.append(seq)
        out.append(seq)
        ids.add(seq.seq_id)

    # ---- one step's batch ------------------------------------------------------------
    def schedule(self) -> list[Sequence]:
        batch = self._schedule_chunked() if self.enable_chunked_prefill else self._schedule_prefill_first()
        if not batch:
            raise RuntimeError("nothing can be scheduled: the cache pool or the token budget is too small")
        return batch

    def _schedule_chunked(self) -> list[Sequence]:
        budget = self.max_num_batched_tokens
        out: list[Sequence] = []
        ids: set[int] = set()
        preempted = False
        decodes = [s for s in self.running if s.num_uncomputed_tokens == 1]
        partials = [s for s in self.running if s.num_uncomputed_tokens > 1]
        for seq in decodes + partials:
            if budget == 0:
                break
            if seq.status != SequenceStatus.RUNNING:      # preempted earlier in this loop
                continue
            n = self._portion(seq.num_uncomputed_tokens, budget)
            before = self.num_preemptions
            ok = self._allocate_or_preempt(seq, n, ids)
            preempted |= self.num_preemptions > before
            if not ok:
                break
            seq.num_scheduled_tokens = n
            budget -= n
            out.append(seq)
            ids.add(seq.seq_id)
        if preempted:
            return out
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            seq = self.waiting[0]
            hits = self.cache.find_prefix_hit(seq.token_ids)
            n_hit = len(hits[0]) if hits else 0
            n = self._portion(seq.num_tokens - n_hit * self.cache.page_size, budget)
            if not self.cache.allocate(seq, n, hits):
                break
            self._start(seq, n, out, ids)
            budget -= n
        return out

    def _schedule_prefill_first(self) -> list[Sequence]:
        budget = self.max_num_batched_tokens
        out: list[Sequence] = []
        ids: set[int] = set()
        while self.waiting and len(self.running) < self.max_num_seqs:
            seq = self.waiting[0]
            hits = self.cache.find_prefix_hit(seq.token_ids)
            n_hit = len(hits[0]) if hits else 0
            n = seq.num_tokens - n_hit * self.cache.page_size
            if n > budget or not self.cache.allocate(seq, n, hits):
                break
            self._start(seq, n, out, ids)
            budget -= n
        if out:
            return out
        for seq in list(self.running):
            if seq.status != SequenceStatus.RUNNING:
                continue
            if not self._allocate_or_preempt(seq, 1, ids):
                break
            seq.num_scheduled_tokens = 1
            out.append(seq)
            ids.add(seq.seq_id)
        return out

    # ---- after the step --------------------------------------------------------------
    def postprocess(self, seqs: Seq[Sequence], token_ids: Seq[Optional[int]]) -> list[Sequence]:
        emitted = []
        for seq, token_id in zip(seqs, token_ids):
            sampled = seq.samples_this_step
            seq.num_computed_tokens += seq.num_scheduled_tokens
            seq.num_scheduled_tokens = 0
            self.cache.hash_full_pages(seq, seq.token_ids)
            self.cache.release_behind_window(seq)
            if not sampled:
                continue
            seq.append_token(token_id)
            emitted.append(seq)
            done = (token_id == self.eos and not seq.sampling_params.ignore_eos) or \
                seq.num_completion_tokens == seq.sampling_params.max_tokens
            if done:
                seq.status = SequenceStatus.FINISHED
                self.cache.free(seq)
                self.running.remove(seq)
        return emitted
