"""Continuous batching under a token budget, with chunked prefill.

The decisions are the reference scheduler's (engine/scheduler.py:26-173); the code is organised around a
``_Step`` object that holds one step's budget and choices.

* ``add`` refuses a request whose prompt + max_tokens exceeds ``max_model_len`` or that an empty pool
  could not hold (ValueError).
* A step has ``max_num_batched_tokens`` tokens to give out.  First come running requests that owe one token
  (decodes), then running requests in the middle of their prompt, both in admission order; then waiting
  requests from the head of the queue, without skipping, while budget, ``max_num_seqs`` and pages last.  A
  prompt is cut where the budget ends, or at ``long_prefill_token_threshold`` if that is set.
* When a running request cannot get pages, the newest running request that is not yet part of the step
  (under ``priority``: the one with the worst (priority, arrival)) is preempted: it gives back everything
  and goes to the front of the queue, to be recomputed later, prompt and generated tokens alike (mostly
  found again as prefix hits).  If the victim is the requester itself, no further running request is
  served in this step.  A step that preempted admits nothing new.
* Without chunked prefill whole prompts are admitted first and decoding happens only in steps that admit
  nothing.
* ``postprocess`` advances the counters, hashes pages that filled, returns pages a window has passed,
  appends the drawn token and finishes a request on EOS (unless ``ignore_eos``) or at ``max_tokens``.
"""
from __future__ import annotations

from collections import deque
from typing import Iterable, Optional, Sequence as Seq

from ..cache.manager import CacheManager
from .sequence import Sequence, SequenceStatus


class _Step:
    """The batch of one step while it is being put together."""

    def __init__(self, budget: int):
        self.budget = budget
        self.chosen: list[Sequence] = []
        self.chosen_ids: set[int] = set()
        self.preempted = False

    def take(self, seq: Sequence, n: int) -> None:
        seq.num_scheduled_tokens = n
        self.budget -= n
        self.chosen.append(seq)
        self.chosen_ids.add(seq.seq_id)


class Scheduler:
    def __init__(self, config, cache: CacheManager):
        self.cache = cache
        self.max_num_seqs: int = config.max_num_seqs
        self.max_num_batched_tokens: int = config.max_num_batched_tokens
        self.long_prefill_token_threshold: int = config.long_prefill_token_threshold
        self.enable_chunked_prefill: bool = config.enable_chunked_prefill
        self.policy: str = config.scheduling_policy
        self.max_model_len: int = config.max_model_len
        self.eos: Optional[int] = config.eos
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.num_preemptions = 0

    # ---- queue ------------------------------------------------------------------------------------------
    def is_finished(self) -> bool:
        return not (self.waiting or self.running)

    @staticmethod
    def _rank(seq: Sequence) -> tuple:
        return seq.priority, seq.arrival_time

    def _enqueue(self, seq: Sequence, at_front: bool) -> None:
        if self.policy == "priority":                     # kept sorted by (priority, arrival)
            pos = sum(1 for other in self.waiting if self._rank(other) <= self._rank(seq))
            self.waiting.insert(pos, seq)
        elif at_front:
            self.waiting.appendleft(seq)
        else:
            self.waiting.append(seq)

    def add(self, seq: Sequence) -> None:
        need = seq.num_prompt_tokens + seq.sampling_params.max_tokens
        if need > self.max_model_len:
            raise ValueError(f"prompt+max_tokens={need} exceeds max_model_len={self.max_model_len}")
        largest_portion = self.max_num_batched_tokens if self.enable_chunked_prefill else need
        if not self.cache.fits_at_all(need, largest_portion):
            pools = [p.num_pages for p in self.cache.pools]
            raise ValueError(f"a request of {need} tokens needs more pages than the cache pool has "
                             f"({pools} pages of {self.cache.page_size})")
        self._enqueue(seq, at_front=False)

    # ---- portions and pages -------------------------------------------------------------------------------
    def _portion(self, owed: int, budget: int) -> int:
        cap = self.long_prefill_token_threshold
        return min(owed if cap <= 0 else min(owed, cap), budget)

    def _evict_one(self, step: _Step) -> Sequence:
        """Preempt the newest (or worst-ranked) running request that is not part of the step yet."""
        candidates = [s for s in self.running if s.seq_id not in step.chosen_ids]
        victim = max(candidates, key=self._rank) if self.policy == "priority" else candidates[-1]
        self.running.remove(victim)
        self.cache.free(victim)
        victim.status = SequenceStatus.WAITING
        victim.num_scheduled_tokens = 0
        self._enqueue(victim, at_front=True)
        self.num_preemptions += 1
        step.preempted = True
        return victim

    def _pages_for_running(self, seq: Sequence, n: int, step: _Step) -> bool:
        """Pages for ``n`` more tokens of a running request, evicting others while the pool is short;
        False if the request itself had to go."""
        while not self.cache.allocate(seq, n):
            if self._evict_one(step) is seq:
                return False
        return True

    def _admit(self, seq: Sequence, n: int, hits, step: _Step) -> bool:
        if not self.cache.allocate(seq, n, hits):
            return False
        self.waiting.popleft()
        seq.status = SequenceStatus.RUNNING
        self.running.append(seq)
        step.take(seq, n)
        return True

    # ---- one step's batch -------------------------------------------------------------------------------------
    def schedule(self) -> list[Sequence]:
        step = _Step(self.max_num_batched_tokens)
        if self.enable_chunked_prefill:
            self._serve_running(step, decodes_only=False)
            if not step.preempted:
                self._admit_waiting(step, whole_prompts=False)
        else:
            self._admit_waiting(step, whole_prompts=True)
            if not step.chosen:
                self._serve_running(step, decodes_only=True)
        if not step.chosen:
            raise RuntimeError("nothing can be scheduled: the cache pool or the token budget is too small")
        return step.chosen

    def _serve_running(self, step: _Step, decodes_only: bool) -> None:
        if decodes_only:
            order: Iterable[Sequence] = list(self.running)
        else:
            order = [s for s in self.running if s.num_uncomputed_tokens == 1] + \
                    [s for s in self.running if s.num_uncomputed_tokens > 1]
        for seq in order:
            if not decodes_only and step.budget == 0:
                return
            if seq.status is not SequenceStatus.RUNNING:          # preempted a moment ago
                continue
            n = 1 if decodes_only else self._portion(seq.num_uncomputed_tokens, step.budget)
            if not self._pages_for_running(seq, n, step):
                return
            step.take(seq, n)

    def _admit_waiting(self, step: _Step, whole_prompts: bool) -> None:
        page = self.cache.page_size
        while self.waiting and len(self.running) < self.max_num_seqs and (whole_prompts or step.budget > 0):
            seq = self.waiting[0]
            hits = self.cache.find_prefix_hit(seq.token_ids)
            owed = seq.num_tokens - (len(hits[0]) if hits else 0) * page
            if whole_prompts:
                if owed > step.budget:
                    return
                n = owed
            else:
                n = self._portion(owed, step.budget)
            if not self._admit(seq, n, hits, step):
                return

    # ---- after the step ---------------------------------------------------------------------------------------
    def postprocess(self, seqs: Seq[Sequence], token_ids: Seq[Optional[int]]) -> list[Sequence]:
        emitted: list[Sequence] = []
        for seq, token in zip(seqs, token_ids):
            draws = seq.samples_this_step
            seq.num_computed_tokens += seq.num_scheduled_tokens
            seq.num_scheduled_tokens = 0
            self.cache.hash_full_pages(seq, seq.token_ids)
            self.cache.release_behind_window(seq)
            if not draws:
                continue
            seq.append_token(token)
            emitted.append(seq)
            if seq.reached_limit(self.eos):
                seq.status = SequenceStatus.FINISHED
                self.running.remove(seq)
                self.cache.free(seq)
        return emitted
