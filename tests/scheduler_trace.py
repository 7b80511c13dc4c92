"""Random workloads for a scheduler and the record of what it decides, step by step.

The same driver runs this repository's ``Scheduler`` + ``CacheManager`` and the reference's ``Scheduler`` +
``BlockManager`` (engine/scheduler.py, engine/block_manager.py there) behind a small adapter each, with a fake model
whose next token is a function of the request's tokens so far.  What is recorded per step: the batch as
(request, tokens computed before, tokens scheduled), then, after the step's tokens are in, the free pages, the
preemptions so far and the block table of every running request.  ``tests/golden/scheduler_traces.json`` holds the
reference's records for ``CASES``; ``tests/test_scheduler_golden.py`` holds this repository's scheduler to them.
"""
from __future__ import annotations

import random

# (name, pages, page size, token budget, max requests at once, chunked prefill, long-prefill threshold, policy, seed)
CASES = [
    ("few_pages_fcfs", 9, 16, 24, 4, True, 0, "fcfs", 1),
    ("small_pages_fcfs", 14, 8, 16, 3, True, 0, "fcfs", 2),
    ("threshold_fcfs", 12, 16, 48, 5, True, 10, "fcfs", 3),
    ("few_pages_priority", 9, 16, 24, 4, True, 0, "priority", 4),
    ("prefill_first_fcfs", 10, 16, 80, 4, False, 0, "fcfs", 5),
    ("prefill_first_priority", 12, 8, 80, 3, False, 0, "priority", 6),
    ("roomy_fcfs", 64, 16, 64, 8, True, 0, "fcfs", 7),
]
MAX_MODEL_LEN = 80
EOS = 117


def fake_token(token_ids) -> int:
    return (sum(token_ids) * 31 + len(token_ids)) % 97 + 100


def workload(seed: int, page: int):
    """[(step at which the request is added, prompt, max_tokens, ignore_eos, priority)], sorted by step: prompts that
    share leading pages, some of them arriving while others run."""
    rng = random.Random(seed)
    shared = [rng.randrange(90) for _ in range(48)]
    out = []
    for i in range(16):
        n = rng.randint(1, 60)
        toks = (shared[:rng.choice([0, 0, page, 2 * page, 2 * page + 3, 40])] + [rng.randrange(90) for _ in range(n)])[:n]
        out.append((0 if i < 9 else rng.randint(1, 25), toks, rng.randint(1, 18), rng.random() < 0.7, rng.randint(0, 2)))
    return sorted(out, key=lambda r: r[0])


def run_case(case, make_adapter) -> list:
    """Drives one scheduler through ``case``; returns the record (a list of steps, JSON-ready)."""
    name, pages, page, budget, max_seqs, chunked, threshold, policy, seed = case
    adapter = make_adapter(num_pages=pages, page_size=page, budget=budget, max_seqs=max_seqs, chunked=chunked,
                           threshold=threshold, policy=policy, eos=EOS, max_model_len=MAX_MODEL_LEN)
    todo = workload(seed, page)
    index = {}                                   # the scheduler's own request id -> index in the workload
    record, step = [], 0
    while todo or not adapter.is_finished():
        while todo and todo[0][0] <= step:
            _, toks, max_tokens, ignore_eos, priority = todo.pop(0)
            rid = adapter.add(toks, max_tokens, ignore_eos, priority)       # None: refused
            record.append({"add": len(index) if rid is not None else -1})
            if rid is not None:
                index[rid] = len(index)
        if adapter.is_finished():
            step += 1
            continue
        batch = adapter.schedule()
        shape = [[index[adapter.id_of(s)], adapter.computed(s), adapter.scheduled(s)] for s in batch]
        tokens = [fake_token(adapter.tokens(s)) if adapter.samples(s) else None for s in batch]
        adapter.postprocess(batch, tokens)
        record.append({"batch": shape, "free": adapter.num_free_pages(), "preemptions": adapter.num_preemptions(),
                       "tables": sorted([index[adapter.id_of(s)], list(adapter.table(s))] for s in adapter.running()),
                       "waiting": [index[adapter.id_of(s)] for s in adapter.waiting()]})
        step += 1
        assert step < 5000
    return record
