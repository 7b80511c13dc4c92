"""This repository's scheduler and cache manager against the reference's own decisions.

``tests/golden/scheduler_traces.json`` was made by running the reference's ``Scheduler`` / ``BlockManager`` on the
CPU (``tests/golden/make_scheduler_golden.py``) over random workloads with few pages, small token budgets, shared
prefixes, late arrivals, both modes and both policies.  Every step must agree: the batch as (request, computed,
scheduled), the free pages, the preemptions, every running request's block table (page numbers included: fresh
pages come from the front of the free list, released ones go to its back) and the waiting queue.  Where the
reference tree is at hand (``$MINI_ENGINE_REF``) it is also run live beside the stored records.
"""
import json
import os
import sys
from types import SimpleNamespace

import pytest

import scheduler_trace
from mini_engine_b200.cache import CacheManager, GroupSpec
from mini_engine_b200.engine.scheduler import Scheduler
from mini_engine_b200.engine.sequence import Sequence
from mini_engine_b200.sampling import SamplingParams

HERE = os.path.dirname(os.path.abspath(__file__))


class OursAdapter:
    def __init__(self, num_pages, page_size, budget, max_seqs, chunked, threshold, policy, eos, max_model_len):
        cfg = SimpleNamespace(max_num_seqs=max_seqs, max_num_batched_tokens=budget, long_prefill_token_threshold=threshold,
                              enable_chunked_prefill=chunked, scheduling_policy=policy, eos=eos, max_model_len=max_model_len)
        self.cache = CacheManager([GroupSpec(None, 2, 16, (0,))], num_pages, page_size, enable_prefix_caching=True)
        self.s = Scheduler(cfg, self.cache)

    def add(self, toks, max_tokens, ignore_eos, priority):
        seq = Sequence(list(toks), SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=ignore_eos), priority)
        try:
            self.s.add(seq)
        except ValueError:
            return None
        return seq.seq_id

    def is_finished(self): return self.s.is_finished()
    def schedule(self): return self.s.schedule()
    def postprocess(self, batch, tokens): self.s.postprocess(batch, tokens)
    def id_of(self, q): return q.seq_id
    def computed(self, q): return q.num_computed_tokens
    def scheduled(self, q): return q.num_scheduled_tokens
    def samples(self, q): return q.samples_this_step
    def tokens(self, q): return q.token_ids
    def table(self, q): return q.block_tables[0]
    def running(self): return self.s.running
    def waiting(self): return list(self.s.waiting)
    def num_free_pages(self): return self.cache.num_free_pages[0]
    def num_preemptions(self): return self.s.num_preemptions


def _first_difference(mine, theirs):
    for k, (a, b) in enumerate(zip(mine, theirs)):
        if a != b:
            return f"record {k}: ours {a} != reference {b}"
    if len(mine) != len(theirs):
        return f"{len(mine)} records, the reference has {len(theirs)}"
    return None


with open(os.path.join(HERE, "golden", "scheduler_traces.json")) as f:
    GOLDEN = json.load(f)


@pytest.mark.parametrize("case", scheduler_trace.CASES, ids=[c[0] for c in scheduler_trace.CASES])
def test_decisions_agree_with_the_reference_record(case):
    theirs = GOLDEN[case[0]]
    mine = json.loads(json.dumps(scheduler_trace.run_case(case, OursAdapter)))
    assert _first_difference(mine, theirs) is None
    steps = [r for r in theirs if "batch" in r]
    assert len(steps) > 20


def test_the_records_cover_what_they_should():
    recs = {name: [r for r in rec if "batch" in r] for name, rec in GOLDEN.items()}
    assert sum(r[-1]["preemptions"] > 0 for r in recs.values()) >= 3                  # pages ran out
    assert any(len(st["batch"]) > 1 and any(n > 1 for _, _, n in st["batch"]) and any(n == 1 for _, _, n in st["batch"])
               for r in recs.values() for st in r)                                     # portions beside decoded tokens
    assert any(c > 0 and c % 8 == 0 and n > 0 for r in recs.values() for st in r
               for i, c, n in st["batch"] if not any(i == j for prev in r[:r.index(st)] for j, _, _ in prev["batch"]))   # a first portion behind a prefix hit


@pytest.mark.skipif(not os.environ.get("MINI_ENGINE_REF"), reason="the reference tree is not at hand ($MINI_ENGINE_REF)")
@pytest.mark.parametrize("case", scheduler_trace.CASES, ids=[c[0] for c in scheduler_trace.CASES])
def test_decisions_agree_with_the_reference_run_live(case):
    sys.path.insert(0, os.path.join(HERE, "golden"))
    from make_scheduler_golden import reference_adapter_factory
    theirs = scheduler_trace.run_case(case, reference_adapter_factory(os.environ["MINI_ENGINE_REF"]))
    assert json.loads(json.dumps(theirs)) == GOLDEN[case[0]]                          # the stored record is the reference's
    mine = scheduler_trace.run_case(case, OursAdapter)
    assert _first_difference(json.loads(json.dumps(mine)), json.loads(json.dumps(theirs))) is None
