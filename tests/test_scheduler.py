"""The scheduler's decisions with a fake runner (no GPU)."""
import random
from types import SimpleNamespace

import pytest

from mini_engine_b200.cache import CacheManager, GroupSpec
from mini_engine_b200.engine.scheduler import Scheduler
from mini_engine_b200.engine.sequence import Sequence, SequenceStatus
from mini_engine_b200.sampling import SamplingParams

FULL = GroupSpec(None, 2, 16, (0,))
WIN = GroupSpec(24, 2, 16, (1,))


def make(num_pages=64, page=16, budget=64, max_seqs=8, chunked=True, threshold=0, policy="fcfs", eos=-1,
         max_len=4096, groups=(FULL,), prefix=True):
    cfg = SimpleNamespace(max_num_seqs=max_seqs, max_num_batched_tokens=budget, long_prefill_token_threshold=threshold,
                          enable_chunked_prefill=chunked, scheduling_policy=policy, eos=eos, max_model_len=max_len)
    cache = CacheManager(list(groups), num_pages, page, enable_prefix_caching=prefix)
    return Scheduler(cfg, cache), cache


def fake_token(seq):                     # what a model would say: a function of the tokens so far
    return (sum(seq.token_ids) * 31 + len(seq.token_ids)) % 97 + 100


def run_step(s):
    batch = s.schedule()
    shape = [(q.seq_id, q.num_computed_tokens, q.num_scheduled_tokens) for q in batch]
    toks = [fake_token(q) if q.samples_this_step else None for q in batch]
    s.postprocess(batch, toks)
    return shape


def seq(n, max_tokens=4, base=0, **kw):
    return Sequence([base + i for i in range(n)], SamplingParams(temperature=0, max_tokens=max_tokens, **kw))


def test_refuses_requests_that_can_never_run():
    s, _ = make(num_pages=4, max_len=100)
    with pytest.raises(ValueError, match="max_model_len"):
        s.add(seq(99, max_tokens=2))
    with pytest.raises(ValueError, match="pages"):
        s.add(seq(60, max_tokens=8))                     # 68 tokens = 5 pages > 4
    s.add(seq(60, max_tokens=4))


def test_prompt_is_cut_under_the_budget_and_decodes_go_first():
    s, _ = make(budget=24)
    a, b = seq(37), seq(9, base=1000)
    s.add(a), s.add(b)
    assert run_step(s) == [(a.seq_id, 0, 24)]                                  # cut where the budget ends
    assert run_step(s) == [(a.seq_id, 24, 13), (b.seq_id, 0, 9)]               # rest + next admitted
    assert a.num_completion_tokens == 1 and b.num_completion_tokens == 1
    assert run_step(s) == [(a.seq_id, 37, 1), (b.seq_id, 9, 1)]                # both decode
    c = seq(30, base=2000)
    s.add(c)
    assert run_step(s) == [(a.seq_id, 38, 1), (b.seq_id, 10, 1), (c.seq_id, 0, 22)]   # decodes first, then the budget's rest
    shape = run_step(s)
    assert shape[0] == (c.seq_id, 22, 8) or shape[-1] == (c.seq_id, 22, 8)


def test_long_prefill_threshold_caps_a_portion():
    s, _ = make(budget=64, threshold=10)
    a = seq(25)
    s.add(a)
    assert [run_step(s)[0][2] for _ in range(3)] == [10, 10, 5]


def test_finishes_at_max_tokens_and_on_eos_and_frees_pages():
    s, cache = make(eos=None)
    a = seq(20, max_tokens=3)
    s.add(a)
    while not s.is_finished():
        run_step(s)
    assert a.status == SequenceStatus.FINISHED and a.num_completion_tokens == 3
    assert cache.num_free_pages == [64]
    b = seq(5, max_tokens=50)
    s.eos = fake_token(b)                                 # the first sampled token is EOS
    s.add(b)
    run_step(s)
    assert b.is_finished and b.num_completion_tokens == 1
    c = seq(5, max_tokens=3, ignore_eos=True)
    s.eos = fake_token(c)
    s.add(c)
    while not s.is_finished():
        run_step(s)
    assert c.num_completion_tokens == 3


def test_head_of_line_admission_stops_at_max_num_seqs():
    s, _ = make(max_seqs=2, budget=64)
    qs = [seq(4, max_tokens=2, base=100 * i) for i in range(3)]
    for q in qs:
        s.add(q)
    assert [x[0] for x in run_step(s)] == [qs[0].seq_id, qs[1].seq_id]
    assert [x[0] for x in run_step(s)] == [qs[0].seq_id, qs[1].seq_id]        # both finish here (2 tokens)
    assert [x[0] for x in run_step(s)] == [qs[2].seq_id]


def test_pages_run_out_newest_is_preempted_and_recomputed():
    # 6 pages of 16: two requests of 40 tokens fill them; decoding past a page edge preempts the newest
    s, cache = make(num_pages=6, budget=128)
    a, b = seq(40, max_tokens=30, base=0), seq(40, max_tokens=30, base=500)
    s.add(a), s.add(b)
    run_step(s)
    assert cache.num_free_pages == [0]
    while s.num_preemptions == 0:                         # a's token at position 48 needs a 4th page
        run_step(s)
    assert s.num_preemptions == 1 and a.num_tokens == 50
    assert b.status == SequenceStatus.WAITING and s.waiting[0] is b and b.block_tables == [[]]
    assert b.num_computed_tokens == 0 and b.num_completion_tokens > 0          # keeps its tokens, loses its pages
    generated_before = list(b.completion_token_ids)
    while not s.is_finished():
        run_step(s)
        cache.check([q for q in (a, b) if not q.is_finished])
    assert b.completion_token_ids[:len(generated_before)] == generated_before
    assert a.num_completion_tokens == 30 and b.num_completion_tokens == 30
    assert cache.num_free_pages == [6]
    # the same requests without memory pressure give the same tokens (the fake model is a function of the tokens)
    s2, _ = make(num_pages=64, budget=128)
    a2, b2 = seq(40, max_tokens=30, base=0), seq(40, max_tokens=30, base=500)
    s2.add(a2), s2.add(b2)
    while not s2.is_finished():
        run_step(s2)
    assert a2.completion_token_ids == a.completion_token_ids and b2.completion_token_ids == b.completion_token_ids


def test_no_admission_in_a_step_that_preempted():
    s, cache = make(num_pages=6, budget=128)
    a, b = seq(47, max_tokens=30), seq(40, max_tokens=30, base=500)
    s.add(a), s.add(b)
    run_step(s)                                           # a: 3 pages, b: 3 pages
    run_step(s)                                           # a -> 48 tokens computed... next token needs page 4
    c = seq(3, base=900)
    s.add(c)
    shape = run_step(s)
    assert s.num_preemptions == 1 and [x[0] for x in shape] == [a.seq_id]      # b preempted, c not admitted now
    assert s.waiting[0] is b and s.waiting[1] is c


def test_self_preemption_when_alone():
    s, cache = make(num_pages=2, budget=128, max_len=200)
    a = seq(30, max_tokens=2)
    s.add(a)
    run_step(s)
    assert a.num_completion_tokens == 1
    run_step(s)
    assert a.is_finished


def test_prefix_hits_shorten_the_first_portion():
    s, cache = make(budget=128)
    a = seq(40, max_tokens=2)
    s.add(a)
    run_step(s), run_step(s)
    assert a.is_finished
    b = Sequence(list(range(32)) + [7, 7, 7], SamplingParams(temperature=0, max_tokens=2))
    s.add(b)
    assert run_step(s) == [(b.seq_id, 32, 3)]             # two full pages found again
    assert b.num_cached_tokens == 32


def test_priority_policy_orders_waiting_and_picks_the_worst_victim():
    s, cache = make(num_pages=6, budget=128, policy="priority")
    lo = Sequence(list(range(40)), SamplingParams(temperature=0, max_tokens=30), priority=5)
    hi = Sequence(list(range(500, 540)), SamplingParams(temperature=0, max_tokens=30), priority=0)
    s.add(lo), s.add(hi)
    assert s.waiting[0] is hi                              # better priority first
    run_step(s)
    while s.num_preemptions == 0:
        run_step(s)
    assert lo.status == SequenceStatus.WAITING and hi.status == SequenceStatus.RUNNING


def test_prefill_first_mode():
    s, _ = make(chunked=False, budget=64)
    a, b = seq(30, max_tokens=3), seq(40, base=100, max_tokens=3)
    s.add(a), s.add(b)
    assert run_step(s) == [(a.seq_id, 0, 30)]              # whole prompts only: 30 + 40 > 64
    assert run_step(s) == [(b.seq_id, 0, 40)]              # admission before decoding
    assert run_step(s) == [(a.seq_id, 30, 1), (b.seq_id, 40, 1)]


def test_window_group_pages_come_back_while_running():
    s, cache = make(num_pages=12, budget=32, groups=(FULL, WIN), max_len=300)
    a = seq(100, max_tokens=20)
    s.add(a)
    while not s.is_finished():
        run_step(s)
        if not a.is_finished:
            assert sum(1 for p in a.block_tables[1] if p >= 0) <= 5          # window 24 + portion 32 -> few pages
        cache.check([a] if not a.is_finished else [])
    assert cache.num_free_pages == [12, 12]


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_finish_with_all_pages_back(seed):
    rng = random.Random(seed)
    groups = (FULL,) if seed % 2 == 0 else (FULL, WIN)
    s, cache = make(num_pages=rng.randint(8, 14), page=rng.choice([8, 16]), budget=rng.choice([16, 24, 48]),
                    max_seqs=rng.randint(2, 5), groups=groups, max_len=150)
    shared = [rng.randrange(90) for _ in range(40)]
    reqs = []
    for i in range(14):
        n = rng.randint(1, 60)
        toks = (shared[:rng.randint(0, 40)] + [rng.randrange(90) for _ in range(n)])[:n]
        q = Sequence(toks, SamplingParams(temperature=0, max_tokens=rng.randint(1, 30), ignore_eos=True))
        try:
            s.add(q)
            reqs.append(q)
        except ValueError:
            pass
    expect = {}
    for q in reqs:                                          # what the fake model would generate without pressure
        ids = list(q.token_ids)
        for _ in range(q.sampling_params.max_tokens):
            ids.append((sum(ids) * 31 + len(ids)) % 97 + 100)
        expect[q.seq_id] = ids[q.num_prompt_tokens:]
    steps = 0
    while not s.is_finished():
        shape = run_step(s)
        assert sum(n for _, _, n in shape) <= s.max_num_batched_tokens
        assert len(s.running) <= s.max_num_seqs
        cache.check([q for q in reqs if q.block_tables and any(q.block_tables)])
        steps += 1
        assert steps < 5000
    for q in reqs:
        assert q.completion_token_ids == expect[q.seq_id]
    assert cache.num_free_pages == [p.num_pages for p in cache.pools]
