"""Generation through the Python entry point against the plain implementation."""
import numpy as np
import pytest
import torch

import helpers
import plain_model
import plain_ops
from tiny_configs import ALL

pytestmark = pytest.mark.gpu


def _llm(name, dtype, **kw):
    from mini_engine_b200 import LLM
    args = dict(dtype=dtype, kvcache_block_size=helpers.config_of(name)[2], num_kvcache_blocks=64, max_num_seqs=8,
                max_num_batched_tokens=64, max_model_len=256)
    args.update(kw)
    return LLM(helpers.model_folder(name), **args)


def _check_greedy(name, dtype, prompt, tokens):
    """Every generated token is the plain implementation's argmax, or within the tolerance of it."""
    ref = helpers.plain_logits(name, list(prompt) + list(tokens))
    tol = 2 * helpers.TOL[dtype] * max(1.0, float(np.abs(ref).max()))
    for k, t in enumerate(tokens):
        row = ref[len(prompt) + k - 1]
        assert row[t] >= row.max() - tol, f"token {k}: {t} is not the plain argmax {row.argmax()}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "B!", "D!"])
def test_greedy_generation(name, dtype):
    from mini_engine_b200 import SamplingParams
    llm = _llm(name, dtype)
    lengths = (5, 17, 33, 9) if name == "A" else (3, 40, 21, 12)
    prompts = helpers.random_requests(helpers.config_of(name)[0]["vocab_size"], lengths, seed=2)
    out = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=8), use_tqdm=False)
    assert [len(o["token_ids"]) for o in out] == [8] * len(prompts)
    for p, o in zip(prompts, out):
        _check_greedy(name, dtype, p, o["token_ids"])
    if dtype == "float32":
        cfg, w = helpers.plain_weights(name)
        assert out[1]["token_ids"] == plain_model.greedy_generate(cfg, w, prompts[1], 8)
    llm.cache.check([])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_with_shared_prefix_and_small_budget(dtype):
    """Six prompts of 3 to 40 tokens, two sharing a 16-token prefix, portions under a budget of 24,
    temperature 0.7 with fixed seeds: every drawn token wins the race on the plain logits."""
    from mini_engine_b200 import SamplingParams
    name = "B"
    llm = _llm(name, dtype, max_num_batched_tokens=24)
    prompts = helpers.random_requests(ALL[name][0]["vocab_size"], (3, 40, 17, 29, 9, 33), seed=3)
    prompts[4] = prompts[1][:16] + prompts[4]
    sps = [SamplingParams(temperature=0.7, max_tokens=6, seed=100 + i, ignore_eos=True) for i in range(6)]
    out = llm.generate(prompts, sps, use_tqdm=False)
    assert llm.cache.num_prefix_hit_tokens >= 16                # the shared prefix was found, not computed again
    margin = 2 * helpers.TOL[dtype] / 0.7
    for i, (p, o) in enumerate(zip(prompts, out)):
        ref = helpers.plain_logits(name, list(p) + o["token_ids"])
        for k, t in enumerate(o["token_ids"]):
            pos = len(p) + k
            keys = plain_ops.sample_keys(torch.from_numpy(ref[pos - 1]), 0.7, 100 + i, pos)
            assert keys[t] >= keys.max() - margin, f"request {i} token {k}"
    # the same seeds give the same tokens whatever the batching
    llm2 = _llm(name, dtype, max_num_batched_tokens=64, max_num_seqs=2)
    out2 = llm2.generate(prompts, sps, use_tqdm=False)
    if dtype == "float32":
        assert [o["token_ids"] for o in out2] == [o["token_ids"] for o in out]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_tokens_behind_a_shared_prefix(dtype):
    """Weights under which the next token hangs on every key in the cache: requests that find their first pages in
    the cache (while the request that wrote them lives, and after it has ended) draw the plain implementation's
    tokens."""
    from mini_engine_b200 import SamplingParams
    name = "B!"
    vocab = helpers.config_of(name)[0]["vocab_size"]
    base, t1, t2, other = helpers.random_requests(vocab, (29, 7, 12, 40), seed=8)
    # Budget 40, three at a time: the first step holds all of request 0 and four tokens of request 1; request 2 is
    # admitted in the second step, while request 0 lives, and finds its three pages; request 3 comes when a request has
    # ended and finds two pages that may have been freed.
    prompts = [base + t1, other, base + t2, base[:17] + t1]
    sp = SamplingParams(temperature=0, max_tokens=8, ignore_eos=True)
    llm = _llm(name, dtype, max_num_batched_tokens=40, max_num_seqs=3)
    out = llm.generate(prompts, sp, use_tqdm=False)
    assert llm.cache.num_prefix_hit_tokens >= 24 + 16                       # 3 and 2 pages of 8 tokens
    for p, o in zip(prompts, out):
        _check_greedy(name, dtype, p, o["token_ids"])
    if dtype == "float32":
        cfg, w = helpers.plain_weights(name)
        for p, o in zip(prompts, out):
            assert o["token_ids"] == plain_model.greedy_generate(cfg, w, p, 8)
    off = _llm(name, dtype, max_num_batched_tokens=40, max_num_seqs=3, enable_prefix_caching=False)
    assert off.generate(prompts, sp, use_tqdm=False) == out or dtype == "bfloat16"
    assert off.cache.num_prefix_hit_tokens == 0


def test_running_out_of_pages_preempts_and_gives_the_same_tokens():
    from mini_engine_b200 import SamplingParams
    name = "A!"
    prompts = helpers.random_requests(helpers.config_of(name)[0]["vocab_size"], (40, 40, 25), seed=4)
    sp = SamplingParams(temperature=0, max_tokens=30, ignore_eos=True)
    roomy = _llm(name, "float32", num_kvcache_blocks=64).generate(prompts, sp, use_tqdm=False)
    tight = _llm(name, "float32", num_kvcache_blocks=7, max_num_batched_tokens=128)
    out = tight.generate(prompts, sp, use_tqdm=False)
    assert tight.scheduler.num_preemptions > 0
    assert [o["token_ids"] for o in out] == [o["token_ids"] for o in roomy]
    cfg, w = helpers.plain_weights(name)
    assert out[2]["token_ids"] == plain_model.greedy_generate(cfg, w, prompts[2], 30)
    tight.cache.check([])
    assert tight.cache.num_free_pages == [7]


def test_the_pool_is_sized_from_a_measured_step_when_no_page_count_is_given():
    from mini_engine_b200 import LLM, SamplingParams
    name = "B!"
    args = dict(dtype="bfloat16", kvcache_block_size=8, max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256)
    llm = LLM(helpers.model_folder(name), num_kvcache_blocks=-1, **args)
    sizing = llm.model_runner.pool_sizing
    assert llm.model_runner.num_pages == 4 * 256 // 8             # all that four requests of 256 tokens can ever fill
    assert llm.config.num_kvcache_blocks == llm.model_runner.num_pages
    assert sizing["work_prompts"] > 0 and sizing["graphs"] > 0 and sizing["budget"] > 0
    prompts = helpers.random_requests(helpers.config_of(name)[0]["vocab_size"], (40, 3, 21), seed=6)
    out = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=6), use_tqdm=False)
    for p, o in zip(prompts, out):
        _check_greedy(name, "bfloat16", p, o["token_ids"])
    with pytest.raises(RuntimeError, match="no device memory left"):
        LLM(helpers.model_folder(name), num_kvcache_blocks=-1, gpu_memory_utilization=1e-6, **args)


def test_request_too_large_is_refused():
    from mini_engine_b200 import SamplingParams
    llm = _llm("A", "float32", num_kvcache_blocks=4)
    with pytest.raises(ValueError):
        llm.generate([list(range(100))], SamplingParams(max_tokens=10), use_tqdm=False)
    with pytest.raises(ValueError, match="max_model_len"):
        llm.generate([list(range(250))], SamplingParams(max_tokens=10), use_tqdm=False)


def test_token_outside_the_vocabulary_is_reported():
    from mini_engine_b200 import SamplingParams
    llm = _llm("A", "float32")
    with pytest.raises(RuntimeError, match="vocabulary"):
        llm.generate([[1, 2, 100000]], SamplingParams(temperature=0, max_tokens=2), use_tqdm=False)


def test_add_request_and_step_surface():
    from mini_engine_b200 import SamplingParams
    llm = _llm("A", "float32")
    a = llm.add_request([1, 2, 3, 4, 5], SamplingParams(temperature=0, max_tokens=2))
    b = llm.add_request([9, 8, 7], SamplingParams(temperature=0, max_tokens=3), priority=1)
    finished, n_prefill, n_decode, emitted = llm.step()
    assert (n_prefill, n_decode, finished, sorted(emitted)) == (8, 0, [], [a, b])
    finished, n_prefill, n_decode, emitted = llm.step()
    assert n_decode == 2 and [f[0] for f in finished] == [a] and len(finished[0][1]) == 2
    while not llm.is_finished():
        finished, *_ = llm.step()
    assert finished[0][0] == b and len(finished[0][1]) == 3
    with pytest.raises(ValueError, match="tokenizer"):
        llm.add_request("some text", SamplingParams())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_of_the_host_change_nothing(dtype):
    """The engine launches the likely next decode step before it has read the current one's tokens.  With and
    without that, the same requests give the same tokens: with different lengths (requests drop out of the
    guessed batch), with an end-of-sequence token that ends requests unforeseen (their rows of the guessed step
    are ignored), and with a request that arrives while others decode (the guessed step is dropped)."""
    from mini_engine_b200 import SamplingParams
    name = "B!"                # the next token hangs on the token fed and on the cache: a neighbour's token shows
    vocab = helpers.config_of(name)[0]["vocab_size"]
    prompts = helpers.random_requests(vocab, (3, 40, 17, 29, 9), seed=5)
    lens = [12, 5, 20, 9, 16]

    def run(overlap, eos=None, late=None):
        llm = _llm(name, dtype, overlap_steps=overlap)
        if eos is not None:
            llm.scheduler.eos = eos
        sps = [SamplingParams(temperature=0.8 if i % 2 else 0.0, max_tokens=n, seed=7 + i, ignore_eos=eos is None)
               for i, n in enumerate(lens)]
        ids = [llm.add_request(p, sp) for p, sp in zip(prompts, sps)]
        done, steps = {}, 0
        while not llm.is_finished():
            out, _, _, _ = llm.step()
            steps += 1
            if late is not None and steps == late:
                ids.append(llm.add_request(prompts[0][::-1], SamplingParams(temperature=0, max_tokens=7)))
            done.update(dict(out))
        llm.cache.check([])
        return [done[i] for i in ids], llm

    plain, llm0 = run(False)
    ahead, llm1 = run(True)
    assert ahead == plain
    for i in (0, 2, 4):                                           # the greedy ones against the plain implementation
        _check_greedy(name, dtype, prompts[i], ahead[i])
    assert llm0.steps_ahead_used == 0 and llm1.steps_ahead_used > 5
    # an end-of-sequence token taken from the middle of a completion: requests now end where the host cannot foresee it
    k = next(k for k in range(4, len(plain[2])) if plain[2][k] not in plain[2][:k])
    eos = plain[2][k]
    plain_eos, _ = run(False, eos=eos)
    ahead_eos, llm2 = run(True, eos=eos)
    assert ahead_eos == plain_eos and len(plain_eos[2]) == k + 1
    assert any(len(plain_eos[i]) > k + 3 for i in (3, 4))         # a request behind it in the batch goes on
    _check_greedy(name, dtype, prompts[4], ahead_eos[4])
    # a request that arrives in the middle: the scheduler then wants a different step than the one guessed
    plain_late, _ = run(False, late=6)
    ahead_late, _ = run(True, late=6)
    assert ahead_late == plain_late and len(ahead_late) == 6
    # a request alone that ends on its end-of-sequence token: the step guessed behind its last one is dropped
    llm = _llm(name, dtype)
    llm.scheduler.eos = eos
    out = llm.generate([prompts[2]], SamplingParams(temperature=0.0, max_tokens=lens[2], seed=9), use_tqdm=False)
    assert out[0]["token_ids"] == plain_eos[2] and llm.steps_ahead_dropped == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_prompt_portions_replayed_from_a_graph_change_nothing(name, dtype):
    # one request's portions of equal size: the first runs eagerly, the second is captured, the others are replayed
    # (at other contexts than the captured one, past a window, on other pages); a second request reuses the graph
    from mini_engine_b200.cache.manager import CacheHolder
    from mini_engine_b200.engine.model_runner import ModelRunner, StepItem
    T, portions = 130, 3
    rng = np.random.default_rng(5)
    vocab = ALL[name][0]["vocab_size"]

    def run(graphs, prompts):
        runner = ModelRunner(helpers.model_folder(name), dtype=dtype, page_size=ALL[name][2], num_pages=64, max_num_seqs=4,
                             max_num_batched_tokens=256, max_model_len=512, use_cuda_graphs=graphs)
        cache = runner.make_cache_manager(False)
        rows = []
        for prompt in prompts:
            h = CacheHolder()
            assert cache.allocate(h, len(prompt))
            for k in range(portions):
                want = [T - 1] if k == portions - 1 else [0, T - 1]     # two shapes: each comes often enough to be captured
                out = runner.step([StepItem(h, prompt[k * T:(k + 1) * T], k * T, want)])
                rows.append(out.logits.float().cpu().numpy().copy())
            cache.free(h)
        runner.check_device_errors()
        return runner, rows

    prompts = [rng.integers(0, vocab, size=T * portions).tolist() for _ in range(3)]
    runner, got = run(True, prompts)
    assert runner.use_cuda_graphs and len(runner._prefill_graphs) == 2 and runner.graph_launches > 0
    _, eager = run(False, prompts)
    for a, b in zip(got, eager):
        assert np.array_equal(a, b)                                     # the same kernels on the same numbers
    ref = helpers.plain_logits(name, prompts[2])
    assert np.abs(got[-1][0] - ref[T * portions - 1]).max() <= helpers.TOL[dtype]


def test_prompt_graphs_are_few_and_the_oldest_goes_first():
    # more shapes than graphs are kept: the oldest is dropped, comes back by a new capture, and results stay the eager ones
    from mini_engine_b200.cache.manager import CacheHolder
    from mini_engine_b200.engine.model_runner import ModelRunner, StepItem
    name, dtype = "D", "bfloat16"
    vocab = ALL[name][0]["vocab_size"]
    rng = np.random.default_rng(9)
    sizes = [128, 129, 130, 131, 132, 133]
    prompts = {T: rng.integers(0, vocab, size=T).tolist() for T in sizes}

    def run(graphs):
        runner = ModelRunner(helpers.model_folder(name), dtype=dtype, page_size=ALL[name][2], num_pages=64, max_num_seqs=4,
                             max_num_batched_tokens=256, max_model_len=256, use_cuda_graphs=graphs)
        cache = runner.make_cache_manager(False)
        rows = []
        for T in sizes + sizes + sizes[:2] + sizes[:2]:
            h = CacheHolder()
            assert cache.allocate(h, T)
            rows.append(runner.step([StepItem(h, prompts[T], 0, [T - 1])]).logits.float().cpu().numpy().copy())
            cache.free(h)
        runner.check_device_errors()
        return runner, rows

    runner, got = run(True)
    assert len(runner._prefill_graphs) == runner.prefill_graph_max == 4
    assert list(runner._prefill_graphs)[-2:] == [(128, 1, False), (129, 1, False)]       # dropped, then captured anew
    _, eager = run(False)
    for a, b in zip(got, eager):
        assert np.array_equal(a, b)
