"""The engine's request loop with a fake model runner (no GPU): steps launched ahead of the host.

The fake draws a token that depends strongly on the token it is fed and on its position, and resolves a token
id ``~j`` through its own ``token_feedback`` exactly as the embedding kernel does.  A step that is fed another
request's token therefore changes every token behind it, and the fake also records what each (request,
position) was fed, so the test can say where a wrong token first went in.
"""
import tempfile

import pytest
import torch

from mini_engine_b200.cache import CacheManager, GroupSpec
from mini_engine_b200.engine.llm_engine import LLMEngine
from mini_engine_b200.engine.model_runner import StepResult
from mini_engine_b200.sampling import SamplingParams
from mini_engine_b200.weights import write_random_model

VOCAB = 211
CFG = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 32, "num_hidden_layers": 1, "num_attention_heads": 2,
       "num_key_value_heads": 1, "head_dim": 16, "intermediate_size": 48, "vocab_size": VOCAB, "rope_theta": 10000.0,
       "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 256}


@pytest.fixture(scope="module")
def folder():
    return write_random_model(tempfile.mkdtemp(prefix="me_loop_"), CFG, seed=0)


def next_token(fed: int, position: int) -> int:
    return (fed * 37 + position * 11 + 5) % VOCAB


class FakeRunner:
    """ModelRunner's surface as the engine uses it, on the host."""

    def __init__(self, max_num_seqs=8, num_pages=64, page_size=16, state=False):
        self.device = torch.device("cpu")
        self.num_pages, self.page_size = num_pages, page_size
        self.error_flag = torch.zeros(4, dtype=torch.int32)
        self.result_dev = torch.zeros(4 + max_num_seqs, dtype=torch.int32)
        self.token_feedback = self.result_dev[4:]
        self.state_needs = {0: object()} if state else {}
        self.last_h2d_bytes = 0
        self.fed = {}                      # (holder id, position) -> every token that was fed there, in order
        self.steps = 0

    def make_cache_manager(self, enable_prefix_caching=True):
        return CacheManager([GroupSpec(None, 1, 16, (0,))], self.num_pages, self.page_size,
                            enable_prefix_caching=enable_prefix_caching)

    def step(self, items, sample=False):
        self.steps += 1
        drawn = []
        feedback = self.token_feedback.clone()          # what the device holds while this step runs
        for it in items:
            toks = [int(feedback[~t]) if t < 0 else int(t) for t in it.tokens]
            for k, t in enumerate(toks):
                self.fed.setdefault((id(it.holder), it.start + k), []).append(t)
            for w in it.want:
                drawn.append(next_token(toks[w], it.start + w))
        return StepResult(None, torch.tensor(drawn, dtype=torch.int32))

    def check_device_errors(self):
        pass


def run(folder, overlap, prompts, max_tokens, eos=None, state=False):
    runner = FakeRunner(state=state)
    llm = LLMEngine(folder, model_runner=runner, kvcache_block_size=16, num_kvcache_blocks=64, max_num_seqs=8,
                    max_num_batched_tokens=64, max_model_len=256, overlap_steps=overlap)
    if eos is not None:
        llm.scheduler.eos = eos
    sps = [SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=eos is None) for n in max_tokens]
    seqs = {}
    real_add = llm.scheduler.add

    def add(seq):
        seqs[seq.seq_id] = seq
        real_add(seq)
    llm.scheduler.add = add
    out = llm.generate(prompts, sps, use_tqdm=False)
    llm.cache.check([])
    return [o["token_ids"] for o in out], llm, runner, seqs


def expected(prompt, n, eos=None):
    toks = list(prompt)
    for _ in range(n):
        toks.append(next_token(toks[-1], len(toks) - 1))
        if eos is not None and toks[-1] == eos:
            break
    return toks[len(prompt):]


PROMPTS = [[3, 1, 4], [1, 5, 9, 2, 6], [5, 3], [5, 8, 9, 7, 9, 3], [2, 3, 8]]
LENS = [14, 9, 20, 12, 17]


@pytest.mark.parametrize("overlap", [False, True])
def test_every_request_continues_from_its_own_token(folder, overlap):
    got, llm, runner, seqs = run(folder, overlap, PROMPTS, LENS)
    assert got == [expected(p, n) for p, n in zip(PROMPTS, LENS)]
    assert (llm.steps_ahead_used > 5) == overlap


def test_a_request_that_ends_on_eos_in_the_middle_of_the_batch_leaves_its_neighbours_alone(folder):
    """Request 1 ends unforeseen on its end-of-sequence token while steps are launched ahead; the step that was
    guessed behind its last one is kept for the others, whose rows in the device's result are then no longer their
    indices in the batch.  Every token fed at every position must be the request's own."""
    eos = expected(PROMPTS[1], LENS[1])[4]
    want = [expected(p, n, eos) for p, n in zip(PROMPTS, LENS)]
    assert len(want[1]) == 5 and sum(len(w) > 8 for w in want[2:]) >= 2       # requests behind it go on for a while
    got, llm, runner, seqs = run(folder, True, PROMPTS, LENS, eos=eos)
    assert llm.steps_ahead_used > 5
    for seq in seqs.values():
        for pos in range(seq.num_prompt_tokens, len(seq.token_ids) - 1):
            fed = runner.fed[(id(seq), pos)]
            assert fed[-1] == seq.token_ids[pos], (f"request {seq.seq_id}: position {pos} was fed {fed}, "
                                                   f"its own token is {seq.token_ids[pos]}")
    assert got == want


def test_no_step_is_launched_ahead_for_a_model_with_state_of_its_own(folder):
    """A dropped guess would have advanced such a state once too often."""
    got, llm, runner, _ = run(folder, True, PROMPTS, LENS, state=True)
    assert got == [expected(p, n) for p, n in zip(PROMPTS, LENS)]
    assert llm.steps_ahead_used == 0 and llm.steps_ahead_dropped == 0
    for (_, pos), fed in runner.fed.items():
        assert len(fed) == 1                   # nothing was computed twice
