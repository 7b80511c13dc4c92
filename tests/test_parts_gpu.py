"""Each part of a layer alone against the plain implementation, and the generality of the assembly:
a toy mixer with state of its own and a schedule that names a layer twice and lets a layer read another
layer's cache, registered from here without touching the framework's files."""
import json
import os
import tempfile
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_model
from tiny_configs import ALL

pytestmark = pytest.mark.gpu
DEV = os.environ.get("MINI_ENGINE_TEST_DEVICE", "cuda:0")


def _runner(name, dtype):
    from mini_engine_b200.engine.model_runner import ModelRunner
    return ModelRunner(helpers.model_folder(name), dtype=dtype, page_size=ALL[name][2], num_pages=32,
                       max_num_seqs=4, max_num_batched_tokens=256, max_model_len=256, use_cuda_graphs=False)


def _one_request_context(runner, n):
    from mini_engine_b200.cache.manager import CacheHolder
    from mini_engine_b200.engine.model_runner import StepItem
    cache = runner.make_cache_manager(False)
    h = CacheHolder()
    assert cache.allocate(h, n)
    runner.build_batch([StepItem(h, [0] * n, 0, [n - 1])], runner.ctx)
    return runner.ctx


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_parts_alone(name, dtype):
    runner = _runner(name, dtype)
    cfg, w = helpers.plain_weights(name)
    T, H = 50, cfg["hidden_size"]
    ctx = _one_request_context(runner, T)
    tol = {"float32": 2e-5, "bfloat16": 2e-2}[dtype]
    act = runner.act_dtype
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=g).to(act)
    xd = x.double()
    block = runner.model.blocks[1]
    p = "model.layers.1."
    # norm (with the residual sum folded in)
    res = torch.randn(T, H, generator=g)
    res_dev = res.clone().to(DEV)
    y = block.mixer_norm.forward(res_dev, x.to(DEV), ctx)
    want = plain_model.rms_norm(res.double() + xd, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    assert (y.double().cpu() - want).abs().max() < tol * 4
    assert torch.allclose(res_dev.cpu().double(), res.double() + xd, atol=1e-6)
    # mixer: attention over the cache, whole sequence from position 0
    theta = cfg["rope_theta"]
    cos, sin = plain_model.rope_tables(cfg["head_dim"], T, theta, torch.float64)
    win = plain_model.layer_windows(cfg)[1]
    want = plain_model.attention_block(xd, w, p + "self_attn.", cfg, cos, sin, win)
    got = block.mixer.forward(x.to(DEV), ctx, runner.model.schedule[1])
    assert (got.double().cpu() - want).abs().max() < tol
    # feed-forward
    want = plain_model.swiglu(xd, w, p + "mlp.")
    got = block.feed_forward.forward(x.to(DEV), ctx)
    assert (got.double().cpu() - want).abs().max() < tol
    # embedding and head
    ids = torch.randint(0, cfg["vocab_size"], (T,), dtype=torch.int32)
    got = runner.model.embed.forward(ids.to(DEV), ctx)
    assert torch.equal(got.cpu().double(), w["model.embed_tokens.weight"][ids.long()])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    got = runner.model.head.forward(x.to(DEV), ctx)
    assert got.dtype == torch.float32 and (got.double().cpu() - xd @ head.T).abs().max() < tol
    # the whole block
    res_dev = res.clone().to(DEV)
    got = block.forward(res_dev, None, ctx, runner.model.schedule[1])
    r = res.double()
    r = r + plain_model.attention_block(plain_model.rms_norm(r, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"]),
                                        w, p + "self_attn.", cfg, cos, sin, win)
    want = plain_model.swiglu(plain_model.rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"]), w, p + "mlp.")
    assert (got.double().cpu() - want).abs().max() < tol * 2
    assert (res_dev.double().cpu() - r).abs().max() < tol * 2


# ---- a toy architecture defined here -------------------------------------------------------------
def _register_toy():
    from mini_engine_b200.config import Architecture, ModelConfig, register_architecture
    from mini_engine_b200.parts import (Block, BlockSpec, FeedForward, LayerCall, Linear, Mixer, ModelPlan, PartSpec,
                                        PositionEncoding, SharedRef, StateNeed, register_block, register_feed_forward,
                                        register_mixer, register_position_encoding)

    class RunningMean(Mixer):
        """out[t] = mean over the request's tokens 0..t of proj(x): its state (a sum and a count) has a
        fixed size per request and lives in a state slot."""

        def __init__(self, hidden_size):
            super().__init__()
            self.h = hidden_size
            self.proj = Linear(hidden_size, [("proj.weight", hidden_size)], name="proj.weight")

        def sub_parts(self):
            return [("", self.proj)]

        def cache_needs(self):
            return [StateNeed((self.h + 1,), "float64")]         # sums over a whole request: kept in 64 bits

        def forward(self, x, ctx, call):
            y = self.proj.forward(x, ctx, "toy_proj").double()
            state = ctx.state(call.cache_slot)
            assert state.dtype == torch.float64
            out = torch.empty_like(y)
            t = 0
            for start, n, slot in zip(ctx.host.starts, ctx.host.lengths, ctx.host.state_slots):
                if start == 0:
                    state[slot] = 0
                cum = torch.cumsum(y[t:t + n], 0) + state[slot, :self.h]
                cnt = state[slot, self.h] + torch.arange(1, n + 1, device=y.device)
                out[t:t + n] = cum / cnt[:, None]
                state[slot, :self.h] = cum[-1]
                state[slot, self.h] += n
                t += n
            return out.to(ctx.act_dtype)

    class SoftExperts(FeedForward):
        """A feed-forward with routing: a router (float32 logits, softmax) weighs the outputs of small experts,
        ``sum_e p_e * down_e(silu(up_e(x)))``.  All experts run and the weights are soft, so the result is a
        continuous function of the input and can be compared with a plain implementation at a tolerance."""
        capturable = True

        def __init__(self, hidden_size, expert_size, num_experts):
            super().__init__()
            self.h, self.e = hidden_size, num_experts
            self.router = Linear(hidden_size, [("router.weight", num_experts)], name="router.weight")
            self.ups = [Linear(hidden_size, [(f"experts.{i}.up.weight", expert_size)], name=f"experts.{i}.up.weight")
                        for i in range(num_experts)]
            self.downs = [Linear(expert_size, [(f"experts.{i}.down.weight", hidden_size)], name=f"experts.{i}.down.weight")
                          for i in range(num_experts)]

        def sub_parts(self):
            return [("", self.router)] + [("", p) for p in self.ups + self.downs]

        def forward(self, x, ctx):
            logits = self.router.forward(x, ctx, "toy_router", out_dtype=torch.float32)
            probs = torch.softmax(logits.float(), dim=-1)
            out = torch.zeros(x.shape[0], self.h, dtype=torch.float32, device=x.device)
            for i in range(self.e):
                hid = self.ups[i].forward(x, ctx, f"toy_up{i}")
                act = torch.nn.functional.silu(hid.float()).to(ctx.act_dtype)
                out += probs[:, i:i + 1] * self.downs[i].forward(act, ctx, f"toy_down{i}").float()
            return out.to(ctx.act_dtype)

    class PostNormBlock(Block):
        """Another arrangement of a layer: ``r = norm(r + mixer(r)); r = norm(r + feed_forward(r))``, each place with a
        norm of its own.  Nothing is left pending: the stream holds the block's result when it returns."""

        def forward(self, residual, delta, ctx, call, upcoming=None):
            assert delta is None                                   # (every block of this toy model is of this kind)
            for norm, part, args in ((self.mixer_norm, self.mixer, (ctx, call)), (self.feed_forward_norm, self.feed_forward, (ctx,))):
                out = part.forward(residual.to(ctx.act_dtype), *args)
                residual.copy_(norm.forward(residual, out, ctx).float())
            return None

    class Interleaved(PositionEncoding):
        """A rotary table whose pairing of elements the kernels do not know: refused by name at the first step."""
        layout = "interleaved"

        def __init__(self, rotary_dim, max_position):
            super().__init__()
            self.rotary_dim, self.max_position = rotary_dim, max_position

        def finalize(self, dtype, device):
            self.cos_sin = torch.zeros(self.max_position, self.rotary_dim, device=device)

    class InterpolatedRotary(PositionEncoding):
        """Another position encoding: rotary angles of position / factor (the table is all the attention mixer asks for)."""
        capturable = True

        def __init__(self, rotary_dim, max_position, theta, factor):
            super().__init__()
            self.rotary_dim, self.max_position, self.theta, self.factor = rotary_dim, max_position, float(theta), float(factor)
            self.cos_sin = None

        def finalize(self, dtype, device):
            d = self.rotary_dim
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
            ang = torch.outer(torch.arange(self.max_position, dtype=torch.float32) / self.factor, inv_freq)
            self.cos_sin = torch.cat((ang.cos(), ang.sin()), dim=-1).contiguous().to(device)

    @dataclass
    class ToyConfig(ModelConfig):
        num_attention_heads: int = 0
        num_key_value_heads: int = 0
        head_dim: int = 0
        intermediate_size: int = 0
        rms_norm_eps: float = 1e-6
        rope_theta: float = 1e4
        pattern: str = ""

        @classmethod
        def from_dict(cls, raw):
            return cls(architecture=raw["architectures"][0], vocab_size=raw["vocab_size"], hidden_size=raw["hidden_size"],
                       num_hidden_layers=raw["num_hidden_layers"], max_position_embeddings=raw["max_position_embeddings"],
                       **{k: raw[k] for k in ("num_attention_heads", "num_key_value_heads", "head_dim", "intermediate_size",
                                              "rms_norm_eps", "rope_theta", "pattern")})

    def plan(cfg):
        norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
        ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
        attn = PartSpec("gqa_attention", {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
                                          "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                                          "qk_norm_eps": cfg.rms_norm_eps, "position_encoding": SharedRef("rope")})
        toy = PartSpec("toy_running_mean", {"hidden_size": cfg.hidden_size})
        blocks = [BlockSpec(mixer=toy if i % 2 else attn, feed_forward=ffn, norm=norm)
                  for i in range(cfg.num_hidden_layers)]
        rope = PartSpec("rope", {"rotary_dim": cfg.head_dim, "max_position": cfg.max_position_embeddings, "theta": cfg.rope_theta})
        if cfg.pattern == "postnorm":        # every layer arranged the other way round, with two different norms
            blocks = [BlockSpec(mixer=attn, feed_forward=ffn, kind="toy_post_norm",
                                mixer_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": 1e-3}),
                                feed_forward_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": 1e-6}))
                      for i in range(cfg.num_hidden_layers)]
            schedule = [LayerCall(i, i) for i in range(cfg.num_hidden_layers)]
        elif cfg.pattern in ("partial", "unknown_layout"):   # attention everywhere; half of each head is rotated
            blocks = [BlockSpec(mixer=attn, feed_forward=ffn, norm=norm) for i in range(cfg.num_hidden_layers)]
            rope = PartSpec("rope", dict(rope.args, rotary_dim=cfg.head_dim // 2))
            if cfg.pattern == "unknown_layout":
                rope = PartSpec("toy_interleaved", {"rotary_dim": cfg.head_dim // 2, "max_position": cfg.max_position_embeddings})
            schedule = [LayerCall(i, i) for i in range(cfg.num_hidden_layers)]
        elif cfg.pattern == "routed":          # attention everywhere with the other position encoding; every second feed-forward routed
            experts = PartSpec("toy_soft_experts", {"hidden_size": cfg.hidden_size, "expert_size": 24, "num_experts": 3})
            blocks = [BlockSpec(mixer=attn, feed_forward=experts if i % 2 else ffn, norm=norm) for i in range(cfg.num_hidden_layers)]
            rope = PartSpec("toy_interpolated_rope", dict(rope.args, factor=2.5))
            schedule = [LayerCall(i, i) for i in range(cfg.num_hidden_layers)]
        elif cfg.pattern == "state":         # attention, running mean, attention, running mean
            schedule = [LayerCall(i, i) for i in range(cfg.num_hidden_layers)]
        else:                                # "twice": layer 0, layer 2, layer 0 again (own cache), layer 2 reading call 1's cache
            schedule = [LayerCall(0, 0), LayerCall(2, 1), LayerCall(0, 2), LayerCall(2, 1, writes_cache=False)]
        return ModelPlan(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, blocks=blocks, schedule=schedule,
                         final_norm=norm, tie_word_embeddings=False, max_position=cfg.max_position_embeddings,
                         shared={"rope": rope})

    register_mixer("toy_running_mean", RunningMean, replace=True)
    register_feed_forward("toy_soft_experts", SoftExperts, replace=True)
    register_position_encoding("toy_interpolated_rope", InterpolatedRotary, replace=True)
    register_position_encoding("toy_interleaved", Interleaved, replace=True)
    register_block("toy_post_norm", PostNormBlock, replace=True)
    register_architecture(Architecture("ToyStateLM", ToyConfig.from_dict, plan), replace=True)


TOY = {"architectures": ["ToyStateLM"], "vocab_size": 200, "hidden_size": 48, "num_hidden_layers": 4,
       "max_position_embeddings": 256, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
       "intermediate_size": 80, "rms_norm_eps": 1e-5, "rope_theta": 1e4, "pattern": "state"}


def _toy_plain(cfg, w, ids):
    """Whole-sequence plain implementation of the toy architecture (float64)."""
    ids = torch.as_tensor(ids)
    T = len(ids)
    cos, sin = plain_model.rope_tables(cfg["head_dim"], T, cfg["rope_theta"], torch.float64)
    if cfg["pattern"] == "routed":
        inv = 1.0 / (cfg["rope_theta"] ** (torch.arange(0, cfg["head_dim"], 2, dtype=torch.float64) / cfg["head_dim"]))
        ang = torch.outer(torch.arange(T, dtype=torch.float64) / 2.5, inv)
        cos, sin = torch.cat((ang.cos(), ang.cos()), -1), torch.cat((ang.sin(), ang.sin()), -1)
    r = w["model.embed_tokens.weight"][ids]
    eps = cfg["rms_norm_eps"]
    rd = cfg["head_dim"] // 2 if cfg["pattern"] == "partial" else cfg["head_dim"]
    if cfg["pattern"] == "partial":
        cos, sin = plain_model.rope_tables(rd, T, cfg["rope_theta"], torch.float64)

    def rotate(t):                                       # the first rd elements of each head; the rest pass through
        return torch.cat((plain_model.apply_rope(t[..., :rd], cos, sin), t[..., rd:]), dim=-1)

    def attn(x, p, kv_from=None):
        nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        q = rotate(plain_model.rms_norm((x @ w[p + "q_proj.weight"].T).view(T, nh, d), w[p + "q_norm.weight"], eps))
        if kv_from is None:
            k = rotate(plain_model.rms_norm((x @ w[p + "k_proj.weight"].T).view(T, nkv, d), w[p + "k_norm.weight"], eps))
            v = (x @ w[p + "v_proj.weight"].T).view(T, nkv, d)
        else:
            k, v = kv_from
        o = plain_model.causal_attention(q, k, v, d ** -0.5)
        return o.reshape(T, nh * d) @ w[p + "o_proj.weight"].T, (k, v)

    def mean_mixer(x, p):
        y = x @ w[p + "proj.weight"].T
        return torch.cumsum(y, 0) / torch.arange(1, T + 1)[:, None]

    def soft_experts(x, p):
        probs = torch.softmax(x @ w[p + "router.weight"].T, dim=-1)
        return sum(probs[:, i:i + 1] * (torch.nn.functional.silu(x @ w[p + f"experts.{i}.up.weight"].T) @ w[p + f"experts.{i}.down.weight"].T)
                   for i in range(3))

    if cfg["pattern"] == "postnorm":
        for layer in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{layer}."
            r = plain_model.rms_norm(r + attn(r, p + "self_attn.")[0], w[p + "input_layernorm.weight"], 1e-3)
            r = plain_model.rms_norm(r + plain_model.swiglu(r, w, p + "mlp."), w[p + "post_attention_layernorm.weight"], 1e-6)
        return (plain_model.rms_norm(r, w["model.norm.weight"], eps) @ w["lm_head.weight"].T).numpy()
    if cfg["pattern"] in ("state", "routed", "partial"):
        calls = [(i, None) for i in range(cfg["num_hidden_layers"])]
    else:
        calls = [(0, None), (2, "write"), (0, None), (2, "read")]
    saved = None
    for layer, mode in calls:
        p = f"model.layers.{layer}."
        x = plain_model.rms_norm(r, w[p + "input_layernorm.weight"], eps)
        if layer % 2 and cfg["pattern"] not in ("routed", "partial"):
            m = mean_mixer(x, p + "self_attn.")
        else:
            m, kv = attn(x, p + "self_attn.", saved if mode == "read" else None)
            if mode == "write":
                saved = kv
        r = r + m
        x = plain_model.rms_norm(r, w[p + "post_attention_layernorm.weight"], eps)
        r = r + (soft_experts(x, p + "mlp.") if cfg["pattern"] == "routed" and layer % 2 else plain_model.swiglu(x, w, p + "mlp."))
    return (plain_model.rms_norm(r, w["model.norm.weight"], eps) @ w["lm_head.weight"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pattern", ["state", "twice", "routed", "postnorm", "partial", "partial64"])
def test_toy_architecture_is_registered_built_and_stepped(pattern, dtype):
    """Parts defined here, in the test (a mixer with state of its own, a feed-forward with routing, another position
    encoding) and orders of layers that name a layer twice or share a cache are registered, built from a model
    folder and stepped through the engine's replay without a change to the package."""
    _register_toy()
    from mini_engine_b200.engine.replay import TraceReplayer
    from mini_engine_b200.weights import write_random_model
    raw = dict(TOY, pattern=pattern)
    if pattern == "partial64":            # head size 64: bfloat16 single tokens would take the decode kernel that rotates
        raw.update(pattern="partial", head_dim=64)     # whole heads; with half a head rotated they take the separate pass
    folder = write_random_model(tempfile.mkdtemp(prefix="me_toy_"), raw, seed=9)
    cfg, w = plain_model.load_folder(folder, torch.float64)
    reqs = helpers.random_requests(raw["vocab_size"], (60, 45, 90, 38), seed=8)
    steps = helpers.trace_portions(reqs[:2]) + helpers.trace_mixed(reqs, max_live=3, seed=2, first_step=1000) \
        + helpers.trace_decode_tail(reqs[2:3], first_step=2000, tail=20)
    rp = TraceReplayer(folder, dtype, helpers.max_live_tokens(steps), page_size=16)
    if pattern == "state":
        assert rp.runner.state_needs and rp.cache.state_slots.num_slots > 0 and not rp.cache.prefix_caching
    elif pattern == "twice":
        assert len(rp.runner.model.slot_needs) == 3           # three cache slots for four calls
    elif pattern == "postnorm":
        assert type(rp.runner.model.blocks[0]).__name__ == "PostNormBlock" and rp.runner.model.blocks[0].mixer_norm.eps == 1e-3
    elif pattern.startswith("partial"):
        assert rp.runner.model.shared["rope"].rotary_dim == raw["head_dim"] // 2
    else:
        assert rp.runner.use_cuda_graphs == (rp.runner.device.type == "cuda")     # these toy parts may be captured
    got = helpers.collect(steps, [rp.run_step(st) for st in steps])
    rp.cache.check([])
    tol = helpers.TOL[dtype]
    for tag, sub in (("p", reqs[:2]), ("m", reqs), ("d", reqs[2:3])):
        for i, r in enumerate(sub):
            ref = _toy_plain(cfg, w, r)
            diff = np.abs(got[f"{tag}{i}"] - ref).max(axis=1)
            assert diff.max() <= tol, f"{pattern} {tag}{i}: first wrong token at {int(np.argmax(diff > tol))} ({diff.max():.3e})"


def test_a_rotary_layout_the_kernels_do_not_know_is_refused_by_name():
    _register_toy()
    from mini_engine_b200 import ops
    from mini_engine_b200.engine.replay import TraceReplayer
    from mini_engine_b200.weights import write_random_model
    folder = write_random_model(tempfile.mkdtemp(prefix="me_toy_"), dict(TOY, pattern="unknown_layout"), seed=9)
    rp = TraceReplayer(folder, "float32", 64, page_size=16)
    with pytest.raises(ops.KernelError, match="rotary layout 'interleaved' is not supported"):
        rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": []})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_mixer_with_state_through_the_engine(dtype):
    """The running-mean mixer through ``LLM.generate``: portions under a small budget, several requests, one ending
    unforeseen on its end-of-sequence token.  The engine launches no step ahead of the host for such a model (a
    dropped guess would advance the state twice), so the tokens are the plain implementation's either way."""
    _register_toy()
    from mini_engine_b200 import LLM, SamplingParams
    from mini_engine_b200.weights import write_random_model
    raw = dict(TOY, pattern="state")
    folder = write_random_model(tempfile.mkdtemp(prefix="me_toy_"), raw, seed=9, matrix_std=0.1)
    cfg, w = plain_model.load_folder(folder, torch.float64)
    prompts = helpers.random_requests(raw["vocab_size"], (30, 7, 19), seed=4)

    def plain_greedy(p, n, eos=None):
        ids = list(p)
        for _ in range(n):
            ids.append(int(_toy_plain(cfg, w, ids)[-1].argmax()))
            if ids[-1] == eos:
                break
        return ids[len(p):]
    want = [plain_greedy(p, 10) for p in prompts]
    i, k = next((i, k) for k in range(2, 9) for i in range(3) if want[i][k] not in want[i][:k])
    eos = want[i][k]                                   # request i ends on it, unforeseen, while others go on
    want = [plain_greedy(p, 10, eos) for p in prompts]
    assert len(want[i]) == k + 1 and max(len(x) for x in want) > k + 1
    outs = []
    for overlap in (True, False):
        llm = LLM(folder, dtype=dtype, kvcache_block_size=16, num_kvcache_blocks=32, max_num_seqs=4, max_num_batched_tokens=16,
                  max_model_len=128, overlap_steps=overlap)
        llm.scheduler.eos = eos
        out = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=10), use_tqdm=False)
        assert llm.steps_ahead_used == 0 and llm.steps_ahead_dropped == 0
        outs.append([o["token_ids"] for o in out])
    assert outs[0] == outs[1]
    if dtype == "float32":
        assert outs[0] == want
