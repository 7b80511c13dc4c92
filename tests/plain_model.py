"""A plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache.

Written from the reference's formulas (each function cites file:line in the reference
tree); it shares no code with ``mini_engine_b200``.  ``tests/golden/make_golden.py``
compared it once with the reference's own model code on the CPU (tiny random models); the
outputs of that run are committed under ``tests/golden/``.

Everything is float64 or float32 torch on the CPU.  ``window`` is not in the reference (all
its layers see every key); the rule used here is the engine's: a query at position p sees
keys j with p - window < j <= p.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch
from safetensors import safe_open


def load_folder(folder: str, dtype=torch.float32):
    """config.json as a dict and all tensors of *.safetensors by their disk names."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    for name in sorted(os.listdir(folder)):
        if name.endswith(".safetensors"):
            with safe_open(os.path.join(folder, name), "pt", device="cpu") as f:
                for k in f.keys():
                    tensors[k] = f.get_tensor(k).to(dtype)
    return cfg, tensors


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    # layers/layernorm.py:11-16: var = mean(x^2); x * rsqrt(var + eps); times weight
    var = x.pow(2).mean(-1, keepdim=True)
    return weight * (x * torch.rsqrt(var + eps))


def rope_tables(head_dim: int, num_positions: int, theta: float, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    # layers/rotary_embedding.py:13-18: inv_freq = 1/theta^(2i/d) in float32; freqs = outer(t, inv_freq);
    # cos/sin of cat(freqs, freqs)
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    t = torch.arange(num_positions).float()
    freqs = torch.outer(t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    # layers/rotary_embedding.py:5-8
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # layers/rotary_embedding.py:20-25; x [T, heads, d], cos/sin [T, d]
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """q [T, nh, d], k, v [T, nkv, d] of ONE request from position 0.

    layers/attention.py:54-59 (causal, scale, grouped heads: query head h reads kv head
    h // (nh / nkv), the consecutive grouping of ``enable_gqa``); softmax over keys j <= p."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.empty_like(q)
    pos = torch.arange(T, device=q.device)
    seen = pos[None, :] <= pos[:, None]
    if window is not None:
        seen &= pos[None, :] > pos[:, None] - window
    for h in range(nh):
        s = (q[:, h, :] @ k[:, h // g, :].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, h // g, :]
    return out


def attention_block(x, w, prefix, cfg, cos, sin, window):
    # models/qwen3.py:28-38: qkv projections, per-head q_norm / k_norm, rope, attention, o_proj
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).view(T, nh, d)
    k = (x @ w[prefix + "k_proj.weight"].T).view(T, nkv, d)
    v = (x @ w[prefix + "v_proj.weight"].T).view(T, nkv, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[prefix + "k_norm.weight"], cfg["rms_norm_eps"])
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, d ** -0.5, window)          # scale: models/qwen3.py:25
    return o.reshape(T, nh * d) @ w[prefix + "o_proj.weight"].T


def swiglu(x, w, prefix):
    # models/qwen3.py:50-51, layers/activation.py:4-7: down(silu(gate(x)) * up(x))
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    return (torch.nn.functional.silu(g) * u) @ w[prefix + "down_proj.weight"].T


def layer_windows(cfg) -> list[Optional[int]]:
    L = cfg["num_hidden_layers"]
    if not cfg.get("use_sliding_window", False):
        return [None] * L
    types = cfg.get("layer_types") or ["sliding_attention" if i >= cfg.get("max_window_layers", L)
                                       else "full_attention" for i in range(L)]
    return [cfg["sliding_window"] if t == "sliding_attention" else None for t in types]


def forward_logits(cfg: dict, w: dict, token_ids, dtype=torch.float64, device=None, positions=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence from position 0 (with ``positions``: of those rows only).

    models/qwen3.py:65-74,86-92 with the residual written the usual way (the reference defers
    each add into the next norm, layers/layernorm.py:19-23, which is the same sum).  ``device``: where the
    arithmetic runs (the same plain torch code; large layer sizes are slow on the host)."""
    w = {k: v.to(device=device, dtype=dtype) for k, v in w.items()}
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=device)
    T = ids.shape[0]
    theta = (cfg.get("rope_parameters") or {}).get("rope_theta", cfg.get("rope_theta"))
    cos, sin = rope_tables(cfg["head_dim"], T, theta, dtype)
    cos, sin = cos.to(device), sin.to(device)
    windows = layer_windows(cfg)
    r = w["model.embed_tokens.weight"][ids]                    # layers/embed_head.py:11
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = rms_norm(r, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        r = r + attention_block(x, w, p + "self_attn.", cfg, cos, sin, windows[i])
        x = rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        r = r + swiglu(x, w, p + "mlp.")
    h = rms_norm(r, w["model.norm.weight"], cfg["rms_norm_eps"])
    if positions is not None:                                  # layers/embed_head.py:19-23: rows gathered before the head
        h = h[torch.as_tensor(positions, dtype=torch.long, device=device)]
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return (h @ head.T).cpu()                                  # layers/embed_head.py:19-23


def greedy_generate(cfg, w, prompt, num_new: int, dtype=torch.float64) -> list[int]:
    """Greedy continuation by recomputing the whole sequence for every token (layers/sampler.py:7)."""
    ids = list(prompt)
    for _ in range(num_new):
        ids.append(int(forward_logits(cfg, w, ids, dtype)[-1].argmax()))
    return ids[len(prompt):]


def sample_row(logits: torch.Tensor, temperature: float, uniform) -> int:
    """layers/sampler.py:5-11 with given noise: argmax(softmax(logits/T) / E), E = -log(u)."""
    if temperature == 0:
        return int(logits.argmax())
    probs = torch.softmax(logits.double() / temperature, dim=-1)
    e = -torch.log(torch.as_tensor(uniform, dtype=torch.float64))
    return int((probs / e).argmax())
