"""Plain PyTorch twins of the CUDA kernels, one per function of ``mini_engine_b200.ops``.

Same arguments as the kernels' wrappers, written from the reference's formulas and for
clarity only (loops over requests and heads).  Tests compare each kernel with its twin; the
twins take tensors on any device and compute in float32.
"""
from __future__ import annotations

import math

import numpy as np
import torch

ATTN_TILE_Q = 16
ATTN_TILE_SIZES = (8, 16, 32, 64, 128)
DECODE_PARTITION = 128


def check_attention_sizes(head_dim, num_heads, num_kv_heads):
    pass


def require_extension():
    pass


def embed(ids, table, out, err):
    # layers/embed_head.py:11
    out.copy_(table[ids.long()].float())


def add_rmsnorm(residual, delta, weight, eps, out, rows=None):
    # layers/layernorm.py:11-23
    if delta is not None and delta.dim() == 3:
        delta = delta.float().sum(0)
    if rows is None:
        if delta is not None:
            residual.add_(delta.float())
        x = residual
    else:
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
    var = x.pow(2).mean(-1, keepdim=True)
    out.copy_(((x * torch.rsqrt(var + eps)) * weight).to(out.dtype))


def silu_mul(x, out):
    # layers/activation.py:4-7
    g, u = x.float().chunk(2, dim=-1)
    out.copy_((torch.nn.functional.silu(g) * u).to(out.dtype))


def linear_partials(x, weight, workspace, name):
    return None


def decode_linear_takes(M, K, weight):
    return False


def linear(x, weight, out, epilogue="none", workspace=None, err=None):
    # layers/linear.py:26,45 (F.linear), float32 accumulate
    y = x.float() @ weight.float().T
    if epilogue == "silu_mul":
        g, u = y.chunk(2, dim=-1)
        y = torch.nn.functional.silu(g) * u
    out.copy_(y.to(out.dtype))


def qk_norm_rope_kv_write(qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, cos_sin,
                          positions, slot_mapping, pool, page_size, rotary_dim=None, layout="half_split"):
    # models/qwen3.py:34-36, layers/rotary_embedding.py:20-25, layers/attention.py:13-18
    T = qkv.shape[0]
    nh, nkv, d = num_heads, num_kv_heads, head_dim
    x = qkv.float().view(T, nh + 2 * nkv, d)
    q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]

    def norm(t, w):
        if w is None:
            return t
        return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)) * w

    def rope(t):
        # the first rd elements are rotated (their two halves paired), the rest pass through
        if cos_sin is None:
            return t
        rd = d if rotary_dim is None else rotary_dim
        cs = cos_sin[positions.long()]
        cos, sin = cs[:, None, : rd // 2], cs[:, None, rd // 2:]
        a, b, rest = t[..., : rd // 2], t[..., rd // 2:rd], t[..., rd:]
        return torch.cat((a * cos - b * sin, b * cos + a * sin, rest), dim=-1)

    q, k = rope(norm(q, q_weight)), rope(norm(k, k_weight))
    res = torch.cat((q, k, v), dim=1).reshape(T, -1).to(qkv.dtype)
    qkv.copy_(res)
    if slot_mapping is not None:
        keep = slot_mapping >= 0
        slots = slot_mapping[keep].long()
        page, off = slots // page_size, slots % page_size
        r3 = res.view(T, nh + 2 * nkv, d)
        pool[page, 0, :, off] = r3[keep][:, nh:nh + nkv]
        pool[page, 1, :, off] = r3[keep][:, nh + nkv:]


def paged_attention(qkv, out, num_heads, num_kv_heads, head_dim, pool, page_size, block_tables, meta,
                    scale, window):
    # layers/attention.py:21-40 restated per request: keys j <= start + i, j < L; csrc/paged_prefill.cu:200-203
    nh, nkv, d = num_heads, num_kv_heads, head_dim
    g = nh // nkv
    cu = meta.cu_seqlens.tolist()
    lens = meta.context_lens.tolist()
    for b in range(meta.num_reqs):
        t0, t1 = cu[b], cu[b + 1]
        n, L = t1 - t0, lens[b]
        if n == 0:
            continue
        if L == 0:
            out[t0:t1] = 0
            continue
        start = L - n
        q = qkv[t0:t1, : nh * d].float().view(n, nh, d)
        j = torch.arange(L, device=qkv.device)
        pages = block_tables[b].long()[j // page_size]
        ok = pages >= 0
        kv = pool[pages.clamp(min=0), :, :, j % page_size].float()      # [L, 2, nkv, d]
        kv = torch.where(ok[:, None, None, None], kv, torch.zeros_like(kv))
        p = start + torch.arange(n, device=qkv.device)
        seen = j[None, :] <= p[:, None]
        if window:
            seen &= j[None, :] > p[:, None] - window
        o = torch.empty(n, nh, d, dtype=torch.float32, device=qkv.device)
        for h in range(nh):
            s = (q[:, h] @ kv[:, 0, h // g].T) * scale
            s = s.masked_fill(~seen, float("-inf"))
            o[:, h] = torch.softmax(s, dim=-1) @ kv[:, 1, h // g]
        out[t0:t1] = o.reshape(n, nh * d).to(out.dtype)


def _mix32(x):
    x = x.astype(np.uint32)
    x ^= x >> np.uint32(16)
    x = (x * np.uint32(0x7FEB352D)).astype(np.uint32)
    x ^= x >> np.uint32(15)
    x = (x * np.uint32(0x846CA68B)).astype(np.uint32)
    x ^= x >> np.uint32(16)
    return x


def sample_keys(logits_row, temperature, seed, position):
    """The float64 keys whose argmax the sampler takes (layers/sampler.py:5-11 as a Gumbel race)."""
    x = logits_row.double().cpu().numpy()
    if temperature == 0:
        return x
    with np.errstate(over="ignore"):
        v = np.arange(x.shape[0], dtype=np.uint32)
        s = _mix32(np.asarray([seed & 0xFFFFFFFF], dtype=np.uint32) + np.uint32(0x9E3779B9))
        p = _mix32((s ^ np.uint32(position & 0xFFFFFFFF)) + np.uint32(0x85EBCA6B))
        h = _mix32((p ^ v) + np.uint32(0xC2B2AE35))
    u = ((h >> np.uint32(9)).astype(np.float64) + 0.5) / 8388608.0
    return x / temperature - np.log(-np.log(u))


def sample(logits, temperatures, seeds, positions, out, workspace=None):
    for r in range(logits.shape[0]):
        keys = sample_keys(logits[r], float(temperatures[r]), int(seeds[r]), int(positions[r]))
        out[r] = int(np.argmax(keys))
