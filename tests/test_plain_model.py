"""The plain implementation against the reference's own outputs (tests/golden) and itself (no GPU)."""
import os

import numpy as np
import pytest
import torch

import plain_model
from mini_engine_b200.weights import write_random_model
from tiny_configs import TINY_A, TINY_B, TINY_C

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_logits.npz")


@pytest.mark.parametrize("name, cfg, seed", [("A", TINY_A, 0), ("B", TINY_B, 1)])
def test_matches_reference_model_outputs(tmp_path, name, cfg, seed):
    gold = np.load(GOLDEN)
    folder = write_random_model(str(tmp_path), cfg, seed, dtype=torch.float32)
    c, w = plain_model.load_folder(folder)
    mine = plain_model.forward_logits(c, w, gold[f"ids_{name}"].tolist())
    assert np.abs(mine.numpy() - gold[f"logits_{name}"]).max() < 2e-6


def test_causality_and_window(tmp_path):
    folder = write_random_model(str(tmp_path), TINY_C, 2, dtype=torch.float32)
    c, w = plain_model.load_folder(folder)
    ids = list(range(7, 67))
    full = plain_model.forward_logits(c, w, ids)
    assert torch.allclose(plain_model.forward_logits(c, w, ids[:30]), full[:30], atol=1e-12)   # causal
    c2 = dict(c, use_sliding_window=False)
    no_win = plain_model.forward_logits(c2, w, ids)
    assert torch.allclose(no_win[:24], full[:24], atol=1e-12)      # the window (24) holds all keys so far
    assert (no_win[30:] - full[30:]).abs().max() > 1e-6            # later it does not


def test_attention_parts():
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 4, 8), torch.randn(5, 2, 8), torch.randn(5, 2, 8)
    o = plain_model.causal_attention(q, k, v, 0.5)
    assert torch.allclose(o[0, 3], v[0, 1])                       # first token sees itself only; head 3 -> kv head 1
    s = (q[2, 1] @ k[:3, 0].T) * 0.5
    assert torch.allclose(o[2, 1], torch.softmax(s, -1) @ v[:3, 0])
    ow = plain_model.causal_attention(q, k, v, 0.5, window=2)
    s = (q[4, 0] @ k[3:5, 0].T) * 0.5
    assert torch.allclose(ow[4, 0], torch.softmax(s, -1) @ v[3:5, 0])


def test_rope_and_norm_parts():
    x = torch.arange(8.0, dtype=torch.float64).view(1, 1, 8)
    cos, sin = plain_model.rope_tables(8, 3, 10000.0, torch.float64)
    assert torch.allclose(plain_model.apply_rope(x, cos[:1], sin[:1]), x)        # position 0: identity
    y = plain_model.apply_rope(x, cos[2:3], sin[2:3])
    assert torch.allclose(y.norm(), x.norm())                                     # a rotation
    assert abs(float(y[0, 0, 0]) - (0 * cos[2, 0] - 4 * sin[2, 0])) < 1e-12
    v = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(plain_model.rms_norm(v, torch.tensor([1.0, 2.0]), 0.0),
                          torch.tensor([[3 / 12.5 ** 0.5, 8 / 12.5 ** 0.5]]))
