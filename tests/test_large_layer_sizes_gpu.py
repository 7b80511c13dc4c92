"""The engine at the layer sizes of Qwen3-8B and Qwen3-32B (one layer, small vocabulary), against the plain
implementation: products with K up to 25,600 (many split-K partial results), groups of 4 and 8 query heads,
hidden sizes that are no power of two."""
import tempfile

import numpy as np
import pytest
import torch

import helpers
import plain_model
from mini_engine_b200.weights import write_random_model

pytestmark = pytest.mark.gpu

SIZES = {
    "8B": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288),
    "32B": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128, intermediate_size=25600),
}


@pytest.mark.parametrize("name", ["8B", "32B"])
def test_one_layer_of_a_large_model(name):
    from mini_engine_b200.engine.replay import TraceReplayer
    cfg = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=1, vocab_size=1000, rope_theta=1e6, rms_norm_eps=1e-6,
               tie_word_embeddings=False, max_position_embeddings=512, **SIZES[name])
    folder = write_random_model(tempfile.mkdtemp(prefix="me_large_"), cfg, seed=4)
    c, w = plain_model.load_folder(folder, torch.float32)
    (ids,) = helpers.random_requests(1000, (150,), seed=6)
    ref = plain_model.forward_logits(c, w, ids, dtype=torch.float32).numpy()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:130], "want": list(range(130))}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[130:147], "want": list(range(17))}], "end": []}]
    steps += [{"step": 2 + k, "entries": [{"id": "a", "tokens": [ids[147 + k]], "want": [0]}], "end": ["a"] if k == 2 else []}
              for k in range(3)]
    for dtype, tol in (("bfloat16", 4e-2), ("float32", 2e-4)):
        rp = TraceReplayer(folder, dtype, 256)
        got = helpers.collect(steps, [rp.run_step(st) for st in steps])["a"]
        diff = np.abs(got - ref).max(axis=1)
        assert diff.max() <= tol * max(1.0, np.abs(ref).max()), f"{name} {dtype}: position {int(diff.argmax())} differs by {diff.max():.3e}"
        del rp
        torch.cuda.empty_cache()
