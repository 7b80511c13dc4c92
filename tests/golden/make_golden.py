"""Runs the reference's own model code on the CPU once and stores its logits.

Usage:  python tests/golden/make_golden.py PATH_OF_THE_REFERENCE_TREE     (or $MINI_ENGINE_REF)

The reference's ``models.qwen3.Qwen3ForCausalLM`` is imported with MINI_ENGINE_OPS=0 (its
pure-PyTorch attention, layers/attention.py:54-59), built from a plain namespace with the
tiny configurations of ``tests/tiny_configs.py``, filled by its own loader
(utils/loader.py:13-38) from a folder written by this repository's random-weights mode, and
run on one whole prompt in float32.  The logits go to ``tests/golden/reference_logits.npz``;
``tests/test_plain_model.py`` compares the plain implementation with them.  The plain
implementation was also compared here directly (printed differences).
"""
import os
import sys
import tempfile
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MINI_ENGINE_REF", "")
if not os.path.isfile(os.path.join(REF, "models", "qwen3.py")):
    sys.exit("give the path of the reference tree (ankur110/mini_engine) as the argument or in $MINI_ENGINE_REF")
os.environ["MINI_ENGINE_OPS"] = "0"
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from mini_engine_b200.weights import write_random_model   # noqa: E402
import plain_model                                         # noqa: E402
from tiny_configs import TINY_A, TINY_B                    # noqa: E402

sys.path.insert(0, REF)
from models.qwen3 import Qwen3ForCausalLM                  # noqa: E402  (the reference's)
from utils.loader import load_model                        # noqa: E402
from utils.context import reset_context                    # noqa: E402

out = {}
for name, cfg, seed in (("A", TINY_A, 0), ("B", TINY_B, 1)):
    folder = write_random_model(tempfile.mkdtemp(), cfg, seed, dtype=torch.float32)
    ns = types.SimpleNamespace(**{k: cfg[k] for k in (
        "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
        "intermediate_size", "vocab_size", "rms_norm_eps", "max_position_embeddings", "tie_word_embeddings")},
        rope_parameters={"rope_theta": cfg["rope_theta"]})
    model = Qwen3ForCausalLM(ns)
    load_model(model, folder)
    model.eval()
    gen = torch.Generator().manual_seed(100 + seed)
    ids = torch.randint(0, cfg["vocab_size"], (37,), generator=gen)
    reset_context()
    with torch.inference_mode():
        ref = model.compute_logits(model(ids, torch.arange(ids.shape[0]))).float()
    c, w = plain_model.load_folder(folder)
    mine = plain_model.forward_logits(c, w, ids.tolist(), dtype=torch.float64)
    diff = (mine - ref.double()).abs().max().item()
    print(f"tiny {name}: reference vs plain implementation, max abs diff {diff:.3e} "
          f"(logits up to {ref.abs().max().item():.3f})")
    assert diff < 1e-5
    out[f"ids_{name}"] = ids.numpy().astype(np.int32)
    out[f"logits_{name}"] = ref.numpy()
np.savez_compressed(os.path.join(HERE, "reference_logits.npz"), **out)
print("wrote", os.path.join(HERE, "reference_logits.npz"))
