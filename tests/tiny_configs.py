"""Tiny Qwen3 configurations for tests: they differ in every size and option."""
from __future__ import annotations


def _cfg(**kw):
    base = {"architectures": ["Qwen3ForCausalLM"], "hidden_act": "silu", "attention_bias": False,
            "torch_dtype": "bfloat16", "max_position_embeddings": 512}
    base.update(kw)
    return base


# 2 layers, grouped heads 4/2, head_dim 16 (heads*head_dim = hidden), tied head, theta 1e4, eps 1e-6
TINY_A = _cfg(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
              tie_word_embeddings=True)
# 3 layers, 8/2 heads (groups of 4), head_dim 32 (heads*head_dim = 256 != hidden 96), sizes that are
# no power of two, untied head, theta 1e6, eps 1e-5
TINY_B = _cfg(hidden_size=96, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2,
              head_dim=32, intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
              tie_word_embeddings=False)
# 4 layers, 6/3 heads, head_dim 48, a window of 24 keys on layers 1 and 3, odd sizes
TINY_C = _cfg(hidden_size=72, num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=3,
              head_dim=48, intermediate_size=200, vocab_size=333, rope_theta=50000.0, rms_norm_eps=3e-6,
              tie_word_embeddings=False, use_sliding_window=True, sliding_window=24,
              layer_types=["full_attention", "sliding_attention", "full_attention", "sliding_attention"])

# 2 layers, 6/2 heads (groups of 3), head_dim 64: the head size the bfloat16 tensor-core attention takes; a window
# of 40 keys on layer 1; pages of 32
TINY_D = _cfg(hidden_size=80, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2,
              head_dim=64, intermediate_size=176, vocab_size=300, rope_theta=20000.0, rms_norm_eps=2e-6,
              tie_word_embeddings=True, use_sliding_window=True, sliding_window=40,
              layer_types=["full_attention", "sliding_attention"])

ALL = {"A": (TINY_A, 0, 16), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16), "D": (TINY_D, 3, 32)}   # config, seed, page size
