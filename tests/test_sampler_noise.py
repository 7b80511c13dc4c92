"""The sampler's counter-based noise as restated on the host (no GPU)."""
import numpy as np

import plain_ops
from mini_engine_b200.sampling import SamplingParams, noise_uniform


def test_noise_is_uniform_and_depends_on_every_key():
    u = noise_uniform(seed=1, position=7, vocab_size=50000)
    assert 0 < u.min() and u.max() < 1 and abs(u.mean() - 0.5) < 0.01
    assert abs(np.mean(u < 0.1) - 0.1) < 0.01
    # 23 bits: every value is a float32 number as it stands (the kernel computes in float32), none of them 0 or 1
    assert np.array_equal(u.astype(np.float32).astype(np.float64), u)
    edge = (np.asarray([0, 2 ** 23 - 1], dtype=np.float64) + 0.5) / 8388608.0
    assert 0 < np.float32(edge[0]) and np.float32(edge[1]) < 1 and np.array_equal(edge.astype(np.float32).astype(np.float64), edge)
    assert not np.array_equal(u, noise_uniform(2, 7, 50000))
    assert not np.array_equal(u, noise_uniform(1, 8, 50000))
    assert np.array_equal(u, noise_uniform(1, 7, 50000))


def test_plain_ops_uses_the_same_noise():
    import torch
    x = torch.zeros(1000)
    keys = plain_ops.sample_keys(x, 1.0, 3, 11)
    u = noise_uniform(3, 11, 1000)
    assert np.allclose(keys, -np.log(-np.log(u)))


def test_exponential_race_follows_the_softmax():
    # layers/sampler.py:9-10: argmax(probs / E) picks token v with probability probs[v]
    import torch
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0])
    T = 0.7
    counts = np.zeros(4)
    for pos in range(4000):
        counts[int(np.argmax(plain_ops.sample_keys(logits, T, 5, pos)))] += 1
    p = torch.softmax(logits / T, 0).numpy()
    assert np.abs(counts / 4000 - p).max() < 0.03


def test_sampling_params_checks():
    import pytest
    assert SamplingParams().temperature == 1.0 and SamplingParams().max_tokens == 64
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1)
    with pytest.raises(ValueError):
        SamplingParams(max_tokens=0)
