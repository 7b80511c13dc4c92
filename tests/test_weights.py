"""Weights by tensor name, their errors, and the random-weights mode (no GPU)."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from mini_engine_b200.weights import WeightsError, build_model_from_config_dict, load_weights, write_random_model
from tiny_configs import TINY_A, TINY_B


def _load(folder, raw, dtype):
    _, model = build_model_from_config_dict(raw)
    return model, load_weights(model, folder, dtype, torch.device("cpu"))


def test_random_mode_writes_a_loadable_folder(tmp_path):
    folder = write_random_model(str(tmp_path), TINY_B, seed=1)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(folder, "config.json"))) == TINY_B
    disk = load_file(os.path.join(folder, "model.safetensors"))
    assert all(t.dtype == torch.bfloat16 for t in disk.values())
    model, params = _load(folder, TINY_B, torch.bfloat16)
    qkv = params["model.layers.0.self_attn.qkv_proj.weight"]
    nh, nkv, d = 8, 2, 32
    assert qkv.shape == ((nh + 2 * nkv) * d, 96) and qkv.dtype == torch.bfloat16
    assert torch.equal(qkv[: nh * d], disk["model.layers.0.self_attn.q_proj.weight"])
    assert torch.equal(qkv[nh * d:(nh + nkv) * d], disk["model.layers.0.self_attn.k_proj.weight"])
    assert torch.equal(qkv[(nh + nkv) * d:], disk["model.layers.0.self_attn.v_proj.weight"])
    gu = params["model.layers.2.mlp.gate_up_proj.weight"]
    assert torch.equal(gu[:224], disk["model.layers.2.mlp.gate_proj.weight"])
    assert torch.equal(gu[224:], disk["model.layers.2.mlp.up_proj.weight"])
    # vectors are held in float32 (exact for bfloat16 files)
    nw = params["model.layers.1.input_layernorm.weight"]
    assert nw.dtype == torch.float32 and torch.equal(nw, disk["model.layers.1.input_layernorm.weight"].float())
    assert abs(float(nw.mean()) - 1.0) < 0.1
    assert params["lm_head.weight"].data_ptr() != params["model.embed_tokens.weight"].data_ptr()


def test_same_seed_same_weights_other_seed_other_weights(tmp_path):
    a = load_file(os.path.join(write_random_model(str(tmp_path / "a"), TINY_A, 7), "model.safetensors"))
    b = load_file(os.path.join(write_random_model(str(tmp_path / "b"), TINY_A, 7), "model.safetensors"))
    c = load_file(os.path.join(write_random_model(str(tmp_path / "c"), TINY_A, 8), "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)


def test_tied_head_shares_storage_and_skips_disk_tensor(tmp_path):
    folder = write_random_model(str(tmp_path), TINY_A, 0)
    path = os.path.join(folder, "model.safetensors")
    disk = load_file(path)
    assert "lm_head.weight" not in disk
    disk["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)   # present but tied: skipped
    save_file(disk, path)
    model, params = _load(folder, TINY_A, torch.bfloat16)
    assert params["lm_head.weight"].data_ptr() == params["model.embed_tokens.weight"].data_ptr()


def test_float32_engine_widens_and_32bit_tensors_stay(tmp_path):
    folder = write_random_model(str(tmp_path), TINY_A, 0)
    path = os.path.join(folder, "model.safetensors")
    disk = load_file(path)
    _, p32 = _load(folder, TINY_A, torch.float32)
    w = p32["model.layers.0.mlp.down_proj.weight"]
    assert w.dtype == torch.float32 and torch.equal(w, disk["model.layers.0.mlp.down_proj.weight"].float())
    disk["model.layers.0.mlp.down_proj.weight"] = disk["model.layers.0.mlp.down_proj.weight"].float() + 1e-4
    save_file(disk, path)
    _, p16 = _load(folder, TINY_A, torch.bfloat16)
    assert p16["model.layers.0.mlp.down_proj.weight"].dtype == torch.float32        # stored in 32-bit: stays
    assert torch.equal(p16["model.layers.0.mlp.down_proj.weight"], disk["model.layers.0.mlp.down_proj.weight"])
    assert p16["model.layers.1.mlp.down_proj.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(str(tmp_path), TINY_B, 1)
    path = os.path.join(folder, "model.safetensors")
    disk = load_file(path)
    del disk["model.layers.1.self_attn.k_proj.weight"]
    del disk["model.norm.weight"]
    disk["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    disk["model.layers.2.mlp.up_proj.weight"] = torch.zeros(10, 96, dtype=torch.bfloat16)
    save_file(disk, path)
    with pytest.raises(WeightsError) as ei:
        _load(folder, TINY_B, torch.bfloat16)
    e = ei.value
    assert e.missing == ["model.layers.1.self_attn.k_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert [(n, tuple(g), tuple(w)) for n, g, w in e.wrong_shape] == \
        [("model.layers.2.mlp.up_proj.weight", (10, 96), (224, 96))]
    text = str(e)
    for word in ("missing", "unexpected", "wrong shapes", "k_proj", "inv_freq", "[224, 96]"):
        assert word in text


def test_no_safetensors_file(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(WeightsError, match="no .safetensors"):
        _load(str(tmp_path), TINY_A, torch.bfloat16)
