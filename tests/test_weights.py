import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TINY_A, TINY_B
from nanohybrid_vlm_b200.config import load_model_config
from nanohybrid_vlm_b200.engine.model import CausalLM
from nanohybrid_vlm_b200.weights import WeightError, load_weights, write_random_model


def build(model_dir, dtype=torch.float32):
    entry, cfg = load_model_config(model_dir)
    return CausalLM(entry.build_spec(cfg), dtype, "cpu")


def test_random_mode_writes_a_model_folder(tmp_path):
    d = write_random_model(str(tmp_path / "a"), TINY_A, seed=0)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(d, "config.json"))) == TINY_A
    t = load_file(os.path.join(d, "model.safetensors"))
    assert "lm_head.weight" not in t                                  # tied head: one table
    assert t["model.layers.1.self_attn.k_proj.weight"].shape == (2 * 16, 64)
    assert t["model.layers.0.mlp.up_proj.weight"].shape == (128, 64)
    assert abs(t["model.embed_tokens.weight"].std().item() - 0.02) < 2e-3
    assert abs(t["model.norm.weight"].mean().item() - 1.0) < 1e-2
    again = load_file(os.path.join(write_random_model(str(tmp_path / "b"), TINY_A, seed=0), "model.safetensors"))
    other = load_file(os.path.join(write_random_model(str(tmp_path / "c"), TINY_A, seed=5), "model.safetensors"))
    assert all(torch.equal(t[k], again[k]) for k in t)
    assert not torch.equal(t["model.norm.weight"], other["model.norm.weight"])


def test_loading_packs_by_name_and_keeps_dtype(tmp_path):
    d = write_random_model(str(tmp_path / "b"), TINY_B, seed=1)
    raw = load_file(os.path.join(d, "model.safetensors"))
    for dtype in (torch.float32, torch.bfloat16):
        model = build(d, dtype)
        tensors = load_weights(model, d)
        qkv = tensors["model.layers.2.self_attn.qkv_proj.weight"]
        assert qkv.dtype == dtype and qkv.shape == ((6 + 2 * 2) * 32, 96)
        p = "model.layers.2.self_attn."
        want = torch.cat([raw[p + "q_proj.weight"], raw[p + "k_proj.weight"], raw[p + "v_proj.weight"]]).to(dtype)
        assert torch.equal(qkv, want)
        gu = tensors["model.layers.0.mlp.gate_up_proj.weight"]
        assert torch.equal(gu[:160], raw["model.layers.0.mlp.gate_proj.weight"].to(dtype))
        assert torch.equal(gu[160:], raw["model.layers.0.mlp.up_proj.weight"].to(dtype))
        assert model.head.w_weight is not model.embedding.w_weight


def test_tied_head_shares_the_table_and_ignores_a_stored_copy(tmp_path):
    d = write_random_model(str(tmp_path / "a"), TINY_A, seed=0)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    save_file(t, path)
    model = build(d)
    load_weights(model, d)
    assert model.head.w_weight is model.embedding.w_weight


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(str(tmp_path / "b"), TINY_B, seed=1)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.self_attn.k_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.mlp.extra.weight"] = torch.zeros(3)
    t["model.layers.2.mlp.down_proj.weight"] = torch.zeros(96, 161)
    t["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16)
    save_file(t, path)
    with pytest.raises(WeightError) as e:
        load_weights(build(d), d)
    err = e.value
    assert err.missing == ["model.layers.1.self_attn.k_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.self_attn.q_norm.weight",
                                               "model.layers.2.mlp.down_proj.weight"]
    text = str(err)
    for needle in ("missing", "unexpected", "wrong shapes", "k_proj", "extra", "(96, 161)", "(96, 160)"):
        assert needle in text


def test_no_safetensors_file(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(FileNotFoundError):
        load_weights(build(str(tmp_path)), str(tmp_path))
