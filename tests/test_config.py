import json
import os

import pytest
import torch

from conftest import TINY_A, TINY_B
from nanohybrid_vlm_b200.config import ARCHITECTURES, Config, ConfigError, load_model_config, register_architecture
from nanohybrid_vlm_b200.models.qwen3 import Qwen3Config, build_spec


def write_config(tmp_path, cfg):
    d = tmp_path / "m"
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps(cfg))
    return str(d)


def test_every_size_comes_from_config_json(tmp_path):
    for raw in (TINY_A, TINY_B):
        entry, cfg = load_model_config(write_config(tmp_path, raw))
        assert entry.name == "Qwen3ForCausalLM"
        for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
                    "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta", "max_position_embeddings",
                    "tie_word_embeddings"):
            assert getattr(cfg, key) == raw[key], key
        assert cfg.dtype == torch.float32
        assert Qwen3Config.from_json_dict(cfg.to_json_dict()) == cfg


def test_defaults_follow_the_reference(tmp_path):
    raw = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "rope_theta", "num_key_value_heads")}
    _, cfg = load_model_config(write_config(tmp_path, raw))
    assert cfg.head_dim == raw["hidden_size"] // raw["num_attention_heads"]
    assert cfg.rope_theta == 1000000.0
    assert cfg.num_key_value_heads == raw["num_attention_heads"]
    raw["rope_scaling"] = {"rope_theta": 5000.0}
    _, cfg = load_model_config(write_config(tmp_path, raw))
    assert cfg.rope_theta == 5000.0


@pytest.mark.parametrize("change,message", [
    ({"hidden_size": None}, "hidden_size"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"torch_dtype": None}, "dtype"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"eos_token_id": [1, 2]}, "eos"),
    ({"architectures": ["LlamaForCausalLM"]}, "unsupported"),
    ({"architectures": None}, "architectures"),
    ({"model_type": "qwen3_5"}, "model_type"),
])
def test_bad_config_is_one_clear_error(tmp_path, change, message):
    raw = {**TINY_A, **change}
    raw = {k: v for k, v in raw.items() if v is not None}
    with pytest.raises(ConfigError, match=message):
        load_model_config(write_config(tmp_path, raw))


def test_missing_or_broken_file(tmp_path):
    with pytest.raises(ConfigError, match="config.json"):
        load_model_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_model_config(str(tmp_path))


def test_registry_maps_names_to_models():
    assert "Qwen3ForCausalLM" in ARCHITECTURES.names()
    with pytest.raises(ValueError, match="already"):
        register_architecture("Qwen3ForCausalLM", parse_config=lambda r: None, build_spec=lambda c: None)
    with pytest.raises(TypeError):
        register_architecture("Broken", parse_config=None, build_spec=None)
    register_architecture("ToyArch", model_types=("toy",), parse_config=lambda r: "cfg", build_spec=lambda c: "spec")
    try:
        assert ARCHITECTURES.resolve({"architectures": ["ToyArch"], "model_type": "toy"}).parse_config({}) == "cfg"
        with pytest.raises(ConfigError, match="model_type"):
            ARCHITECTURES.resolve({"architectures": ["ToyArch"], "model_type": "other"})
    finally:
        ARCHITECTURES.unregister("ToyArch")


def test_spec_is_data(tmp_path):
    _, cfg = load_model_config(write_config(tmp_path, TINY_B))
    spec = build_spec(cfg)
    spec.validate()
    assert len(spec.layers) == 3 and [r.layer for r in spec.order] == [0, 1, 2]
    mixer = spec.layers[1].mixer.spec
    assert (mixer.kind, mixer["num_heads"], mixer["num_kv_heads"], mixer["head_dim"]) == ("gqa_attention", 6, 2, 32)
    assert mixer["position"]["theta"] == 1000000.0 and mixer["qk_norm_eps"] == 1e-5
    assert spec.layers[2].ffn.spec["intermediate_size"] == 160
    assert spec.head.spec["tied"] is False


def test_engine_options(tmp_path):
    d = write_config(tmp_path, TINY_A)
    c = Config(d, max_model_len=100000, kvcache_block_size=16)
    assert c.max_model_len == TINY_A["max_position_embeddings"]      # clamped as the reference does
    assert c.dtype == torch.float32 and c.eos == -1
    assert Config(d, dtype="bfloat16").dtype == torch.bfloat16
    assert Config(write_config(tmp_path, TINY_B)).eos == 7
    for bad in (dict(tensor_parallel_size=2), dict(kvcache_block_size=0), dict(scheduler_policy="x"),
                dict(gpu_memory_utilization=1.5), dict(dtype="float16"),
                dict(max_num_seqs=0)):
        with pytest.raises(ConfigError):
            Config(d, **bad)
    with pytest.raises(ConfigError):
        Config(os.path.join(d, "nowhere"))
