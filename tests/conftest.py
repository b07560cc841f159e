import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# Two tiny Qwen3 configurations that differ in every size and option: layers, width, head
# counts and group size, head size (heads * head_dim equal to the width or not), feed-forward
# width, vocabulary, rope base, eps, tied or separate head, longest position.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256,
              torch_dtype="float32", hidden_act="silu", attention_bias=False)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=96, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=2, head_dim=32, intermediate_size=160, vocab_size=384,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512,
              torch_dtype="float32", hidden_act="silu", attention_bias=False, eos_token_id=7)
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1)}
# a head size and (with pages of 64) a page size that the tcgen05 prompt-attention kernel takes; three query heads
# share the one KV head, so a block's 128 rows hold 42 tokens and two rows of padding
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=120, num_hidden_layers=2,
              num_attention_heads=3, num_key_value_heads=1, head_dim=64, intermediate_size=200, vocab_size=300,
              rope_theta=50000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=512,
              torch_dtype="float32", hidden_act="silu", attention_bias=False)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders (config.json, model.safetensors) of the two tiny configurations, in a temporary place."""
    from nanohybrid_vlm_b200.weights import write_random_model
    out = {}
    for name, (cfg, seed) in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(str(d), cfg, seed)
        out[name] = str(d)
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    from plain_qwen3 import PlainQwen3
    return {name: PlainQwen3(d) for name, d in model_dirs.items()}
