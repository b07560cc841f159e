"""Trace replay at sizes that take the less-travelled paths of the kernels: a head size that is no power of two
(80, padded shared-memory rows), one whose rows are three swizzle atoms wide (192), a width that is no multiple
of 8 (no vector loads, no weight-streaming kernel), groups of three query heads, odd vocabularies.  Most of the
prompt in one step and the last 32 tokens one by one, against the plain implementation, in both precisions."""
import numpy as np
import pytest

import trace_tools as tt
from plain_qwen3 import PlainQwen3

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", rope_theta=10000.0, rms_norm_eps=1e-6,
            tie_word_embeddings=False, max_position_embeddings=256, torch_dtype="float32", hidden_act="silu",
            attention_bias=False)
ODD = {
    "head80": dict(hidden_size=72, num_hidden_layers=1, num_attention_heads=9, num_key_value_heads=3, head_dim=80,
                   intermediate_size=136, vocab_size=211),
    "width100": dict(hidden_size=100, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
                     intermediate_size=52, vocab_size=130),
    "head192": dict(hidden_size=96, num_hidden_layers=1, num_attention_heads=3, num_key_value_heads=1, head_dim=192,
                    intermediate_size=120, vocab_size=150, tie_word_embeddings=True),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ODD))
def test_replay_at_odd_sizes(name, dtype, tmp_path):
    from nanohybrid_vlm_b200.weights import write_random_model
    cfg = dict(BASE, **ODD[name])
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    write_random_model(str(model_dir), cfg, 7)
    plain = PlainQwen3(str(model_dir))
    rng = np.random.default_rng(5)
    reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate((40, 71, 90, 33))}
    out = tmp_path / "out"
    out.mkdir()
    got = tt.run_trace(str(model_dir), dtype, tt.decode_tail(reqs), str(out), vocab=cfg["vocab_size"])
    for rid, toks in reqs.items():
        ref = plain.logits(toks).numpy()
        g = np.stack([got[rid][p] for p in range(len(toks))])
        err = np.abs(g - ref).max(axis=1)
        bound = 2e-5 if dtype == "float32" else 0.06 * ref.std()
        assert (err <= bound).all(), f"{name} {rid}: first bad position {int((err > bound).argmax())}, worst {err.max():.3e}"
