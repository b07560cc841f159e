"""The plain implementation against logits that the reference's own model code produced on the CPU
(tests/golden/make_reference_golden.py wrote them).  The weights are regenerated from the same
configuration and seed, so the test also pins the random-weights mode."""
import os

import numpy as np
import pytest

from conftest import TINY

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", list(TINY))
def test_plain_matches_reference_model_code(name, plain_models, model_dirs):
    """float32 plain against the reference run in float64 (tight), bfloat16 plain against the reference
    run in bfloat16 (both round at the same places; what is left is the order of the sums inside
    the matrix products, a few units of bfloat16's last place on logits of this size)."""
    import torch
    from plain_qwen3 import PlainQwen3
    data = np.load(os.path.join(GOLDEN, f"reference_logits_{name}.npz"))
    lengths = data["lengths"].tolist()
    tokens = data["prompts"].tolist()
    plain_bf16 = PlainQwen3(model_dirs[name], torch.bfloat16)
    at = 0
    for i, n in enumerate(lengths):
        prompt = tokens[at:at + n]
        got = plain_models[name].logits(prompt).numpy()
        np.testing.assert_allclose(got, data["all_logits_f64"][at:at + n], rtol=0, atol=1e-6)
        np.testing.assert_allclose(got[-1], data["last_logits_f64"][i], rtol=0, atol=1e-6)
        got16 = plain_bf16.logits(prompt).numpy()
        ref16 = data["all_logits_bf16"][at:at + n]
        assert np.abs(got16 - ref16).max() <= 0.012 * max(1.0, np.abs(ref16).max())
        assert np.abs(got16 - ref16).mean() <= 0.0012 * max(1.0, np.abs(ref16).max())
        at += n
