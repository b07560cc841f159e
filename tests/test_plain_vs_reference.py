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


def _unpack(data) -> dict:
    """``<name>__bf16`` arrays hold the upper 16 bits of float32 numbers (the logits were bfloat16)."""
    out = {}
    for k in data.files:
        v = data[k]
        if k.endswith("__bf16"):
            out[k[:-6]] = (v.astype(np.uint32) << 16).view(np.float32)
        else:
            out[k] = v
    return out


def _errors(got, ref):
    scale = max(1.0, float(np.abs(ref).max()))
    err = np.abs(got - ref)
    return float(err.max()) / scale, float(err.mean()) / scale


def _close_in_bf16(got, ref, what):
    """The largest error as in the comparison on the CPU (three steps of bfloat16 at the logits' size).  The mean
    may be half a step (0.002): on the GPU the reference also rounds the softmax weights to bfloat16 before the
    product with the values, and its products sum in the library's order; measured 0.0006 to 0.0013.  A fault
    of the attention's meaning is far outside both (see the test of that below)."""
    worst, mean = _errors(got, ref)
    assert worst <= 0.012, f"{what}: largest error {worst:.4f} of the logits' size"
    assert mean <= 0.002, f"{what}: mean error {mean:.5f} of the logits' size"


def _gpu_golden(name):
    data = _unpack(np.load(os.path.join(GOLDEN, f"reference_logits_{name}_gpu.npz")))
    flat = data["prompts"].tolist()
    prompts, at = [], 0
    for n in data["lengths"].tolist():
        prompts.append(flat[at:at + n])
        at += n
    return data, prompts


@pytest.mark.parametrize("name", list(TINY))
def test_plain_matches_reference_run_with_its_own_attention_calls(name, model_dirs):
    """bfloat16 plain against logits of the reference's model code run on a B200 with its real attention
    calls (tests/golden/make_reference_golden_gpu.py): whole prompts through ``flash_attn_varlen_func``; a
    second portion of each prompt that attends to the first through the paged cache (more keys than queries,
    so the place of the causal mask is pinned); the last tokens one per step through
    ``flash_attn_with_kvcache``; and the reference's engine generating greedily."""
    import torch
    from plain_qwen3 import PlainQwen3
    data, prompts = _gpu_golden(name)
    plain = PlainQwen3(model_dirs[name], torch.bfloat16)
    full = [plain.logits(p).numpy() for p in prompts]
    routes = 0
    for i, p in enumerate(prompts):
        _close_in_bf16(full[i], data[f"whole_{i}"], f"prompt {i} whole")
        for route in ("chunk", "decode"):
            if f"{route}_{i}" in data:
                a = int(data[f"{route}_{i}_start"])
                ref = data[f"{route}_{i}"]
                _close_in_bf16(full[i][a:a + len(ref)], ref, f"prompt {i} {route} from {a}")
                routes += 1
    assert routes >= 2 * (len(prompts) - 2)          # all but the shortest prompts have both
    # the engine: step k holds, per request, the logits from which its k-th new token was chosen
    assert int(data["engine_ok"]) == 1
    tokens = data["engine_tokens"]
    for i, p in enumerate(prompts):
        seq = list(p)
        for k in range(tokens.shape[1]):
            got = plain.logits(seq)[-1].numpy()
            ref = data[f"engine_logits_{k}"][i]
            _close_in_bf16(got, ref, f"prompt {i}, new token {k}")
            t = int(tokens[i, k])
            assert t == int(ref.argmax())
            assert got[t] >= got.max() - 0.03       # two logits that close may swap between two bfloat16 runs
            seq.append(t)


@pytest.mark.parametrize("fault", ["scale", "heads"])
@pytest.mark.parametrize("name", list(TINY))
def test_the_comparison_would_catch_another_attention(name, fault, model_dirs, monkeypatch):
    """A score scale that is 10 % off, or query head h reading KV head h % num_kv_heads instead of
    h // group, puts the plain implementation outside the bounds of the comparison above."""
    import torch
    import plain_qwen3
    stock = plain_qwen3.causal_attention

    def off_scale(q, k, v, scale):
        return stock(q, k, v, scale * 1.1)

    def other_heads(q, k, v, scale):
        nkv = k.shape[1]
        return torch.cat([stock(q[:, h:h + 1], k[:, h % nkv:h % nkv + 1], v[:, h % nkv:h % nkv + 1], scale)
                          for h in range(q.shape[1])], dim=1)

    monkeypatch.setattr(plain_qwen3, "causal_attention", off_scale if fault == "scale" else other_heads)
    data, prompts = _gpu_golden(name)
    plain = plain_qwen3.PlainQwen3(model_dirs[name], torch.bfloat16)
    i = len(prompts) - 2
    worst, mean = _errors(plain.logits(prompts[i]).numpy(), data[f"whole_{i}"])
    assert worst > 2 * 0.012 and mean > 1.5 * 0.002, (worst, mean)
