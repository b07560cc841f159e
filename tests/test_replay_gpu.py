"""Trace replay through bin/trace_run against the plain implementation: the same requests
whole, with the last 32 tokens decoded one by one, in portions of changing size, and mixed
with other requests in a pool so small that pages are used again; in 32-bit and bfloat16;
on two tiny configurations."""
import numpy as np
import pytest

import trace_tools as tt
from conftest import TINY, TINY_C

pytestmark = pytest.mark.gpu

LENGTHS = (40, 71, 90, 33, 57, 64, 1, 9)
# float32: the engine and the plain implementation add the same numbers in another order.
# bfloat16: activations are rounded to 8 bits of mantissa after every op; the plain implementation
# in float32 is the truth, and the error is measured against the spread of the logits.
F32_TOL = 2e-5
BF16_REL_TOL = 0.06


def requests_for(name):
    cfg, seed = TINY[name]
    rng = np.random.default_rng(100 + seed)
    return {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate(LENGTHS)}


@pytest.fixture(scope="module")
def references(plain_models):
    return {name: {rid: plain_models[name].logits(t).numpy() for rid, t in requests_for(name).items()}
            for name in TINY}


def check(got, ref, reqs, dtype):
    for rid, toks in reqs.items():
        assert sorted(got[rid]) == list(range(len(toks))), f"{rid}: positions missing"
        g = np.stack([got[rid][p] for p in range(len(toks))])
        assert np.isfinite(g).all()
        err = np.abs(g - ref[rid])
        if dtype == "float32":
            p = int(err.max(axis=1).argmax())
            assert err.max() <= F32_TOL, f"{rid}: first bad position {int((err.max(axis=1) > F32_TOL).argmax())}, worst {p}: {err.max():.3e}"
        else:
            scale = ref[rid].std()
            bad = err.max(axis=1) > BF16_REL_TOL * scale
            assert not bad.any(), f"{rid}: first bad position {int(bad.argmax())}: {err.max() / scale:.3f} of the logits' spread"


MODES = {"whole": tt.whole, "decode_tail": tt.decode_tail, "portions": tt.portions, "mixed": tt.mixed}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("name", list(TINY))
def test_replay_matches_plain(name, mode, dtype, model_dirs, references, tmp_path):
    cfg, _ = TINY[name]
    reqs = requests_for(name)
    steps = MODES[mode](reqs)
    got = tt.run_trace(model_dirs[name], dtype, steps, str(tmp_path), vocab=cfg["vocab_size"],
                       page_size=16 if name == "A" else 8)
    check(got, references[name], reqs, dtype)


@pytest.mark.parametrize("name", list(TINY))
def test_float32_logits_do_not_depend_on_the_cutting(name, model_dirs, tmp_path):
    """In 32-bit every kernel fixes the order of its sums per output element, so the logits of a
    position are the same bits however the tokens were cut and batched and wherever their pages lie."""
    cfg, _ = TINY[name]
    reqs = requests_for(name)
    outs = []
    for i, mode in enumerate(("whole", "portions", "mixed")):
        d = tmp_path / mode
        d.mkdir()
        outs.append(tt.run_trace(model_dirs[name], "float32", MODES[mode](reqs), str(d), page_size=8 + 8 * (i % 2)))
    for rid, toks in reqs.items():
        for p in range(len(toks)):
            assert np.array_equal(outs[0][rid][p], outs[1][rid][p]) and np.array_equal(outs[0][rid][p], outs[2][rid][p]), \
                f"{rid} position {p} differs between ways of cutting"


@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_replay_through_the_tcgen05_prompt_kernel(mode, tmp_path):
    """bfloat16 with a head size of 64 and pages of 64 keys: prompt portions run through the tcgen05 kernel
    (first and last tiles partly filled, portions beside decoded tokens, pages used again)."""
    from plain_qwen3 import PlainQwen3
    from nanohybrid_vlm_b200.kernels import attention_tcgen05
    from nanohybrid_vlm_b200.weights import write_random_model
    cfg = TINY_C
    assert attention_tcgen05.supports(cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"], 64)
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    write_random_model(str(model_dir), cfg, 5)
    plain = PlainQwen3(str(model_dir))
    rng = np.random.default_rng(105)
    reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate((140, 71, 200, 33, 65, 64, 2, 129))}
    ref = {rid: plain.logits(t).numpy() for rid, t in reqs.items()}
    out = tmp_path / "out"
    out.mkdir()
    got = tt.run_trace(str(model_dir), "bfloat16", MODES[mode](reqs), str(out), vocab=cfg["vocab_size"], page_size=64)
    check(got, ref, reqs, "bfloat16")


@pytest.mark.parametrize("page_size", [1, 24, 256])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_with_pages_that_do_not_divide_64(dtype, page_size, model_dirs, references, tmp_path):
    """Pages of one token, of 24 and of 256 (the reference's own page size): the pool is counted in tokens
    rounded up to the least common multiple of 64 and the page size, and the logits stay the plain model's."""
    cfg, _ = TINY["B"]
    reqs = requests_for("B")
    got = tt.run_trace(model_dirs["B"], dtype, tt.mixed(reqs), str(tmp_path), vocab=cfg["vocab_size"],
                       page_size=page_size, max_num_seqs=4)
    check(got, references["B"], reqs, dtype)


def test_replay_from_a_configuration_and_a_seed(tmp_path):
    """``--config FILE --seed N`` instead of a folder: the weights are made on the device, one draw per checkpoint
    tensor, and the plain implementation, which makes them by the same rule, gives the same logits."""
    import json
    import torch
    from plain_qwen3 import PlainQwen3, random_weights_on_device
    cfg, _ = TINY["B"]
    path = tmp_path / "config.json"
    path.write_text(json.dumps(cfg))
    plain = PlainQwen3(None, cfg=cfg, weights={k: t.cpu() for k, t in random_weights_on_device(cfg, 77, "cuda").items()})
    reqs = requests_for("B")
    ref = {rid: plain.logits(t).numpy() for rid, t in reqs.items()}
    out = tmp_path / "out"
    got = tt.run_trace(None, "float32", tt.portions(reqs), str(out), vocab=cfg["vocab_size"], page_size=8,
                       config_file=str(path), seed=77)
    check(got, ref, reqs, "float32")
    assert not torch.equal(plain.w["model.norm.weight"],
                           PlainQwen3(None, cfg=cfg, weights=random_weights_on_device(cfg, 78, "cpu")).w["model.norm.weight"])
