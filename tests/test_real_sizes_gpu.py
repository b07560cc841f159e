"""The engine at the layer sizes of the benchmark model (width 4096, 32 query and 8 KV heads of 128,
feed-forward 12288, pages of 256 tokens), two layers, a vocabulary that is no power of two: the kernels
that serving uses at full size (streaming GEMMs with tensor maps, tensor-core attention, captured graphs)
against the plain implementation, in 32-bit and in bfloat16."""
import numpy as np
import pytest

import trace_tools as tt

pytestmark = pytest.mark.gpu

REAL = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096, num_hidden_layers=2,
            num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=32003,
            rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096,
            torch_dtype="bfloat16", hidden_act="silu", attention_bias=False)


@pytest.fixture(scope="module")
def real_model(tmp_path_factory):
    from nanohybrid_vlm_b200.weights import write_random_model
    from plain_qwen3 import PlainQwen3
    d = str(tmp_path_factory.mktemp("real_sizes"))
    write_random_model(d, REAL, seed=2)
    return d, PlainQwen3(d)          # the plain model computes in float32 from the stored bfloat16 weights


@pytest.fixture(scope="module")
def tokens():
    rng = np.random.default_rng(7)
    return {"a": rng.integers(0, REAL["vocab_size"], 300).tolist(), "b": rng.integers(0, REAL["vocab_size"], 41).tolist()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_at_real_layer_sizes(real_model, tokens, dtype, tmp_path):
    d, plain = real_model
    # request a: 290 tokens at once, then token by token beside request b's portions; pages of 64 tokens
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens["a"][:290], "want": [0, 255, 256, 289]}], "end": []}]
    at_b = 0
    for i in range(10):
        n = (17, 2, 22)[i] if i < 3 else 0
        entries = [{"id": "a", "tokens": [tokens["a"][290 + i]], "want": [0]}]
        if n:
            entries.append({"id": "b", "tokens": tokens["b"][at_b:at_b + n], "want": [n - 1]})
            at_b += n
        steps.append({"step": i + 1, "entries": entries, "end": ["a"] if i == 9 else []})
    steps[3]["end"] = ["b"]
    got = tt.run_trace(d, dtype, steps, str(tmp_path), vocab=REAL["vocab_size"], page_size=64)
    ref = {r: plain.logits(t).numpy() for r, t in tokens.items()}
    worst = (0.0, 0.0)
    for rid, rows in got.items():
        for pos, row in rows.items():
            diff = row - ref[rid][pos]
            err, spread = np.abs(diff).max(), ref[rid][pos].std()
            if dtype == "float32":
                assert err <= 2e-4 * max(1.0, np.abs(ref[rid][pos]).max()), f"{rid} position {pos}: {err:.3e}"
            else:
                # bfloat16 keeps 8 bits: a logit of size 4 is stored to +-0.016 whatever came before, and some twenty
                # roundings of the activations lie before it.  Over 32,003 logits the largest error is several
                # times the typical one, so both are bounded: the typical (rms) and the largest.
                rms = float(np.sqrt((diff ** 2).mean()))
                worst = max(worst, (rms / spread, err / spread))
                assert rms <= 0.02 * spread, f"{rid} position {pos}: rms error {rms / spread:.4f} of the spread"
                assert err <= 0.10 * spread, f"{rid} position {pos}: largest error {err / spread:.3f} of the spread"
    print("worst (rms, max) error as a share of the logits' spread:", worst)
    assert sorted(got["a"]) == [0, 255, 256, 289, *range(290, 300)] and sorted(got["b"]) == [16, 18, 40]


def test_generation_at_real_layer_sizes_through_graphs(real_model, tokens):
    from nanohybrid_vlm_b200 import LLM, SamplingParams
    d, plain = real_model
    llm = LLM(d, kvcache_block_size=256, num_kvcache_blocks=8, max_num_seqs=4, max_num_batched_tokens=512,
              max_model_len=1024)
    prompts = [tokens["a"][:200], tokens["b"]]
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True), use_tqdm=False)
    for p, o in zip(prompts, out):
        seq = list(p)
        for t in o["token_ids"]:
            lg = plain.logits(seq)[-1]
            assert lg[t] >= lg.max() - 0.08 * lg.std(), f"token {t} at position {len(seq)} is not near the plain model's best"
            seq.append(t)
    from nanohybrid_vlm_b200.kernels import ops
    assert ops.stream_k_error() == 0
