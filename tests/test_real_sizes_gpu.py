"""The engine at the layer sizes, page size and vocabulary of the benchmark model (width 4096, 32 query and 8 KV
heads of 128, feed-forward 12288, vocabulary 151,936, pages of 256 tokens), TWO layers instead of 36: the kernels
that serving uses at full size (weight-streaming products, tensor-core attention, captured graphs, the head over
the whole vocabulary) against the plain implementation, in 32-bit and in bfloat16, in all four ways of cutting.

The model is given to ``bin/trace_run`` as (config, seed); the plain implementation makes the same tensors from
the rule of the random-weights mode and computes on the GPU in float32 (no reduced-precision matrix mode)."""
import json

import numpy as np
import pytest
import torch

import trace_tools as tt

pytestmark = pytest.mark.gpu

REAL = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096, num_hidden_layers=2,
            num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
            rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096,
            torch_dtype="bfloat16", hidden_act="silu", attention_bias=False)
SEED = 2
PAGE = 256
LENGTHS = {"a": 530, "b": 41, "c": 300, "d": 257, "e": 64, "f": 2}
MODES = {"whole": tt.whole, "decode_tail": tt.decode_tail, "portions": tt.portions, "mixed": tt.mixed}


def keep(position, rid):
    """Where logits are compared: the first tokens, both sides of every page edge, the last 33, and every 29th."""
    n = LENGTHS[rid]
    return position < 2 or position % PAGE in (PAGE - 2, PAGE - 1, 0, 1) or position >= n - 33 or position % 29 == 0


@pytest.fixture(scope="module")
def config_file(tmp_path_factory):
    path = tmp_path_factory.mktemp("real_sizes") / "config.json"
    path.write_text(json.dumps(REAL))
    return str(path)


@pytest.fixture(scope="module")
def requests():
    rng = np.random.default_rng(7)
    return {rid: rng.integers(0, REAL["vocab_size"], n).tolist() for rid, n in LENGTHS.items()}


@pytest.fixture(scope="module")
def plains():
    """The plain implementation on the GPU with the weights of (REAL, SEED): as drawn (the 32-bit engine's), and
    rounded to bfloat16 (the bfloat16 engine's), both computing in float32."""
    from plain_qwen3 import PlainQwen3, random_weights_on_device
    assert not torch.backends.cuda.matmul.allow_tf32
    w = random_weights_on_device(REAL, SEED, "cuda")
    out = {"float32": PlainQwen3(None, cfg=REAL, weights=w),
           "bfloat16": PlainQwen3(None, cfg=REAL, weights={k: t.bfloat16().float() for k, t in w.items()})}
    del w
    return out


@pytest.fixture(scope="module")
def references(plains, requests):
    out = {}
    for dtype, plain in plains.items():
        out[dtype] = {}
        for rid, toks in requests.items():
            rows = [p for p in range(len(toks)) if keep(p, rid)]
            lg = plain.logits(toks, rows=rows).cpu().numpy()
            out[dtype][rid] = dict(zip(rows, lg))
    return out


@pytest.fixture(scope="module")
def replayed(config_file, requests, tmp_path_factory):
    """Runs of bin/trace_run, each made once: (mode, dtype) -> {request: {position: logits}}."""
    done = {}

    def run(mode, dtype):
        if (mode, dtype) not in done:
            steps = tt.thin(MODES[mode](requests), keep)
            out = tmp_path_factory.mktemp(f"replay_{mode}_{dtype}")
            done[mode, dtype] = tt.run_trace(None, dtype, steps, str(out), vocab=REAL["vocab_size"], page_size=PAGE,
                                             config_file=config_file, seed=SEED, max_num_seqs=4)
        return done[mode, dtype]
    return run


def bf16_errors(row, ref):
    """(rms error, largest error) as shares of the logits' spread."""
    diff = row - ref
    spread = float(ref.std())
    return float(np.sqrt((diff ** 2).mean())) / spread, float(np.abs(diff).max()) / spread


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
def test_replay_at_real_sizes_two_layers_page_256_full_vocabulary(mode, dtype, replayed, references, requests):
    got = replayed(mode, dtype)
    worst = (0.0, 0.0)
    for rid, toks in requests.items():
        ref = references[dtype][rid]
        assert sorted(got[rid]) == sorted(ref), f"{rid}: positions missing"
        for pos, want in ref.items():
            row = got[rid][pos]
            assert np.isfinite(row).all(), f"{rid} position {pos}: not finite (a slot read that no step wrote?)"
            if dtype == "float32":
                err = np.abs(row - want).max()
                assert err <= 2e-4 * max(1.0, np.abs(want).max()), f"{rid} position {pos}: {err:.3e}"
            else:
                # bfloat16 keeps 8 bits: a logit of size 4 is stored to +-0.016 whatever came before, and some twenty
                # roundings of the activations lie before it.  Over 151,936 logits the largest error is several
                # times the typical one, so both are bounded: the typical (rms) and the largest.
                rms, big = bf16_errors(row, want)
                worst = max(worst, (rms, big))
                assert rms <= 0.02, f"{rid} position {pos}: rms error {rms:.4f} of the spread"
                assert big <= 0.10, f"{rid} position {pos}: largest error {big:.3f} of the spread"
    print(f"{mode} {dtype}: worst (rms, max) error as a share of the logits' spread:", worst)


def test_float32_logits_at_real_sizes_do_not_depend_on_the_cutting(replayed, requests):
    outs = [replayed(mode, "float32") for mode in ("whole", "decode_tail", "portions", "mixed")]
    for rid in requests:
        for pos, row in outs[0][rid].items():
            for other in outs[1:]:
                assert np.array_equal(row, other[rid][pos]), f"{rid} position {pos} differs between ways of cutting"


@pytest.fixture(scope="module")
def model_folder(config_file, tmp_path_factory):
    """A folder that holds only config.json: the engine makes the weights of (REAL, SEED) on the device."""
    import os
    return os.path.dirname(config_file)


def test_generation_at_real_sizes_through_graphs(model_folder, plains, requests):
    """Greedy generation through the entry point (prompts in portions, then captured decode graphs): at every
    step the logits behind each chosen token are the plain model's for the same tokens, within the bound of the
    bfloat16 replay, and the chosen token is the largest of them."""
    from nanohybrid_vlm_b200 import LLM, SamplingParams
    llm = LLM(model_folder, random_weights_seed=SEED, kvcache_block_size=PAGE, num_kvcache_blocks=8, max_num_seqs=4,
              max_num_batched_tokens=256, max_model_len=1024, poison_cache=True)
    plain = plains["bfloat16"]
    prompts = [requests["c"][:200], requests["b"], requests["d"]]
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    seqs = {llm.add_request(list(p), sp): list(p) for p in prompts}
    checked = 0
    while not llm.is_finished():
        llm.step()
        ids = llm.last_sampled_ids
        if not ids:
            continue
        logits = llm.model_runner.last_logits[:len(ids)].cpu().numpy()
        for row, seq_id in zip(logits, ids):
            want = plain.logits(seqs[seq_id], rows=[len(seqs[seq_id]) - 1])[0].cpu().numpy()
            rms, big = bf16_errors(row, want)
            assert rms <= 0.02 and big <= 0.10, f"request {seq_id} at {len(seqs[seq_id])} tokens: {rms:.4f}, {big:.3f}"
            seqs[seq_id].append(int(row.argmax()))
            checked += 1
    assert checked == 15 and llm.model_runner._graphs, "the decode steps should have run through captured graphs"
    done = {m.seq_id: m.num_completion_tokens for m in llm.get_completed_request_metrics()}
    assert all(v == 5 for v in done.values()) and len(done) == 3


def test_a_decode_graph_of_64_requests_against_eager_and_plain(model_folder, plains):
    """40 requests of 1 to 600 tokens decode for a few steps as one batch: through the captured graph of the
    64-request bucket (24 idle entries beside them) and eagerly.  Both give the plain model's logits, and each
    other's, within the bound of the bfloat16 replay (the products of 40 and of 64 rows are tiled differently)."""
    from nanohybrid_vlm_b200.config import Config
    from nanohybrid_vlm_b200.engine.batch import StepItem
    from nanohybrid_vlm_b200.engine.runner import ModelRunner
    rng = np.random.default_rng(11)
    lengths = [1, 2, 255, 256, 257, 600] + rng.integers(3, 600, 34).tolist()
    steps = 3
    toks = [rng.integers(0, REAL["vocab_size"], n + steps).tolist() for n in lengths]
    plain = plains["bfloat16"]
    results = {}
    for eager in (False, True):
        runner = ModelRunner(Config(model_folder, kvcache_block_size=PAGE, num_kvcache_blocks=130, max_num_seqs=64,
                                    max_num_batched_tokens=4096, max_model_len=1024, enforce_eager=eager,
                                    poison_cache=True, enable_prefix_cache=False), random_weights_seed=SEED)
        at = 0
        while at < len(toks):                       # prompts, a few per step
            group = list(range(at, min(at + 6, len(toks))))
            items = []
            for i in group:
                runner.cache.allocate(i, lengths[i])
                items.append(StepItem(i, toks[i][:lengths[i]], 0, []))
            runner.step(items)
            at += 6
        rows = []
        for s in range(steps):
            items = []
            for i in range(len(toks)):
                runner.cache.allocate(i, lengths[i] + s + 1)
                items.append(StepItem(i, [toks[i][lengths[i] + s]], lengths[i] + s, [0]))
            runner.run(items, [(0.0, 1, lengths[i] + s + 1) for i in range(len(toks))])
            rows.append(runner.last_logits.float().cpu().numpy().copy())
        assert bool(runner._graphs) != eager and (eager or 64 in runner._graphs)
        results[eager] = rows
        del runner
        torch.cuda.empty_cache()
    for s in range(steps):
        for i in range(len(toks)):
            n = lengths[i] + s + 1
            want = plain.logits(toks[i][:n], rows=[n - 1])[0].cpu().numpy()
            for eager in (False, True):
                rms, big = bf16_errors(results[eager][s][i], want)
                assert rms <= 0.02 and big <= 0.10, f"request {i} ({n} tokens), eager={eager}: {rms:.4f}, {big:.3f}"
            rms, big = bf16_errors(results[False][s][i], results[True][s][i])
            assert rms <= 0.02 and big <= 0.10, f"request {i}: graph and eager differ by {rms:.4f}, {big:.3f}"
