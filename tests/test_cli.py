"""The command line: ``python -m nanohybrid_vlm_b200.cli`` (generate, make-random, replay, bench)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, TINY

CLI = [sys.executable, "-m", "nanohybrid_vlm_b200.cli"]


def run(args, **kw):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return subprocess.run(args, capture_output=True, text=True, env=env, cwd=kw.pop("cwd", ROOT), **kw)


def test_make_random_writes_a_folder_that_the_plain_model_reads(tmp_path):
    from plain_qwen3 import PlainQwen3
    cfg, seed = TINY["A"]
    config = tmp_path / "sizes.json"
    config.write_text(json.dumps(cfg))
    out = tmp_path / "model"
    r = run(CLI + ["make-random", "--model", str(out), "--config", str(config), "--seed", str(seed)])
    assert r.returncode == 0, r.stderr
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    assert PlainQwen3(str(out)).logits([1, 2, 3]).shape == (3, cfg["vocab_size"])
    # the same seed gives the same file, another seed another
    again = tmp_path / "again"
    run(CLI + ["make-random", "--model", str(again), "--config", str(config), "--seed", str(seed)])
    from safetensors.torch import load_file
    import torch
    a, b = load_file(str(out / "model.safetensors")), load_file(str(again / "model.safetensors"))
    assert sorted(a) == sorted(b) and all(torch.equal(a[k], b[k]) for k in a)
    run(CLI + ["make-random", "--model", str(again), "--config", str(config), "--seed", str(seed + 1)])
    c = load_file(str(again / "model.safetensors"))
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])


def test_command_line_refuses_what_it_does_not_know(tmp_path):
    assert run(CLI + ["no-such-command"]).returncode == 2
    assert run(CLI + ["generate", "--model", str(tmp_path)]).returncode != 0          # no prompt, no config.json
    r = run(CLI + ["bench", "--gpus", "2"])
    assert r.returncode == 2 and "N=1 only" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(TINY))
def test_generate_prints_the_plain_models_greedy_tokens(name, model_dirs, plain_models):
    cfg, _ = TINY[name]
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (7, 30)]
    args = CLI + ["generate", "--model", model_dirs[name], "--dtype", "float32", "--temperature", "0", "--max-tokens", "6",
                  "--ignore-eos", "--kvcache-block-size", "16", "--num-kvcache-blocks", "32", "--max-num-seqs", "4",
                  "--max-model-len", "128", "--max-num-batched-tokens", "64", "--quiet"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    r = run(args)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [l["prompt"] for l in lines] == prompts
    assert [l["token_ids"] for l in lines] == [plain_models[name].greedy(p, 6) for p in prompts]


@pytest.mark.gpu
def test_generate_with_random_weights_and_a_seeded_temperature(tmp_path):
    """``--random-weights`` needs only config.json in the folder; the same seeds give the same tokens."""
    cfg, _ = TINY["B"]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    args = CLI + ["generate", "--model", str(tmp_path), "--random-weights", "--seed", "5", "--temperature", "0.8",
                  "--sampling-seed", "9", "--max-tokens", "5", "--ignore-eos", "--kvcache-block-size", "8",
                  "--num-kvcache-blocks", "32", "--max-num-seqs", "2", "--max-model-len", "64", "--quiet",
                  "--prompt-ids", "4,5,6"]
    a, b = run(args), run(args)
    assert a.returncode == 0, a.stderr[-3000:]
    assert json.loads(a.stdout.splitlines()[-1])["token_ids"] == json.loads(b.stdout.splitlines()[-1])["token_ids"]
    assert len(json.loads(a.stdout.splitlines()[-1])["token_ids"]) == 5


@pytest.mark.gpu
def test_replay_subcommand_is_trace_run(model_dirs, tmp_path):
    import trace_tools as tt
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3, 9], "want": [0, 3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [8], "want": [0]}], "end": ["a"]}]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    outs = []
    for k, cmd in enumerate((CLI + ["replay"], [sys.executable, tt.TRACE_RUN])):
        out = tmp_path / f"out{k}"
        r = run(cmd + ["--model", model_dirs["A"], "--dtype", "float32", "--out", str(out), "--max-tokens", "64"], input=text)
        assert r.returncode == 0, r.stderr[-3000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
        outs.append([np.fromfile(out / f"{i}.f32", dtype="<f4") for i in range(2)])
    assert all(np.array_equal(x, y) for x, y in zip(*outs))
