"""Helpers of the replay tests: build traces in several ways of cutting and batching, run
``bin/trace_run`` on them and collect the logits per request and position."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def round_up(n: int, unit: int = 64) -> int:
    return -(-n // unit) * unit


def thin(steps: list[dict], keep) -> list[dict]:
    """The same steps with logits wanted only where ``keep(position in the request, request id)`` says so
    (models with a large vocabulary: every row costs a product with the whole head)."""
    at: dict = {}
    out = []
    for st in steps:
        entries = []
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            entries.append(dict(e, want=[w for w in e["want"] if keep(base + w, e["id"])]))
            at[e["id"]] = base + len(e["tokens"])
        out.append(dict(st, entries=entries))
    return out


def whole(requests: dict) -> list[dict]:
    """Each request alone and whole."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def decode_tail(requests: dict, tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests: dict, sizes=(13, 7, 2, 31, 2, 5, 64, 3, 2, 17)) -> list[dict]:
    """Portions of changing size, down to two tokens."""
    steps, k = [], 0
    for rid, toks in requests.items():
        at = 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            at += n
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[at - n:at],
                                                            "want": list(range(n))}],
                          "end": [rid] if at == len(toks) else []})
    return steps


def mixed(requests: dict, live: int = 4, first: int = 24, portion: int = 11, seed: int = 0) -> list[dict]:
    """Up to `live` requests at a time.  A request starts with a portion of `first` tokens, goes on in
    portions of changing size for a while and then token by token; requests at different stages share
    a step, some sit a step out, and a finished request's place (and pages) goes to the next one."""
    rng = np.random.default_rng(seed)
    queue = list(requests.items())
    active: dict[str, int] = {}
    steps = []
    while queue or active:
        while queue and len(active) < live:
            rid, _ = queue.pop(0)
            active[rid] = 0
        entries, ends = [], []
        for rid in list(active):
            toks, at = requests[rid], active[rid]
            if at > 0 and len(active) > 1 and rng.random() < 0.2:
                continue                                    # left out of this step, goes on later
            if at == 0:
                n = min(first, len(toks))
            elif at < len(toks) // 2:
                n = min(int(rng.integers(2, portion + 1)), len(toks) - at)
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": list(range(n))})
            active[rid] = at + n
            if at + n == len(toks):
                ends.append(rid)
                del active[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ends})
    return steps


def max_live_tokens(steps: list[dict], unit: int = 64) -> int:
    """The most tokens that live requests hold at any time, each request's count rounded up to ``unit``."""
    held, most = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(round_up(n, unit) for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return most


def run_trace(model_dir: str | None, dtype: str, steps: list[dict], out_dir: str, max_tokens: int | None = None,
              page_size: int | None = None, vocab: int | None = None, env=None, poison: bool = True,
              config_file: str | None = None, seed: int | None = None, max_num_seqs: int | None = None) -> dict:
    """Run bin/trace_run (on a folder, or on ``config_file`` and ``seed``); returns {request: {position: logits row}}.
    The cache pools start as NaN unless ``poison`` is False."""
    import math
    unit = math.lcm(64, page_size) if page_size else 64
    cmd = [sys.executable, TRACE_RUN, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens or max_live_tokens(steps, unit))]
    cmd += ["--model", model_dir] if config_file is None else ["--config", config_file, "--seed", str(seed)]
    if page_size:
        cmd += ["--page-size", str(page_size)]
    if max_num_seqs:
        cmd += ["--max-num-seqs", str(max_num_seqs)]
    if poison:
        cmd += ["--poison"]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, env=env)
    assert r.returncode == 0, f"trace_run failed ({r.returncode}):\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], "a 'done <step>' line is missing"
    return collect(steps, out_dir, vocab)


def collect(steps: list[dict], out_dir: str, vocab: int | None) -> dict:
    got: dict = {}
    at: dict = {}
    for st in steps:
        wanted = sum(len(e["want"]) for e in st["entries"])
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
            for e in st["entries"]:
                at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
            continue
        data = np.fromfile(path, dtype="<f4")
        assert data.size % wanted == 0
        data = data.reshape(wanted, -1)
        if vocab is not None:
            assert data.shape[1] == vocab
        r = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                got.setdefault(e["id"], {})[base + w] = data[r]
                r += 1
            at[e["id"]] = base + len(e["tokens"])
    return got
