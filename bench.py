"""Benchmark of the engine's decode and prefill steps on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload 0.6b|32b      the baseline's other two workloads, through the Python entry point
    python bench.py --breakdown              where a decode step's and a prefill's time goes, by kind of kernel

The default run has the layer sizes of the Qwen3-8B-shaped configuration (36 layers, width 4096,
32/8 heads of 128, feed-forward 12288, vocabulary 151936), bfloat16, random weights, batch 8,
2,048-token uniform-random prompts, decoding inside a 4,096-token context.  A "step" is one decode
step of the whole batch.  It prints ONE JSON line:

* ``value``: decoded tokens per second, K steps of the model runner timed on the device with CUDA events (a step is
  launched before the host has read the tokens of the step before it, as generation does it);
* ``e2e``: the same through the Python entry point (``LLM.add_request`` / ``LLM.step``): host
  token lists in, chosen tokens back on the host every step;
* ``prefill``: one 2,048-token prompt in one step; ``frac`` = its flops / time / bf16 peak;
* ``roofline``: bytes the decode step has to read (every weight once, the cache of the live
  requests) / time, against the HBM peak;
* ``points``: decode at batch 1 and 64.

Peaks come from MEASURED_PEAKS.json beside this file if present, else the fallback figures
6.65 TB/s and 1.59 PFLOP/s.  Weights (16 GB) exceed L2 many times over, so every timed step
reads them from HBM; no L2 flush is needed and ``config.l2`` says so.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIG_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096, num_hidden_layers=36,
                 num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                 vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                 max_position_embeddings=40960, torch_dtype="bfloat16", hidden_act="silu", attention_bias=False)
# the other two shapes that the baseline names (random weights, seeds 3 and 4), run with --workload
CONFIG_06B = dict(CONFIG_8B, hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                  intermediate_size=3072, tie_word_embeddings=True)
CONFIG_32B = dict(CONFIG_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                  intermediate_size=25600)
FULL_LAYERS = 36
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE = 256
SEED = 2
METRIC = "decode tok/s at batch 8 (Qwen3-8B-shaped bf16, 2,048-token prompts, context 4,096)"


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            out["hbm_gbs"] = float(raw.get("hbm_gbs", out["hbm_gbs"]))
            out["bf16_tflops"] = float(raw.get("bf16_tflops", out["bf16_tflops"]))
            out["source"] = "measured"
        except (OSError, ValueError):
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def model_numbers(cfg: dict, layers: int) -> dict:
    H, nq, nkv, d, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                           cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = (nq + 2 * nkv) * d * H + nq * d * H + 2 * I * H + I * H + 2 * H + 2 * d
    return {"layer_params": per_layer, "head_params": V * H, "kv_bytes_per_token": 2 * nkv * d * 2 * layers,
            "weight_bytes": 2 * (layers * per_layer + V * H + H)}


def prefill_flops(cfg: dict, layers: int, T: int) -> float:
    H, nq, d, V = cfg["hidden_size"], cfg["num_attention_heads"], cfg["head_dim"], cfg["vocab_size"]
    n = model_numbers(cfg, layers)
    linear = 2.0 * T * (layers * (n["layer_params"] - 2 * H - 2 * d)) + 2.0 * V * H   # one logits row
    attention = layers * 4.0 * nq * d * (T * (T + 1) / 2)                              # causal QK^T and PV
    return linear + attention


def bench_ours(args) -> dict:
    import torch

    from nanohybrid_vlm_b200 import LLM, SamplingParams
    from nanohybrid_vlm_b200.engine import StepItem
    from nanohybrid_vlm_b200.kernels import library as klib

    layers = args.layers
    cfg = dict(CONFIG_8B, num_hidden_layers=layers)
    pk = peaks()
    nums = model_numbers(cfg, layers)
    gen = torch.Generator().manual_seed(SEED)

    def prompts(n):
        return [torch.randint(0, cfg["vocab_size"], (PROMPT_LEN,), generator=gen).tolist() for _ in range(n)]

    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        max_b = max(args.batch, 64)
        pages = max_b * (CONTEXT // PAGE) + 2 * (CONTEXT // PAGE)
        llm = LLM(d, random_weights_seed=SEED, kvcache_block_size=PAGE, num_kvcache_blocks=pages,
                  max_model_len=CONTEXT, max_num_seqs=max_b, max_num_batched_tokens=8192, seed=SEED,
                  enforce_eager=args.eager, async_decode=not args.sync,
                  decode_weight_copy=False if args.no_weight_copy else None)
    runner = llm.model_runner
    params = SamplingParams(temperature=0.0, max_tokens=CONTEXT - PROMPT_LEN, ignore_eos=True)

    def device_decode(batch: int, steps: int, warmup: int):
        """Prefill `batch` prompts, then time `steps` decode steps with CUDA events around the runner's
        step-and-sample call (the captured graph of the step, its metadata copy before, the read of the
        chosen tokens after)."""
        ids = [f"d{batch}_{i}" for i in range(batch)]
        toks = prompts(batch)
        lens = {}
        for i, p in zip(ids, toks):          # prefill one request per step (8,192-token budget)
            runner.cache.allocate(i, PROMPT_LEN + 1)
            logits = runner.step([StepItem(i, p, 0, [PROMPT_LEN - 1])])
            lens[i] = PROMPT_LEN
        last = {i: 1 for i in ids}

        flight = [None]

        def one():
            """One decode step as generation runs it: launched before the tokens of the step before it have been
            read (they pass on the device), then that step's tokens are read; with --sync, or eagerly, run and read."""
            items = []
            for i in ids:
                runner.cache.allocate(i, lens[i] + 1)
                items.append(StepItem(i, [last[i]], lens[i], [0]))
            sampling = [(0.0, n, lens[i] + 1) for n, i in enumerate(ids)]
            if args.sync or args.eager:
                chosen = runner.run(items, sampling)
            else:
                handle = runner.launch(items, sampling, feed_from=flight[0], feed=list(range(len(ids))))
                chosen = flight[0].read() if flight[0] is not None else [last[i] for i in ids]
                flight[0] = handle
            for i, t in zip(ids, chosen):
                last[i] = t
                lens[i] += 1

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        klib.LAUNCHES = 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx0 = lens[ids[0]]
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = klib.LAUNCHES
        ctx_mid = ctx0 + steps / 2
        if flight[0] is not None:
            flight[0].read()
        for i in ids:
            runner.cache.free(i)
        return ms, launches, ctx_mid

    def e2e_decode(batch: int, steps: int, warmup: int):
        """The same through the public API: token lists in, chosen tokens on the host every step."""
        for p in prompts(batch):
            llm.add_request(p, params)
        while llm.scheduler.waiting:
            llm.step()
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        h0, d0 = llm.h2d_bytes, llm.d2h_bytes
        t0 = time.perf_counter()
        n_tok = 0
        for _ in range(steps):
            _, stats = llm.step()
            n_tok += stats.num_decode_tokens
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        h2d, d2h = (llm.h2d_bytes - h0) / steps, (llm.d2h_bytes - d0) / steps
        llm.abort_all()
        return n_tok / dt, h2d, d2h

    if args.only == "decode":
        ms, launches, _ = device_decode(args.batch, args.steps, args.warmup)
        print(f"decode batch {args.batch}: {ms:.3f} ms/step, {launches} launches")
        return None
    # prefill of one 2,048-token prompt (3 warm-ups)
    p = prompts(1)[0]
    times = []
    for it in range(5):
        runner.cache.allocate("pf", PROMPT_LEN)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([StepItem("pf", p, 0, [PROMPT_LEN - 1])])
        e1.record()
        torch.cuda.synchronize()
        runner.cache.free("pf")
        if it >= 3:
            times.append(e0.elapsed_time(e1))
    pf_ms = sum(times) / len(times)
    if args.only == "prefill":
        print(f"prefill {PROMPT_LEN} tokens: {pf_ms:.3f} ms")
        return None
    pf_flops = prefill_flops(cfg, layers, PROMPT_LEN)

    sampler = ClockSampler()
    sampler.start()
    ms, launches, ctx_mid = device_decode(args.batch, args.steps, args.warmup)
    clocks = sampler.stop()
    e2e_tps, h2d, d2h = e2e_decode(args.batch, args.steps, args.warmup)
    points = {}
    for b in (1, 64):
        pms, _, _ = device_decode(b, max(4, args.steps // 2), 3)
        points[f"decode_b{b}"] = round(b / pms * 1e3, 1)

    # every layer's matrices and the head's table once (the embedding is read only at the batch's rows),
    # plus the keys and values of the live requests at the middle of the timed steps
    step_bytes = nums["weight_bytes"] + args.batch * ctx_mid * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    value = args.batch / ms * 1e3
    return {
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform-random token ids, random weights N(0,0.02), seed 2)",
        "impl": "ours",
        "config": {"model": "Qwen3-8B-shaped", "layers": layers, "layers_full": FULL_LAYERS, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": PAGE,
                   "parallelism": "single-gpu", "l2": "inputs_exceed_l2 (16 GB of weights per step, no flush)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e_tps, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "prefill": {"value": round(PROMPT_LEN / pf_ms * 1e3, 1), "tokens": PROMPT_LEN, "ms": round(pf_ms, 3),
                    "frac": round(pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
    }


def percentile(values, q: float) -> float:
    v = sorted(values)
    return v[min(len(v) - 1, int(q * len(v)))] if v else 0.0


def bench_workload(args) -> dict:
    """The baseline's other two workloads, driven as a user would: ``LLM.add_request`` for every request, then
    ``LLM.step`` until all are done (host token lists in, chosen tokens back on the host every step).

    0.6b: Qwen3-0.6B-shaped, 256 requests with uniform-random prompts of 64 to 4,096 tokens and 256 new tokens
    each under continuous batching.  32b: Qwen3-32B-shaped, 32 requests of 4,096 tokens, 128 new tokens each.
    ``value`` is generated tokens per second over the steps in which every live request decodes (the steady
    state that the roofline describes); ``run`` has the whole run, prompts included."""
    import torch

    from nanohybrid_vlm_b200 import LLM, SamplingParams

    if args.workload == "0.6b":
        cfg, seed, name = dict(CONFIG_06B), 3, "Qwen3-0.6B-shaped"
        n_req, new, context, max_seqs = 256, 256, 8192, 256
        gen = torch.Generator().manual_seed(seed)
        lens = torch.randint(64, 4097, (n_req,), generator=gen).tolist()
        what = "256 requests, prompts U[64,4096], 256 new tokens, continuous batching"
    else:
        cfg, seed, name = dict(CONFIG_32B), 4, "Qwen3-32B-shaped"
        n_req, new, context, max_seqs = 32, 128, 8192, 32
        gen = torch.Generator().manual_seed(seed)
        lens = [4096] * n_req
        what = "batch 32, 4,096-token prompts, 128 new tokens"
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers if args.layers != FULL_LAYERS else full_layers
    cfg["num_hidden_layers"] = layers
    if args.requests:
        n_req, lens = args.requests, lens[:args.requests]
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist() for n in lens]
    pk = peaks()
    nums = model_numbers(cfg, layers)
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        llm = LLM(d, random_weights_seed=seed, kvcache_block_size=PAGE, max_model_len=context, max_num_seqs=max_seqs,
                  max_num_batched_tokens=16384, seed=seed, enforce_eager=args.eager, enable_prefix_cache=False,
                  async_decode=not args.sync)
    params = SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True)
    # warm-up: one short request through prefill and the decode graph of the smallest bucket
    llm.generate([prompts[0][:64]], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True), use_tqdm=False)
    torch.cuda.synchronize()

    sampler = ClockSampler()
    sampler.start()
    for p in prompts:
        llm.add_request(p, params)
    records = []                               # (prefill tokens, decode tokens, seconds, live cache tokens after the step)
    h0, d0 = llm.h2d_bytes, llm.d2h_bytes
    from nanohybrid_vlm_b200.kernels import library as klib
    klib.LAUNCHES = 0
    t_start = time.perf_counter()
    while not llm.is_finished():
        t0 = time.perf_counter()
        _, stats = llm.step()
        dt = time.perf_counter() - t0
        live = sum(s.num_cached_tokens for s in llm.scheduler.running) + sum(s.num_cached_tokens for s in llm.scheduler.waiting)
        records.append((stats.num_prefill_tokens, stats.num_decode_tokens, dt, live))
    torch.cuda.synchronize()
    wall = time.perf_counter() - t_start
    clocks = sampler.stop()
    out_tokens = n_req * new
    most = max(r[1] for r in records)
    steady = [r for r in records if r[0] == 0 and r[1] == most]         # every live request decodes, the batch is full
    if len(steady) > 8:
        steady = steady[2:]                                             # the first ones capture the graph of their bucket
    ms = [r[2] * 1e3 for r in steady]
    mean_ms = sum(ms) / len(ms)
    mean_live = sum(r[3] for r in steady) / len(steady)
    # every layer's matrices and the head's table once (a tied table is the same bytes; the embedding reads only the
    # batch's rows), plus the keys and values of the live requests
    step_bytes = nums["weight_bytes"] + mean_live * nums["kv_bytes_per_token"]
    achieved = step_bytes / (mean_ms * 1e-3) / 1e9
    value = most / mean_ms * 1e3
    metrics = llm.get_completed_request_metrics()
    ttft = [m.ttft_ms for m in metrics if m.ttft_ms is not None]
    return {
        "metric": f"decode tok/s in the steady state of the workload ({name} bf16: {what})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": len(steady), "warmup": 1,
        "ms_per_step": round(mean_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": f"synthetic (uniform-random token ids, random weights N(0,0.02), seed {seed})", "impl": "ours",
        "config": {"model": name, "layers": layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "tied": cfg["tie_word_embeddings"],
                   "global_batch": most, "requests": n_req, "new_tokens": new, "seq_len": context, "page_size": PAGE,
                   "parallelism": "single-gpu", "l2": "inputs_exceed_l2 (weights and cache per step, no flush)",
                   "peaks": pk["source"], "cache_pages": llm.config.num_kvcache_blocks,
                   "decode_weight_copy": bool(llm.config.decode_weight_copy)},
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int((llm.h2d_bytes - h0) / len(records)),
                "d2h_bytes_per_step": int((llm.d2h_bytes - d0) / len(records))},
        "gpu_launches": int(klib.LAUNCHES),
        "run": {"seconds": round(wall, 3), "steps": len(records), "generated_tokens": out_tokens,
                "generated_tok_s": round(out_tokens / wall, 1),
                "prompt_tokens": sum(lens), "all_tok_s": round((out_tokens + sum(lens)) / wall, 1),
                "preemptions": llm.scheduler.num_preemptions,
                "ttft_ms_p50": round(percentile(ttft, 0.5), 1), "ttft_ms_max": round(max(ttft), 1)},
        "step_ms": {"p50": round(percentile(ms, 0.5), 3), "p90": round(percentile(ms, 0.9), 3), "p99": round(percentile(ms, 0.99), 3),
                    "mean_live_cache_tokens": int(mean_live)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clocks,
    }


def bench_breakdown(args) -> dict:
    """Where the time of a decode step (batch 8, context 2,048) and of a 2,048-token prefill goes, by kind of
    kernel: CUDA events around every launch of an EAGER run with few layers (default 2; the layers are alike).
    No profiler is needed.  In an eager run every launch also waits for the host, so a kind's time includes the
    gaps before its launches: compare the shares within a column, and the prefill column (long kernels) more
    than the decode column (kernels of a few microseconds)."""
    import torch

    from nanohybrid_vlm_b200 import LLM
    from nanohybrid_vlm_b200.engine import StepItem
    from nanohybrid_vlm_b200.kernels import ops

    layers = args.layers if args.layers != FULL_LAYERS else 2
    cfg = dict(CONFIG_8B, num_hidden_layers=layers)
    gen = torch.Generator().manual_seed(SEED)
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        llm = LLM(d, random_weights_seed=SEED, kvcache_block_size=PAGE, num_kvcache_blocks=10 * (CONTEXT // PAGE),
                  max_model_len=CONTEXT, max_num_seqs=8, max_num_batched_tokens=8192, seed=SEED, enforce_eager=True)
    runner = llm.model_runner
    kinds = {"linear": "gemm", "swiglu_first_half": "gemm", "rmsnorm": "norm", "qk_norm_rope_store": "rope_store",
             "attention": "attention", "attention_decode_fused": "attention", "silu_mul": "silu", "embed": "embed",
             "sample": "sample", "to_f32": "convert"}
    events, depth = [], [0]
    stock = {name: getattr(ops, name) for name in kinds}

    def timed(name, fn):
        def call(*a, **kw):
            if depth[0]:                         # a launch inside a launch that is timed already
                return fn(*a, **kw)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            depth[0] += 1
            e0.record()
            try:
                return fn(*a, **kw)
            finally:
                e1.record()
                depth[0] -= 1
                events.append((kinds[name], e0, e1))
        return call

    def measure(step_fn, repeats):
        for _ in range(3):
            step_fn()
        torch.cuda.synchronize()
        for name, fn in stock.items():
            setattr(ops, name, timed(name, fn))
        events.clear()
        w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        try:
            w0.record()
            for _ in range(repeats):
                step_fn()
            w1.record()
            torch.cuda.synchronize()
        finally:
            for name, fn in stock.items():
                setattr(ops, name, fn)
        total = {}
        for kind, e0, e1 in events:
            total[kind] = total.get(kind, 0.0) + e0.elapsed_time(e1) * 1e3 / repeats
        out = {k: round(v, 1) for k, v in sorted(total.items(), key=lambda kv: -kv[1])}
        out["step_us"] = round(w0.elapsed_time(w1) * 1e3 / repeats, 1)
        return out

    prompts = [torch.randint(0, cfg["vocab_size"], (PROMPT_LEN,), generator=gen).tolist() for _ in range(8)]

    def prefill():
        runner.cache.allocate("pf", PROMPT_LEN)
        runner.step([StepItem("pf", prompts[0], 0, [PROMPT_LEN - 1])])
        runner.cache.free("pf")

    pf = measure(prefill, 3)
    lens = {}
    for i, p in enumerate(prompts):
        runner.cache.allocate(i, PROMPT_LEN + 1)
        runner.step([StepItem(i, p, 0, [])])
        lens[i] = PROMPT_LEN

    def decode():
        items = []
        for i in lens:
            runner.cache.allocate(i, lens[i] + 1)
            items.append(StepItem(i, [1], lens[i], [0]))
            lens[i] += 1
        runner.run(items, [(0.0, 1, lens[i]) for i in lens])

    dec = measure(decode, 8)
    return {"breakdown_us": {"decode_b8_ctx2048": dec, "prefill_2048": pf}, "layers": layers, "model": "Qwen3-8B-shaped",
            "dtype": "bf16", "how": "CUDA events around each launch of an eager run; the gaps before a kind's launches count "
            "toward it; the head, the sampler and the embedding run once per step, the rest once per layer"}


def _unavailable(reason: str) -> dict:
    return {"impl": "reference", "unavailable": " ".join(str(reason).split())[:300]}


def _write_reference_model(folder: str, cfg: dict) -> None:
    """A model folder the reference can open: config.json, a stand-in tokenizer (one word per token id; the
    reference's engine insists on one, nanovllm/inputs.py:186-193) and safetensors shards with the same
    kind of random weights as the other arm, written layer by layer."""
    import torch
    from safetensors.torch import save_file
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    from nanohybrid_vlm_b200.weights.random_init import tensor_seed

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(cfg, eos_token_id=0, bos_token_id=0), f)
    vocab = {f"t{i}": i for i in range(cfg["vocab_size"])}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="t0", unk_token="t0").save_pretrained(folder)

    H, nq, nkv, d, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                           cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])

    def draw(name, shape, norm=False):
        gen = torch.Generator(device="cuda").manual_seed(tensor_seed(SEED, name))
        t = torch.empty(shape, dtype=torch.float32, device="cuda").normal_(0.0, 0.01 if norm else 0.02, generator=gen)
        return ((1.0 + t) if norm else t).to(torch.bfloat16).cpu()

    shard = {n: draw(n, s) for n, s in (("model.embed_tokens.weight", (V, H)), ("lm_head.weight", (V, H)))}
    shard["model.norm.weight"] = draw("model.norm.weight", (H,), norm=True)
    save_file(shard, os.path.join(folder, "model-head.safetensors"))
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shard = {}
        for n, s in (("self_attn.q_proj.weight", (nq * d, H)), ("self_attn.k_proj.weight", (nkv * d, H)),
                     ("self_attn.v_proj.weight", (nkv * d, H)), ("self_attn.o_proj.weight", (H, nq * d)),
                     ("mlp.gate_proj.weight", (I, H)), ("mlp.up_proj.weight", (I, H)), ("mlp.down_proj.weight", (H, I))):
            shard[p + n] = draw(p + n, s)
        for n, s in (("input_layernorm.weight", (H,)), ("post_attention_layernorm.weight", (H,)),
                     ("self_attn.q_norm.weight", (d,)), ("self_attn.k_norm.weight", (d,))):
            shard[p + n] = draw(p + n, s, norm=True)
        save_file(shard, os.path.join(folder, f"model-layer-{i:03d}.safetensors"))


def bench_reference(args) -> dict:
    """The unmodified reference (installed under baseline/_ref) through its own public API:
    LLM(path).add_request / step, the same model shape, prompts, batch and timing as the other arm."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "nanovllm")):
        return _unavailable("baseline/_ref is not installed (pip install --no-index --no-deps --target baseline/_ref <reference>)")
    try:
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device")
        sys.path.insert(0, ref_root)
        from nanovllm import LLM, SamplingParams
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"the reference cannot be imported: {type(e).__name__}: {e}")
    layers = args.layers
    cfg = dict(CONFIG_8B, num_hidden_layers=layers)
    gen = torch.Generator().manual_seed(SEED)

    def prompts(n):
        return [torch.randint(0, cfg["vocab_size"], (PROMPT_LEN,), generator=gen).tolist() for _ in range(n)]

    folder = tempfile.mkdtemp(prefix="ref_model_")
    try:
        _write_reference_model(folder, cfg)
        llm = LLM(folder, max_model_len=CONTEXT, max_num_seqs=max(args.batch, 64), kvcache_block_size=PAGE,
                  enforce_eager=args.eager, gpu_memory_utilization=0.85)
        sp = SamplingParams(temperature=0.0, max_tokens=CONTEXT - PROMPT_LEN, ignore_eos=True)

        def decode(batch, steps, warmup):
            for p in prompts(batch):
                llm.add_request(p, sp)
            while llm.scheduler.waiting:
                llm.step()
            for _ in range(warmup):
                llm.step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record()
            for _ in range(steps):
                llm.step()
            e1.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            for seq in list(llm.scheduler.running):       # drop the requests: their pages go back
                llm.scheduler.block_manager.deallocate(seq)
            llm.scheduler.running.clear()
            return e0.elapsed_time(e1) / steps, batch * steps / wall

        sampler = ClockSampler()
        sampler.start()
        ms, e2e_tps = decode(args.batch, args.steps, args.warmup)
        clocks = sampler.stop()
        points = {}
        for b in (1, 64):
            pms, _ = decode(b, max(4, args.steps // 2), 3)
            points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
        times = []
        for it in range(5):
            llm.add_request(prompts(1)[0], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            llm.step()
            torch.cuda.synchronize()
            if it >= 3:
                times.append((time.perf_counter() - t0) * 1e3)
        pf_ms = sum(times) / len(times)
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"the reference does not run here: {type(e).__name__}: {e}")
    finally:
        import shutil
        shutil.rmtree(folder, ignore_errors=True)
    pk = peaks()
    nums = model_numbers(cfg, layers)
    step_bytes = nums["weight_bytes"] + args.batch * (PROMPT_LEN + args.warmup + args.steps / 2) * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    return {
        "metric": METRIC, "value": round(args.batch / ms * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform-random token ids, random weights N(0,0.02), seed 2)",
        "impl": "reference",
        "config": {"model": "Qwen3-8B-shaped", "layers": layers, "layers_full": FULL_LAYERS, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": PAGE,
                   "parallelism": "single-gpu", "l2": "inputs_exceed_l2 (16 GB of weights per step, no flush)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e_tps, 1), "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
        "gpu_launches": None,
        "prefill": {"value": round(PROMPT_LEN / pf_ms * 1e3, 1), "tokens": PROMPT_LEN, "ms": round(pf_ms, 3),
                    "frac": round(prefill_flops(cfg, layers, PROMPT_LEN) / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "clocks": clocks,
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--eager", action="store_true", help="no CUDA graphs (for per-kernel profiling)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run only the decode steps or only the prefill step (profiling); prints no JSON line")
    ap.add_argument("--layers", type=int, default=FULL_LAYERS,
                    help="fewer layers than the full model (sizes of a layer unchanged); recorded in config")
    ap.add_argument("--workload", default="8b", choices=["8b", "0.6b", "32b"],
                    help="8b: the headline line; 0.6b / 32b: the baseline's other workloads through LLM.add_request / step")
    ap.add_argument("--sync", action="store_true", help="read every decode step's tokens before the next is launched (async_decode off)")
    ap.add_argument("--no-weight-copy", action="store_true",
                    help="decode from the row-major matrices (no per-SM copies of the weights: half the weight memory)")
    ap.add_argument("--requests", type=int, default=0, help="fewer requests than the workload names (trying it out)")
    ap.add_argument("--breakdown", action="store_true",
                    help="time by kind of kernel in an eager run with --layers layers (default 2); prints one JSON line")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (N=1 only)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.breakdown:
        out = bench_breakdown(args)
    elif args.workload != "8b":
        if args.impl == "reference":
            out = _unavailable("the reference arm is run for the headline workload only")
        else:
            out = bench_workload(args)
    else:
        out = bench_reference(args) if args.impl == "reference" else bench_ours(args)
    if out is not None:
        print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
