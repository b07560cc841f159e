"""Command line of the engine.

    python -m nanohybrid_vlm_b200.cli generate --model DIR --prompt-ids 1,2,3 [--prompt-ids 4,5] [options]
    python -m nanohybrid_vlm_b200.cli make-random --model DIR --config CONFIG.json --seed N
    python -m nanohybrid_vlm_b200.cli replay --model DIR --dtype D --out DIR --max-tokens N < trace.jsonl
    python -m nanohybrid_vlm_b200.cli bench [--workload 8b|0.6b|32b] [--breakdown] [...]       (bench.py's options)

Options carry the names of the engine's options (and, where the reference has them, its names:
nanovllm/config.py:9-152, nanovllm/sampling_params.py:5-15), with dashes for underscores.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _add_engine_options(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
    ap.add_argument("--dtype", default=None, choices=["bfloat16", "float32"], help="default: the checkpoint's")
    ap.add_argument("--max-num-batched-tokens", type=int, default=16384)
    ap.add_argument("--max-num-seqs", type=int, default=512)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--kvcache-block-size", type=int, default=256)
    ap.add_argument("--num-kvcache-blocks", type=int, default=-1)
    ap.add_argument("--scheduler-policy", default="decode_first", choices=["decode_first", "prefill_first"])
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--enable-prefix-cache", dest="enable_prefix_cache", action="store_true", default=None,
                    help="share pages between requests with a common prefix (default: where the model allows it)")
    ap.add_argument("--no-prefix-cache", dest="enable_prefix_cache", action="store_false")
    ap.add_argument("--decode-weight-copy", dest="decode_weight_copy", action="store_true", default=None,
                    help="keep a second copy of the matrices a decode step streams, laid out per SM (default: when it fits)")
    ap.add_argument("--no-decode-weight-copy", dest="decode_weight_copy", action="store_false")
    ap.add_argument("--profile-ranges", action="store_true", help="NVTX ranges around the step and every layer run")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--random-weights", action="store_true",
                    help="ignore the folder's safetensors and make weights on the device from --seed")


def cmd_generate(args) -> int:
    from . import LLM, SamplingParams
    prompts: list = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids or []]
    prompts += list(args.prompt or [])
    if not prompts:
        print("give --prompt-ids or --prompt", file=sys.stderr)
        return 2
    llm = LLM(args.model, dtype=args.dtype, max_num_batched_tokens=args.max_num_batched_tokens,
              max_num_seqs=args.max_num_seqs, max_model_len=args.max_model_len,
              gpu_memory_utilization=args.gpu_memory_utilization, kvcache_block_size=args.kvcache_block_size,
              num_kvcache_blocks=args.num_kvcache_blocks, scheduler_policy=args.scheduler_policy,
              enforce_eager=args.enforce_eager, seed=args.seed, enable_prefix_cache=args.enable_prefix_cache,
              decode_weight_copy=args.decode_weight_copy, profile_ranges=args.profile_ranges,
              random_weights_seed=args.seed if args.random_weights else None)
    sp = SamplingParams(temperature=args.temperature, max_tokens=args.max_tokens, ignore_eos=args.ignore_eos,
                        seed=args.sampling_seed)
    for prompt, out in zip(prompts, llm.generate(prompts, sp, use_tqdm=not args.quiet)):
        print(json.dumps({"prompt": prompt, "token_ids": out["token_ids"], "text": out["text"]}))
    return 0


def cmd_make_random(args) -> int:
    from .weights import write_random_model
    with open(args.config) as f:
        config = json.load(f)
    write_random_model(args.model, config, args.seed)
    print(f"wrote {os.path.join(args.model, 'config.json')} and model.safetensors (seed {args.seed})")
    return 0


def cmd_replay(args, rest) -> int:
    script = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    os.execv(sys.executable, [sys.executable, script, *rest])


def cmd_bench(rest) -> int:
    script = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    if not os.path.isfile(script):
        print(f"bench.py is not beside the package ({script})", file=sys.stderr)
        return 2
    os.execv(sys.executable, [sys.executable, script, *rest])


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        return cmd_replay(None, argv[1:])
    if argv and argv[0] == "bench":
        return cmd_bench(argv[1:])
    ap = argparse.ArgumentParser(prog="nanohybrid_vlm_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate from token-id or text prompts")
    _add_engine_options(g)
    g.add_argument("--prompt-ids", action="append", help="comma-separated token ids; may be repeated")
    g.add_argument("--prompt", action="append", help="text (needs the folder's tokenizer); may be repeated")
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--max-tokens", type=int, default=64)
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--sampling-seed", type=int, default=None)
    g.add_argument("--quiet", action="store_true")
    m = sub.add_parser("make-random", help="write a model folder with random weights")
    m.add_argument("--model", required=True)
    m.add_argument("--config", required=True, help="a config.json to copy the sizes from")
    m.add_argument("--seed", type=int, default=0)
    sub.add_parser("replay", help="trace replay; arguments as bin/trace_run")
    sub.add_parser("bench", help="the benchmark program; arguments as bench.py")
    args = ap.parse_args(argv)
    return {"generate": cmd_generate, "make-random": cmd_make_random}[args.command](args)


if __name__ == "__main__":
    sys.exit(main())
