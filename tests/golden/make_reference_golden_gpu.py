"""Runs the reference's OWN Qwen3 model code (Bluexvy/NanoHybrid-VLM, nanovllm/models/qwen3.py) in bfloat16
on a GPU with its REAL attention calls (``flash_attn_varlen_func`` and ``flash_attn_with_kvcache`` of
nanovllm/layers/attention.py:62-74, its Triton cache store :10-40, its compiled norm / rotation / SiLU ops), on
the two tiny random models of tests/conftest.py, and stores the logits in ``reference_logits_<name>_gpu.npz``
beside this script.  ``tests/test_plain_vs_reference.py`` compares the plain implementation with these files on
the CPU, so the attention core of the oracle (scale, which keys a query sees when earlier context lies in the
cache, which KV head a query head reads) is pinned on the reference's output too, not on a reading of it.

Nothing of the reference is replaced.  What this script does itself is what the reference's model runner does
around the model: it makes the paged cache tensor and hands each attention layer its slice
(nanovllm/engine/model_runner.py:870-905), and sets the step's context (``set_context``) as
``prepare_prefill`` / ``prepare_decode`` do (:924-1146).  Three routes per model:

* ``whole``: every prompt whole, packed in one varlen step (no block tables);
* ``chunk``: the first part of every prompt in one step, then a second portion that attends to the first
  through the cache (block tables, more keys than queries: the causal mask's bottom-right alignment);
* ``decode``: the last tokens one per step, all prompts as one batch (``flash_attn_with_kvcache``).

A second part drives the reference's engine itself (``LLM.add_request`` / ``LLM.step``, its scheduler, block
manager and graphs off) on the same folder and records the logits that its ``compute_logits`` returned and the
greedy tokens; it is stored when it ran (``engine_ok``).

    python tests/golden/make_reference_golden_gpu.py [/path/to/NanoHybrid-VLM or its installed copy [output folder]]
"""
import json
import os
import sys
import tempfile
from types import SimpleNamespace

import numpy as np
import torch
import torch.distributed as dist
from safetensors import safe_open
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, ".."))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

PAGE = 256                      # the reference's page size (nanovllm/config.py:159)
LENGTHS = {"A": (5, 17, 33, 120, 250), "B": (1, 9, 40, 71, 300, 400)}
NEW_TOKENS = 6                  # greedy tokens through the engine


def pack(out: dict) -> dict:
    """Logits are bfloat16 numbers widened to float32: keep their upper 16 bits only (``<name>__bf16``)."""
    packed = {}
    for k, v in out.items():
        if isinstance(v, np.ndarray) and v.dtype == np.float32:
            bits = np.ascontiguousarray(v).view(np.uint32)
            assert not (bits & 0xFFFF).any(), f"{k} is not made of bfloat16 numbers"
            packed[k + "__bf16"] = (bits >> 16).astype(np.uint16)
        else:
            packed[k] = v
    return packed


def load_into(model, cfg, folder):
    """The reference's own packing: q|k|v rows and gate|up rows (nanovllm/layers/linear.py:102-108,153-167)."""
    params = dict(model.named_parameters())
    nq, nkv, hd, inter = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"])
    packed = {"q_proj": ("qkv_proj", 0, nq * hd), "k_proj": ("qkv_proj", nq * hd, nkv * hd),
              "v_proj": ("qkv_proj", (nq + nkv) * hd, nkv * hd), "gate_proj": ("gate_up_proj", 0, inter),
              "up_proj": ("gate_up_proj", inter, inter)}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f, torch.no_grad():
        for key in f.keys():
            t = f.get_tensor(key)
            for part, (name, off, rows) in packed.items():
                if f".{part}." in key:
                    params[key.replace(part, name)].data[off:off + rows].copy_(t)
                    break
            else:
                if key in params:
                    params[key].data.copy_(t)
    if cfg["tie_word_embeddings"]:
        model.lm_head.weight.data = model.model.embed_tokens.weight.data


def direct_routes(Qwen3ForCausalLM, set_context, cfg, folder, prompts):
    dev = "cuda"
    hf = SimpleNamespace(**cfg, rope_scaling=None)
    torch.set_default_dtype(torch.bfloat16)
    torch.set_default_device(dev)
    model = Qwen3ForCausalLM(hf)
    torch.set_default_device("cpu")
    torch.set_default_dtype(torch.float32)
    load_into(model, cfg, folder)
    L, nkv, d = cfg["num_hidden_layers"], cfg["num_key_value_heads"], cfg["head_dim"]
    pages_per = [-(-len(p) // PAGE) for p in prompts]
    num_pages = sum(pages_per) + 3
    kv = torch.zeros(2, L, num_pages, PAGE, nkv, d, dtype=torch.bfloat16, device=dev)
    layer = 0
    for module in model.modules():
        if hasattr(module, "k_cache") and hasattr(module, "v_cache"):
            module.k_cache, module.v_cache = kv[0, layer], kv[1, layer]
            layer += 1
    assert layer == L
    # pages handed out in an order that is not the order of the requests
    order = list(range(num_pages))[::-1]
    tables, at = [], 0
    for n in pages_per:
        tables.append(order[at:at + n])
        at += n
    width = max(pages_per)
    table_t = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32, device=dev)

    def slots(i, a, b):
        return [tables[i][p // PAGE] * PAGE + p % PAGE for p in range(a, b)]

    def i32(x):
        return torch.tensor(x, dtype=torch.int32, device=dev)

    def prefill(parts, with_tables):
        """parts: (request, first token, one past the last).  Returns logits of every row."""
        ids, pos, slot, cu_q, cu_k = [], [], [], [0], [0]
        for i, a, b in parts:
            ids += prompts[i][a:b]
            pos += list(range(a, b))
            slot += slots(i, a, b)
            cu_q.append(cu_q[-1] + b - a)
            cu_k.append(cu_k[-1] + b)
        rows = [i for i, _, _ in parts]
        set_context(True, i32(cu_q), i32(cu_k if with_tables else cu_q), max(b - a for _, a, b in parts),
                    max(b for _, _, b in parts) if with_tables else max(b - a for _, a, b in parts), i32(slot), None,
                    table_t[rows].contiguous() if with_tables else None)
        hidden = model(torch.tensor(ids, device=dev), torch.tensor(pos, device=dev))
        return torch.nn.functional.linear(hidden, model.lm_head.weight).float().cpu().numpy()

    out = {}
    with torch.inference_mode():
        every = prefill([(i, 0, len(p)) for i, p in enumerate(prompts)], False)
        at = 0
        for i, p in enumerate(prompts):
            out[f"whole_{i}"] = every[at:at + len(p)]
            at += len(p)
        kv.zero_()
        first = [max(1, len(p) * 2 // 5) for p in prompts]
        tail = [min(8, len(p) // 3) for p in prompts]
        prefill([(i, 0, first[i]) for i in range(len(prompts))], False)
        parts = [(i, first[i], len(p) - tail[i]) for i, p in enumerate(prompts) if len(p) - tail[i] > first[i]]
        every = prefill(parts, True)
        at = 0
        for i, a, b in parts:
            out[f"chunk_{i}"] = every[at:at + b - a]
            out[f"chunk_{i}_start"] = np.array(a)
            at += b - a
        done = [len(p) - tail[i] for i, p in enumerate(prompts)]
        decoded = {i: [] for i in range(len(prompts))}
        while any(done[i] < len(p) for i, p in enumerate(prompts)):
            live = [i for i, p in enumerate(prompts) if done[i] < len(p)]
            set_context(False, slot_mapping=i32([slots(i, done[i], done[i] + 1)[0] for i in live]),
                        context_lens=i32([done[i] + 1 for i in live]), block_tables=table_t[live].contiguous())
            hidden = model(torch.tensor([prompts[i][done[i]] for i in live], device=dev),
                           torch.tensor([done[i] for i in live], device=dev))
            lg = model.compute_logits(hidden).float().cpu().numpy()
            for r, i in enumerate(live):
                decoded[i].append(lg[r])
                done[i] += 1
        for i, rows in decoded.items():
            if rows:
                out[f"decode_{i}"] = np.stack(rows)
                out[f"decode_{i}_start"] = np.array(len(prompts[i]) - len(rows))
    del model, kv
    torch.cuda.empty_cache()
    return out


def engine_route(reference_root, cfg, folder, prompts):
    """The reference's engine on the folder: its logits at the last row of every step's requests, and its greedy
    tokens.  Needs what its loader and input processor insist on: ``lm_head.weight`` in the file even when the
    head is tied, and a tokenizer."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    eng = tempfile.mkdtemp(prefix="ref_engine_")
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    if cfg["tie_word_embeddings"]:
        tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, os.path.join(eng, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(eng, "config.json"), "w") as f:
        json.dump(dict(cfg, eos_token_id=0, bos_token_id=0), f)
    tok = Tokenizer(models.WordLevel({f"t{i}": i for i in range(cfg["vocab_size"])}, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="t0", unk_token="t0").save_pretrained(eng)

    from nanovllm import LLM, SamplingParams
    llm = LLM(eng, max_model_len=cfg["max_position_embeddings"], max_num_seqs=8, kvcache_block_size=PAGE,
              enforce_eager=True, gpu_memory_utilization=0.5, max_num_batched_tokens=2048)
    model = llm.model_runner.model
    seen = []
    stock = model.compute_logits

    def recording(hidden):
        lg = stock(hidden)
        seen.append(lg.float().cpu().numpy())
        return lg

    model.compute_logits = recording
    sp = SamplingParams(temperature=0.0, max_tokens=NEW_TOKENS, ignore_eos=True)
    out = llm.generate([list(p) for p in prompts], sp, use_tqdm=False)
    model.compute_logits = stock
    tokens = np.array([o["token_ids"] for o in out], dtype=np.int32)
    return tokens, seen


def main(reference_root: str, out_dir: str) -> None:
    sys.path.insert(0, reference_root)
    from conftest import TINY
    from nanohybrid_vlm_b200.weights import write_random_model

    store = tempfile.mkdtemp()
    dist.init_process_group("gloo", init_method=f"file://{store}/pg", world_size=1, rank=0)
    from nanovllm.models.qwen3 import Qwen3ForCausalLM
    from nanovllm.utils.context import set_context

    todo = []
    for name, (cfg, seed) in TINY.items():
        cfg = dict(cfg, torch_dtype="bfloat16")
        folder = os.path.join(store, name)
        write_random_model(folder, cfg, seed)          # the file holds the weights rounded to bfloat16
        rng = np.random.default_rng(2000 + seed)
        prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in LENGTHS[name]]
        out = direct_routes(Qwen3ForCausalLM, set_context, cfg, folder, prompts)
        out["prompts"] = np.array(sum(prompts, []), dtype=np.int32)
        out["lengths"] = np.array(LENGTHS[name])
        todo.append((name, cfg, folder, prompts, out))
        print(name, "direct routes done:", sorted(k for k in out if not k.endswith("_start"))[:4], "...")
    dist.destroy_process_group()
    import subprocess
    for name, cfg, folder, prompts, out in todo:
        # one process per model: the engine keeps its cache and its process group until the process ends
        part = os.path.join(store, f"engine_{name}.npz")
        with open(os.path.join(store, f"engine_{name}.json"), "w") as f:
            json.dump({"cfg": cfg, "folder": folder, "prompts": prompts, "out": part}, f)
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--engine", reference_root,
                            os.path.join(store, f"engine_{name}.json")])
        if r.returncode == 0 and os.path.isfile(part):
            with np.load(part) as data:
                out.update({k: data[k] for k in data.files})
            out["engine_ok"] = np.array(1)
            print(name, "engine route done:", out["engine_tokens"].tolist())
        else:
            out["engine_ok"] = np.array(0)
            print(name, f"engine route did not run (exit code {r.returncode})")
        os.makedirs(out_dir, exist_ok=True)
        np.savez_compressed(os.path.join(out_dir, f"reference_logits_{name}_gpu.npz"), **pack(out))


def engine_main(reference_root: str, job_file: str) -> None:
    sys.path.insert(0, reference_root)
    with open(job_file) as f:
        job = json.load(f)
    tokens, seen = engine_route(reference_root, job["cfg"], job["folder"], job["prompts"])
    out = {"engine_tokens": tokens, "engine_steps": np.array(len(seen))}
    for k, lg in enumerate(seen):
        out[f"engine_logits_{k}"] = lg
    np.savez_compressed(job["out"], **out)


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "--engine":
        engine_main(sys.argv[2], sys.argv[3])
        sys.exit(0)
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "..", "..", "baseline", "_ref"),
         sys.argv[2] if len(sys.argv) > 2 else HERE)
