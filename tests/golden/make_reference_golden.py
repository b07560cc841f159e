"""Runs the reference's OWN Qwen3 model code (Bluexvy/NanoHybrid-VLM, nanovllm/models/qwen3.py) on the
CPU, on the two tiny random models of tests/conftest.py, and stores the logits of a few prompts in
``reference_logits_<name>.npz`` beside this script.  ``tests/test_plain_vs_reference.py`` compares the
plain implementation with these files, so the oracle of all other tests is anchored on the
reference's code for everything but the attention core.

What had to be stood in for, because it has no CPU form: ``flash_attn_varlen_func`` (replaced by a
masked softmax over the packed sequences) and the process group that the reference's layers
query at construction (a one-rank gloo group).  ``torch.compile`` is switched off.

The reference cannot run in float32: its RMSNorm works in place on ``x.float()``, which for a float32
input is the input itself, so the residual stream is overwritten (nanovllm/layers/layernorm.py:21-25,
34-39); it is written for bfloat16 checkpoints.  It is therefore run twice: in float64 (every cast
copies, the norm statistics and the rotation are still rounded to float32 where the reference says
so), which the plain implementation in float32 must match closely, and in bfloat16, which pins the
places where the reference rounds.

    python tests/golden/make_reference_golden.py /path/to/NanoHybrid-VLM
"""
import os
import sys
import tempfile
from types import SimpleNamespace

os.environ["TORCHDYNAMO_DISABLE"] = "1"

import numpy as np
import torch
import torch.distributed as dist
from safetensors import safe_open

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, ".."))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

PROMPT_LENGTHS = (5, 17, 33)


def masked_attention(q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k, softmax_scale, causal,
                     block_table=None):
    out = torch.empty_like(q)
    group = q.shape[1] // k.shape[1]
    for s in range(len(cu_seqlens_q) - 1):
        a, b = int(cu_seqlens_q[s]), int(cu_seqlens_q[s + 1])
        ct = torch.float64 if q.dtype == torch.float64 else torch.float32
        qs = q[a:b].to(ct).transpose(0, 1)
        ks = k[a:b].to(ct).transpose(0, 1).repeat_interleave(group, 0)
        vs = v[a:b].to(ct).transpose(0, 1).repeat_interleave(group, 0)
        sc = qs @ ks.transpose(1, 2) * softmax_scale
        n = b - a
        sc = sc.masked_fill(~torch.ones(n, n, dtype=torch.bool).tril(), float("-inf"))
        out[a:b] = (torch.softmax(sc, -1) @ vs).transpose(0, 1).to(q.dtype)
    return out


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from conftest import TINY
    from nanohybrid_vlm_b200.weights import write_random_model

    store = tempfile.mkdtemp()
    dist.init_process_group("gloo", init_method=f"file://{store}/pg", world_size=1, rank=0)
    import nanovllm.layers.attention as ref_attention
    from nanovllm.models.qwen3 import Qwen3ForCausalLM
    from nanovllm.utils.context import set_context
    ref_attention.flash_attn_varlen_func = masked_attention

    for name, (cfg, seed) in TINY.items():
        d = os.path.join(store, name)
        write_random_model(d, cfg, seed)
        hf = SimpleNamespace(**cfg, rope_scaling=None)
        results = {}
        for dtype in (torch.float64, torch.bfloat16):
            results[dtype] = run_reference(Qwen3ForCausalLM, set_context, hf, cfg, d, seed, dtype)
        prompts = results[torch.float64][0]
        np.savez_compressed(os.path.join(HERE, f"reference_logits_{name}.npz"),
                            prompts=np.array(sum(prompts, []), dtype=np.int32), lengths=np.array(PROMPT_LENGTHS),
                            last_logits_f64=results[torch.float64][1], all_logits_f64=results[torch.float64][2],
                            last_logits_bf16=results[torch.bfloat16][1], all_logits_bf16=results[torch.bfloat16][2])
        print(name, "logits", results[torch.float64][2].shape)


def run_reference(Qwen3ForCausalLM, set_context, hf, cfg, d, seed, dtype):
    if True:
        torch.set_default_dtype(dtype)
        model = Qwen3ForCausalLM(hf)
        torch.set_default_dtype(torch.float32)
        params = dict(model.named_parameters())
        nq, nkv, hd, inter = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                              cfg["intermediate_size"])
        with safe_open(os.path.join(d, "model.safetensors"), framework="pt") as f, torch.no_grad():
            for key in f.keys():
                t = f.get_tensor(key)
                # the reference's own packing: q|k|v rows and gate|up rows (nanovllm/layers/linear.py:102-108,153-167)
                for part, (packed, off, rows) in {"q_proj": ("qkv_proj", 0, nq * hd), "k_proj": ("qkv_proj", nq * hd, nkv * hd),
                                                  "v_proj": ("qkv_proj", (nq + nkv) * hd, nkv * hd),
                                                  "gate_proj": ("gate_up_proj", 0, inter),
                                                  "up_proj": ("gate_up_proj", inter, inter)}.items():
                    if f".{part}." in key:
                        params[key.replace(part, packed)].data[off:off + rows].copy_(t)
                        break
                else:
                    params[key].data.copy_(t)
        if cfg["tie_word_embeddings"]:
            model.lm_head.weight.data = model.model.embed_tokens.weight.data
        rng = np.random.default_rng(1000 + seed)
        prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in PROMPT_LENGTHS]
        ids = torch.tensor(sum(prompts, []))
        pos = torch.cat([torch.arange(len(p)) for p in prompts])
        cu = torch.tensor(np.cumsum([0] + [len(p) for p in prompts]), dtype=torch.int32)
        set_context(True, cu, cu, max(PROMPT_LENGTHS), max(PROMPT_LENGTHS), None, None, None)
        with torch.no_grad():
            hidden = model(ids, pos)
            last = model.compute_logits(hidden).float().numpy()          # last row of each prompt
            every = torch.nn.functional.linear(hidden, model.lm_head.weight).float().numpy()
        return prompts, last.astype(np.float32), every.astype(np.float32)


if __name__ == "__main__":
    main(sys.argv[1])
