"""Plain, slow Qwen3-dense implementation used as the oracle by the tests.

Whole sequences, no cache, one function per part, PyTorch on the CPU (or any
device the tensors live on).  It shares no code with the engine: it reads
``config.json`` and ``model.safetensors`` itself and uses the checkpoint's own
tensor names (separate q/k/v and gate/up matrices).

Every function cites the file:line of Bluexvy/NanoHybrid-VLM whose formula it
restates, and the whole is held to the reference's own output twice
(``tests/test_plain_vs_reference.py``): ``tests/golden/make_reference_golden.py``
ran the reference's ``Qwen3ForCausalLM`` on the CPU (its flash-attn call
replaced by a masked softmax, because that package has no CPU kernel), and
``tests/golden/make_reference_golden_gpu.py`` ran it on a B200 with its real
attention calls: whole prompts, portions that attend to earlier context in
the paged cache, single decoded tokens, and its engine generating greedily.
The logits of both lie under ``tests/golden/``.

``dtype`` is the storage dtype between ops (the reference's model dtype):
float32 makes every cast an identity; bfloat16 rounds at the places where the
reference rounds.  Matrix products accumulate in float32 and round once.
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch
from safetensors import safe_open


# --------------------------------------------------------------------------- parts

def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x @ W^T, W stored [out, in] (nanovllm/layers/linear.py:40,66)."""
    return (x.float() @ w.float().t()).to(x.dtype)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """nanovllm/layers/layernorm.py:16-26: statistics in fp32, cast back, then times w."""
    dt = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return xf.to(dt) * w.to(dt)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float):
    """nanovllm/layers/layernorm.py:28-40: fp32 sum, residual rounded once, the norm
    uses the unrounded sum."""
    dt = x.dtype
    s = x.float() + residual.float()
    new_residual = s.to(dt)
    var = s.pow(2).mean(dim=-1, keepdim=True)
    y = (s * torch.rsqrt(var + eps)).to(dt) * w.to(dt)
    return y, new_residual


def rope_table(head_dim: int, max_position: int, theta: float):
    """nanovllm/layers/rotary_embedding.py:83-89: fp32 inverse frequencies and angles."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    t = torch.arange(max_position, dtype=torch.float)
    freqs = torch.einsum("i,j->ij", t, inv_freq)
    return freqs.cos(), freqs.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """nanovllm/layers/rotary_embedding.py:6-14: half-split rotation in fp32.
    x [T, heads, d]; cos/sin [T, d/2]."""
    x1, x2 = torch.chunk(x.float(), 2, dim=-1)
    c, s = cos[:, None, :], sin[:, None, :]
    y1 = x1 * c - x2 * s
    y2 = x2 * c + x1 * s
    return torch.cat((y1, y2), dim=-1).to(x.dtype)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """Causal softmax attention of one whole sequence with grouped heads
    (the call at nanovllm/layers/attention.py:67-70; scale d^-0.5 from
    nanovllm/models/qwen3.py:39).  q [T,nq,d], k/v [T,nkv,d]; query head h reads
    KV head h // (nq/nkv).  Scores and softmax in fp32, output cast to q's dtype."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    qf = q.float().transpose(0, 1)                                   # [nq,T,d]
    kf = k.float().transpose(0, 1).repeat_interleave(group, dim=0)   # [nq,T,d]
    vf = v.float().transpose(0, 1).repeat_interleave(group, dim=0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale
    mask = torch.ones(T, T, dtype=torch.bool, device=q.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf)                                          # [nq,T,d]
    return o.transpose(0, 1).to(q.dtype)


def attention_mixer(x, positions, w, prefix, cfg, cos, sin):
    """nanovllm/models/qwen3.py:72-88: QKV, per-head q/k RMSNorm before RoPE,
    attention, output projection."""
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    T = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"]).view(T, nq, d)
    k = linear(x, w[prefix + "k_proj.weight"]).view(T, nkv, d)
    v = linear(x, w[prefix + "v_proj.weight"]).view(T, nkv, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
    q = apply_rope(q, cos[positions], sin[positions])
    k = apply_rope(k, cos[positions], sin[positions])
    o = causal_attention(q, k, v, d ** -0.5)
    return linear(o.reshape(T, nq * d), w[prefix + "o_proj.weight"])


def swiglu_mlp(x, w, prefix):
    """nanovllm/models/qwen3.py:113-117 with nanovllm/layers/activation.py:9-11:
    silu(gate) * up in fp32, rounded once (the reference compiles that op), then down."""
    g = linear(x, w[prefix + "gate_proj.weight"]).float()
    u = linear(x, w[prefix + "up_proj.weight"]).float()
    act = (g * torch.sigmoid(g) * u).to(x.dtype)
    return linear(act, w[prefix + "down_proj.weight"])


def decoder_layer(h, residual, positions, w, i, cfg, cos, sin):
    """nanovllm/models/qwen3.py:146-159: pre-norm block, residual carried apart,
    every sub-block's output added inside the next norm."""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    if residual is None:
        residual = h
        x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
    else:
        x, residual = add_rms_norm(h, residual, w[p + "input_layernorm.weight"], eps)
    a = attention_mixer(x, positions, w, p + "self_attn.", cfg, cos, sin)
    x, residual = add_rms_norm(a, residual, w[p + "post_attention_layernorm.weight"], eps)
    m = swiglu_mlp(x, w, p + "mlp.")
    return m, residual


# --------------------------------------------------------------------------- model

def checkpoint_shapes(cfg: dict) -> dict:
    """Names, shapes and kinds ("matrix" / "norm") of a Qwen3 checkpoint's tensors
    (nanovllm/models/qwen3.py:42-70,100-109,143-144,169-171,201; q/k/v and gate/up apart, as
    checkpoints store them, nanovllm/models/qwen3.py:187-193)."""
    H, nq, nkv, d = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    I, V = cfg["intermediate_size"], cfg["vocab_size"]
    out = {"model.embed_tokens.weight": ((V, H), "matrix"), "model.norm.weight": ((H,), "norm")}
    if not cfg["tie_word_embeddings"]:
        out["lm_head.weight"] = ((V, H), "matrix")
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out.update({
            p + "self_attn.q_proj.weight": ((nq * d, H), "matrix"), p + "self_attn.k_proj.weight": ((nkv * d, H), "matrix"),
            p + "self_attn.v_proj.weight": ((nkv * d, H), "matrix"), p + "self_attn.o_proj.weight": ((H, nq * d), "matrix"),
            p + "self_attn.q_norm.weight": ((d,), "norm"), p + "self_attn.k_norm.weight": ((d,), "norm"),
            p + "mlp.gate_proj.weight": ((I, H), "matrix"), p + "mlp.up_proj.weight": ((I, H), "matrix"),
            p + "mlp.down_proj.weight": ((H, I), "matrix"),
            p + "input_layernorm.weight": ((H,), "norm"), p + "post_attention_layernorm.weight": ((H,), "norm")})
    return out


def random_weights_on_device(cfg: dict, seed: int, device) -> dict:
    """The tensors of the engine's random-weights mode WITHOUT a folder, restated from its rule (there is no
    counterpart in the reference): every checkpoint tensor is one float32 draw of its whole shape on the
    device from a generator seeded with the first 8 bytes (little-endian, top bit cleared) of
    sha256("<seed>:<tensor name>"); matrices N(0, 0.02), norm weights 1 + N(0, 0.01)."""
    import hashlib
    out = {}
    for name, (shape, kind) in checkpoint_shapes(cfg).items():
        digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
        gen = torch.Generator(device=device).manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
        t = torch.empty(shape, dtype=torch.float32, device=device)
        out[name] = t.normal_(0.0, 0.02, generator=gen) if kind == "matrix" else 1.0 + t.normal_(0.0, 0.01, generator=gen)
    return out


class PlainQwen3:
    def __init__(self, model_dir: str | None, dtype: torch.dtype = torch.float32, *, cfg: dict | None = None,
                 weights: dict | None = None):
        """From a folder (config.json, model.safetensors), or from a config dictionary and a dictionary of
        tensors under the checkpoint's names (on any device; the model computes where they live)."""
        if cfg is None:
            with open(os.path.join(model_dir, "config.json")) as f:
                cfg = json.load(f)
        cfg = dict(cfg)
        cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
        cfg.setdefault("rope_theta", 1000000)
        self.cfg = cfg
        self.dtype = dtype
        self.w = {}
        if weights is not None:
            self.w = {name: t.to(dtype) for name, t in weights.items()}
        else:
            with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as f:
                for name in f.keys():
                    self.w[name] = f.get_tensor(name).to(dtype)
        if cfg["tie_word_embeddings"]:
            self.w["lm_head.weight"] = self.w["model.embed_tokens.weight"]
        self.device = self.w["model.norm.weight"].device
        self.cos, self.sin = rope_table(cfg["head_dim"], cfg["max_position_embeddings"], cfg["rope_theta"])
        self.cos, self.sin = self.cos.to(self.device), self.sin.to(self.device)

    @torch.no_grad()
    def logits(self, token_ids, rows=None) -> torch.Tensor:
        """fp32 logits [T, V] at every position of one whole sequence, or at the positions ``rows`` only
        (nanovllm/models/qwen3.py:173-183,205-216; nanovllm/layers/embed_head.py:38,61)."""
        cfg, w = self.cfg, self.w
        ids = torch.as_tensor(token_ids, dtype=torch.long, device=self.device)
        positions = torch.arange(len(ids), device=self.device)
        h = w["model.embed_tokens.weight"][ids]
        residual = None
        for i in range(cfg["num_hidden_layers"]):
            h, residual = decoder_layer(h, residual, positions, w, i, cfg, self.cos, self.sin)
        h, _ = add_rms_norm(h, residual, w["model.norm.weight"], cfg["rms_norm_eps"])
        if rows is not None:
            h = h[torch.as_tensor(rows, dtype=torch.long, device=self.device)]
        return linear(h, w["lm_head.weight"]).float()

    def greedy(self, prompt, max_tokens: int):
        """Greedy continuation, recomputing the whole sequence for every token."""
        seq = list(prompt)
        out = []
        for _ in range(max_tokens):
            tok = int(self.logits(seq)[-1].argmax())
            out.append(tok)
            seq.append(tok)
        return out


# --------------------------------------------------------------------------- sampling

_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32(counter, key, rounds: int = 10):
    """Philox4x32-10 (Salmon et al., 'Parallel random numbers: as easy as 1, 2, 3').
    counter: 4 arrays of uint64 holding 32-bit words; key: two ints."""
    c = [np.asarray(x, dtype=np.uint64) & np.uint64(0xFFFFFFFF) for x in counter]
    k0, k1 = np.uint64(key[0] & 0xFFFFFFFF), np.uint64(key[1] & 0xFFFFFFFF)
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(rounds):
        p0 = np.uint64(_PHILOX_M0) * c[0]
        p1 = np.uint64(_PHILOX_M1) * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
        k0 = (k0 + np.uint64(_PHILOX_W0)) & mask
        k1 = (k1 + np.uint64(_PHILOX_W1)) & mask
    return c


def exponential_noise(seed: int, position: int, vocab: int) -> np.ndarray:
    """Exp(1) noise for every vocabulary entry of one sampling decision, keyed by the
    request's seed and the position of the token being chosen."""
    idx = np.arange(vocab, dtype=np.uint64)
    blocks = idx >> np.uint64(2)
    words = philox4x32(
        [blocks, np.full_like(blocks, position & 0xFFFFFFFF), np.zeros_like(blocks), np.zeros_like(blocks)],
        (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF),
    )
    lane = (idx & np.uint64(3)).astype(np.int64)
    r = np.choose(lane, words).astype(np.uint32)
    u = ((r >> np.uint32(9)).astype(np.float64) + 0.5) * (1.0 / 8388608.0)   # 23 bits, in (0,1)
    return np.maximum(-np.log(u), 1e-10)


def sample(logits: torch.Tensor, temperature: float, seed: int, position: int) -> int:
    """nanovllm/layers/sampler.py:12-65: argmax when temperature is 0, else
    argmax(softmax(logits / T) / noise) with noise ~ Exp(1) clamped at 1e-10.
    Computed in float64 here so that ties come only from the logits themselves."""
    lf = logits.double().numpy()
    if temperature == 0:
        return int(lf.argmax())
    noise = exponential_noise(seed, position, lf.shape[0])
    return int((lf / temperature - np.log(noise)).argmax())
