"""Each part of a layer alone against the plain implementation's function for it, and a toy
architecture, defined here, whose layers mix a mixer with fixed-size state of its own with attention,
run one layer twice and let a run read another run's cache; another with a windowed layer; a third with a
feed-forward that routes tokens to experts, a learnt position table, another norm and another arrangement of a
layer's parts: each registered, built from random weights and stepped without a change to the framework's files."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def build_part(registry, spec, hidden, dtype=torch.float32, max_position=256, seed=0):
    from nanohybrid_vlm_b200.parts import BuildEnv
    env = BuildEnv(hidden, dtype, "cuda", max_position)
    obj = registry.get(spec.kind)(spec, env)
    g = torch.Generator().manual_seed(seed)
    host = {}
    for decl in obj.params():
        t = torch.randn(decl.shape, generator=g) * 0.05
        if decl.init == "norm":
            t = 1 + t
        host[decl.name] = t.to(dtype)
    obj.bind({k: v.cuda() for k, v in host.items()})
    return obj, host


class OneRequest:
    """A cache and batch builder for parts tested alone: one group of pages, requests by name."""

    def __init__(self, need, page_size=8, num_pages=64, dtype=torch.float32, vocab=1000):
        from nanohybrid_vlm_b200.cache import CacheLayout, CacheManager, CacheStorage
        from nanohybrid_vlm_b200.engine.batch import BatchBuilder
        from nanohybrid_vlm_b200.parts import LayerRun
        self.layout = CacheLayout.from_needs([need])
        self.cm = CacheManager(self.layout.groups, page_size, num_pages)
        self.storage = CacheStorage(self.layout, [LayerRun(0)], page_size, [num_pages], 0, dtype, "cuda")
        self.storage.pages[0].fill_(float("nan"))
        self.builder = BatchBuilder(self.cm, vocab, "cuda", 512, 8, 64)

    def batch(self, items):
        from nanohybrid_vlm_b200.engine.batch import StepItem
        built = []
        for rid, start, n in items:
            self.cm.allocate(rid, start + n)
            built.append(StepItem(rid, [0] * n, start, []))
        b = self.builder.build(built)
        return b, self.storage.view(0, None, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from nanohybrid_vlm_b200.parts import NORMS, part
    norm, w = build_part(NORMS, part("rmsnorm", width=96, eps=1e-5), 96, dtype)
    g = torch.Generator().manual_seed(1)
    x, r = torch.randn(7, 96, generator=g).to(dtype), torch.randn(7, 96, generator=g).to(dtype)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(norm.forward(x.cuda()).cpu().float(), plain.rms_norm(x, w["weight"], 1e-5).float(), **tol)
    res = r.clone().cuda()
    y, new_r = plain.add_rms_norm(x, r, w["weight"], 1e-5)
    torch.testing.assert_close(norm.forward_add(x.cuda(), res).cpu().float(), y.float(), **tol)
    torch.testing.assert_close(res.cpu().float(), new_r.float(), **tol)
    rows = torch.tensor([6, 2], dtype=torch.int32).cuda()
    torch.testing.assert_close(norm.forward_add_rows(x.cuda(), r.cuda(), rows).cpu().float(), y[[6, 2]].float(), **tol)
    # a norm stored as an offset from one
    off, w = build_part(NORMS, part("rmsnorm", width=96, eps=1e-5, weight_offset=1.0), 96, dtype)
    torch.testing.assert_close(off.forward(x.cuda()).cpu().float(),
                               plain.rms_norm(x, (1 + w["weight"].float()).to(dtype), 1e-5).float(), **tol)


def test_position_part_shares_one_table():
    from nanohybrid_vlm_b200.parts import BuildEnv, part
    env = BuildEnv(64, torch.float32, "cuda", 300)
    spec = part("rope", theta=5000.0, rotary_dim=24, max_position=300)
    a, b = env.position(spec), env.position(part("rope", theta=5000.0, rotary_dim=24, max_position=300))
    assert a is b and env.position(None) is None
    table, rot = a.rotary()
    cos, sin = plain.rope_table(24, 300, 5000.0)
    assert rot == 24 and torch.equal(table.cpu(), torch.cat((cos, sin), -1))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,hidden", [(6, 2, 32, 96), (4, 4, 16, 80)])
def test_attention_part_whole_and_in_portions(dtype, nq, nkv, d, hidden):
    from nanohybrid_vlm_b200.parts import MIXERS, part
    rope = part("rope", theta=10000.0, rotary_dim=d, max_position=256)
    spec = part("gqa_attention", num_heads=nq, num_kv_heads=nkv, head_dim=d, qk_norm_eps=1e-6, position=rope)
    mixer, w = build_part(MIXERS, spec, hidden, dtype)
    T = 45
    x = (torch.randn(T, hidden, generator=torch.Generator().manual_seed(2))).to(dtype)
    names = {"q_proj.weight": w["qkv_proj.weight"][:nq * d], "k_proj.weight": w["qkv_proj.weight"][nq * d:(nq + nkv) * d],
             "v_proj.weight": w["qkv_proj.weight"][(nq + nkv) * d:], "o_proj.weight": w["o_proj.weight"],
             "q_norm.weight": w["q_norm.weight"], "k_norm.weight": w["k_norm.weight"]}
    cfg = dict(num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d, rms_norm_eps=1e-6)
    cos, sin = plain.rope_table(d, 256, 10000.0)
    ref = plain.attention_mixer(x, torch.arange(T), names, "", cfg, cos, sin).float()
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-3)
    env = OneRequest(mixer.cache_need(), dtype=dtype)
    b, view = env.batch([("whole", 0, T)])
    torch.testing.assert_close(mixer.forward(x.cuda(), b, view).cpu().float(), ref, **tol)
    got, at = [], 0
    for n in (13, 2, 29, 1):
        b, view = env.batch([("cut", at, n)])
        got.append(mixer.forward(x[at:at + n].cuda(), b, view).cpu().float())
        at += n
    torch.testing.assert_close(torch.cat(got), ref, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from nanohybrid_vlm_b200.parts import FEED_FORWARDS, part
    ffn, w = build_part(FEED_FORWARDS, part("swiglu", intermediate_size=160), 96, dtype)
    x = torch.randn(9, 96, generator=torch.Generator().manual_seed(3)).to(dtype)
    names = {"gate_proj.weight": w["gate_up_proj.weight"][:160], "up_proj.weight": w["gate_up_proj.weight"][160:],
             "down_proj.weight": w["down_proj.weight"]}
    tol = dict(rtol=1e-4, atol=1e-6) if dtype == torch.float32 else dict(rtol=3e-2, atol=1e-3)
    torch.testing.assert_close(ffn.forward(x.cuda(), None).cpu().float(), plain.swiglu_mlp(x, names, "").float(), **tol)


def test_embedding_and_head_parts():
    from nanohybrid_vlm_b200.parts.embedding import LMHead, TokenEmbedding
    from nanohybrid_vlm_b200.parts import BuildEnv, part
    env = BuildEnv(48, torch.float32, "cuda", 64)
    emb = TokenEmbedding(part("token_embedding", vocab_size=101), env)
    table = torch.randn(101, 48, generator=torch.Generator().manual_seed(4))
    emb.bind({"weight": table.cuda()})
    ids = torch.tensor([5, 100, 0, 5], dtype=torch.int32)
    assert torch.equal(emb.forward(ids.cuda()).cpu(), table[ids.long()])
    head = LMHead(part("lm_head", vocab_size=101, tied=True), env)
    assert head.params() == []
    head.tie(emb)
    x = torch.randn(3, 48, generator=torch.Generator().manual_seed(5))
    torch.testing.assert_close(head.forward(x.cuda()).cpu(), x @ table.t(), rtol=1e-5, atol=1e-5)


# ------------------------------------------------------------------------------------------------ toy architecture

TOY = dict(architectures=["ToyStateLM"], model_type="toy_state", hidden_size=48, vocab_size=97, state_decay=0.75,
           num_attention_heads=3, num_key_value_heads=1, head_dim=16, intermediate_size=64, rms_norm_eps=1e-5,
           rope_theta=1000.0, max_position_embeddings=128, torch_dtype="float32")


def register_toy():
    """A mixer with state of its own (an exponential moving average of its inputs, kept per request in a
    slot) and an architecture that uses it, both defined here."""
    from nanohybrid_vlm_b200.config import ModelConfig, register_architecture
    from nanohybrid_vlm_b200.parts import (MIXERS, FixedStateNeed, LayerRun, LayerSpec, Mixer, ModelSpec, ParamDecl,
                                           PartUse, part)

    class MovingAverageMixer(Mixer):
        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.decay = float(spec["decay"])

        def params(self):
            H = self.env.hidden_size
            return [ParamDecl("out.weight", (H, H))]

        def cache_need(self):
            return FixedStateNeed((self.env.hidden_size,), "float32")

        def forward(self, x, batch, cache):
            y = torch.empty_like(x)
            slots = batch.state_slots.tolist()
            for s in range(batch.n_seqs):
                a, b = batch.host_cu_q[s], batch.host_cu_q[s + 1]
                if slots[s] < 0:
                    y[a:b] = 0
                    continue
                state = cache.state[slots[s]]
                if batch.host_kv_len[s] - (b - a) == 0:      # the request starts: its slot may hold another's state
                    state.zero_()
                for t in range(a, b):
                    state.mul_(self.decay).add_(x[t].float(), alpha=1 - self.decay)
                    y[t] = (self.w_out_weight.float() @ state).to(x.dtype)
            return y

    MIXERS.register("moving_average", MovingAverageMixer, replace=True)

    def parse(raw):
        cfg = ModelConfig(architecture="ToyStateLM", model_type=raw["model_type"], vocab_size=raw["vocab_size"],
                          hidden_size=raw["hidden_size"], max_position_embeddings=raw["max_position_embeddings"],
                          dtype=torch.float32, eos_token_id=None)
        object.__setattr__(cfg, "raw", raw)
        return cfg

    def build(cfg):
        raw = cfg.raw
        H = raw["hidden_size"]
        norm = part("rmsnorm", width=H, eps=raw["rms_norm_eps"])
        ffn = part("swiglu", intermediate_size=raw["intermediate_size"])
        rope = part("rope", theta=raw["rope_theta"], rotary_dim=raw["head_dim"], max_position=raw["max_position_embeddings"])
        attn = part("gqa_attention", num_heads=raw["num_attention_heads"], num_kv_heads=raw["num_key_value_heads"],
                    head_dim=raw["head_dim"], qk_norm_eps=raw["rms_norm_eps"], position=rope)
        avg = part("moving_average", decay=raw["state_decay"])

        def layer(i, mixer):
            return LayerSpec(part("prenorm_residual"), PartUse(mixer, f"layers.{i}.mixer."), PartUse(norm, f"layers.{i}.norm1."),
                             PartUse(ffn, f"layers.{i}.ffn."), PartUse(norm, f"layers.{i}.norm2."))

        return ModelSpec(architecture="ToyStateLM", hidden_size=H, vocab_size=raw["vocab_size"],
                         max_position=raw["max_position_embeddings"],
                         embedding=PartUse(part("token_embedding", vocab_size=raw["vocab_size"]), "embed."),
                         layers=(layer(0, avg), layer(1, attn)),
                         # layer 0 runs twice (its second run has a state of its own); the last run reads the keys
                         # and values that the first attention run stored
                         order=(LayerRun(0), LayerRun(1), LayerRun(0), LayerRun(1, cache_from=1)),
                         final_norm=PartUse(norm, "final_norm."),
                         head=PartUse(part("lm_head", vocab_size=raw["vocab_size"], tied=False), "head."))

    register_architecture("ToyStateLM", model_types=("toy_state",), parse_config=parse, build_spec=build, replace=True)


def toy_plain_logits(w, tokens):
    """The toy model over one whole sequence, written out plainly."""
    raw, T = TOY, len(tokens)
    nq, nkv, d, eps = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], raw["rms_norm_eps"]
    cos, sin = plain.rope_table(d, raw["max_position_embeddings"], raw["rope_theta"])
    pos = torch.arange(T)
    h = w["embed.weight"][torch.tensor(tokens)]

    def average(x, i):
        s, out = torch.zeros(raw["hidden_size"]), []
        for t in range(T):
            s = raw["state_decay"] * s + (1 - raw["state_decay"]) * x[t]
            out.append(w[f"layers.{i}.mixer.out.weight"] @ s)
        return torch.stack(out)

    def qkv(x, i):
        p = f"layers.{i}.mixer."
        q = plain.linear(x, w[p + "q_proj.weight"]).view(T, nq, d)
        k = plain.linear(x, w[p + "k_proj.weight"]).view(T, nkv, d)
        v = plain.linear(x, w[p + "v_proj.weight"]).view(T, nkv, d)
        q = plain.apply_rope(plain.rms_norm(q, w[p + "q_norm.weight"], eps), cos[pos], sin[pos])
        k = plain.apply_rope(plain.rms_norm(k, w[p + "k_norm.weight"], eps), cos[pos], sin[pos])
        return q, k, v

    residual, kept = None, None
    for run, (i, kind) in enumerate([(0, "avg"), (1, "attn"), (0, "avg"), (1, "shared")]):
        if residual is None:
            residual, x = h, plain.rms_norm(h, w[f"layers.{i}.norm1.weight"], eps)
        else:
            x, residual = plain.add_rms_norm(h, residual, w[f"layers.{i}.norm1.weight"], eps)
        if kind == "avg":
            a = average(x, i)
        else:
            q, k, v = qkv(x, i)
            if kind == "attn":
                kept = (k, v)
            o = plain.causal_attention(q, kept[0], kept[1], d ** -0.5)
            a = plain.linear(o.reshape(T, nq * d), w[f"layers.{i}.mixer.o_proj.weight"])
        x, residual = plain.add_rms_norm(a, residual, w[f"layers.{i}.norm2.weight"], eps)
        h = plain.swiglu_mlp(x, w, f"layers.{i}.ffn.")
    x, _ = plain.add_rms_norm(h, residual, w["final_norm.weight"], eps)
    return plain.linear(x, w["head.weight"])


def test_toy_architecture_with_a_state_mixer_registers_builds_and_steps(tmp_path):
    from safetensors.torch import load_file
    from nanohybrid_vlm_b200.config import ARCHITECTURES, Config
    from nanohybrid_vlm_b200.engine import ModelRunner, StepItem
    from nanohybrid_vlm_b200.parts import MIXERS
    from nanohybrid_vlm_b200.weights import write_random_model
    register_toy()
    try:
        d = write_random_model(str(tmp_path / "toy"), TOY, seed=9)
        w = load_file(f"{d}/model.safetensors")
        assert "layers.0.mixer.out.weight" in w and "layers.1.mixer.k_proj.weight" in w
        runner = ModelRunner(Config(d, kvcache_block_size=4, num_kvcache_blocks=40, max_num_seqs=3,
                                    max_num_batched_tokens=64, max_model_len=128, enforce_eager=True))
        assert runner.cache.slots is not None and runner.cache.slots.num_slots == 3       # state slots appeared
        assert [g.window for g in runner.layout.groups] == [None]
        assert runner.layout.run_group == [None, 0, None, None]
        rng = np.random.default_rng(0)
        reqs = {r: rng.integers(0, TOY["vocab_size"], n).tolist() for r, n in (("a", 30), ("b", 17), ("c", 41), ("d", 9))}
        ref = {r: toy_plain_logits(w, t) for r, t in reqs.items()}
        # a, b, c in portions of different sizes side by side; d takes over a finished request's slot and pages
        plan = {"a": [7, 2, 21], "b": [1, 1, 15], "c": [20, 20, 1]}
        at = {r: 0 for r in reqs}
        got = {r: [] for r in reqs}
        for step in range(3):
            items = []
            for r, cuts in plan.items():
                n = cuts[step]
                runner.cache.allocate(r, at[r] + n)
                items.append(StepItem(r, reqs[r][at[r]:at[r] + n], at[r], list(range(n))))
                at[r] += n
            logits = runner.step(items).cpu()
            k = 0
            for it in items:
                got[it.req_id].append(logits[k:k + len(it.tokens)])
                k += len(it.tokens)
        runner.cache.free("b")
        runner.cache.allocate("d", 9)
        assert runner.cache.state_slot("d") == 1                                           # b's slot, reused
        got["d"].append(runner.step([StepItem("d", reqs["d"], 0, list(range(9)))]).cpu())
        for r in reqs:
            torch.testing.assert_close(torch.cat(got[r]), ref[r], rtol=1e-4, atol=2e-5)
        runner.cache.check()
    finally:
        ARCHITECTURES.unregister("ToyStateLM")
        MIXERS.unregister("moving_average")


# ------------------------------------------------------------------------------------------------ a windowed layer

WINDOW = dict(architectures=["ToyWindowLM"], model_type="toy_window", hidden_size=64, vocab_size=120, window=11,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=96, rms_norm_eps=1e-6,
              rope_theta=10000.0, max_position_embeddings=256, torch_dtype="float32")


def register_window_toy():
    from nanohybrid_vlm_b200.config import ModelConfig, register_architecture
    from nanohybrid_vlm_b200.parts import LayerRun, LayerSpec, ModelSpec, PartUse, part

    def parse(raw):
        cfg = ModelConfig(architecture="ToyWindowLM", model_type=raw["model_type"], vocab_size=raw["vocab_size"],
                          hidden_size=raw["hidden_size"], max_position_embeddings=raw["max_position_embeddings"],
                          dtype=torch.float32, eos_token_id=None)
        object.__setattr__(cfg, "raw", raw)
        return cfg

    def build(cfg):
        raw = cfg.raw
        H = raw["hidden_size"]
        norm = part("rmsnorm", width=H, eps=raw["rms_norm_eps"])
        ffn = part("swiglu", intermediate_size=raw["intermediate_size"])
        rope = part("rope", theta=raw["rope_theta"], rotary_dim=raw["head_dim"], max_position=raw["max_position_embeddings"])

        def attn(window):
            return part("gqa_attention", num_heads=raw["num_attention_heads"], num_kv_heads=raw["num_key_value_heads"],
                        head_dim=raw["head_dim"], qk_norm_eps=raw["rms_norm_eps"], position=rope, window=window)

        def layer(i, mixer):
            return LayerSpec(part("prenorm_residual"), PartUse(mixer, f"layers.{i}.attn."), PartUse(norm, f"layers.{i}.norm1."),
                             PartUse(ffn, f"layers.{i}.ffn."), PartUse(norm, f"layers.{i}.norm2."))

        # all keys, the last `window` keys, all keys: two cache groups with pages of their own
        return ModelSpec(architecture="ToyWindowLM", hidden_size=H, vocab_size=raw["vocab_size"],
                         max_position=raw["max_position_embeddings"],
                         embedding=PartUse(part("token_embedding", vocab_size=raw["vocab_size"]), "embed."),
                         layers=(layer(0, attn(None)), layer(1, attn(raw["window"])), layer(2, attn(None))),
                         order=(LayerRun(0), LayerRun(1), LayerRun(2)),
                         final_norm=PartUse(norm, "final_norm."),
                         head=PartUse(part("lm_head", vocab_size=raw["vocab_size"], tied=True), "head."))

    register_architecture("ToyWindowLM", model_types=("toy_window",), parse_config=parse, build_spec=build, replace=True)


def window_plain_logits(w, tokens):
    raw, T = WINDOW, len(tokens)
    nq, nkv, d, eps = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], raw["rms_norm_eps"]
    cos, sin = plain.rope_table(d, raw["max_position_embeddings"], raw["rope_theta"])
    pos = torch.arange(T)
    h = w["embed.weight"][torch.tensor(tokens)]
    residual = None
    for i, window in enumerate((None, raw["window"], None)):
        p = f"layers.{i}."
        if residual is None:
            residual, x = h, plain.rms_norm(h, w[p + "norm1.weight"], eps)
        else:
            x, residual = plain.add_rms_norm(h, residual, w[p + "norm1.weight"], eps)
        q = plain.linear(x, w[p + "attn.q_proj.weight"]).view(T, nq, d)
        k = plain.linear(x, w[p + "attn.k_proj.weight"]).view(T, nkv, d)
        v = plain.linear(x, w[p + "attn.v_proj.weight"]).view(T, nkv, d)
        q = plain.apply_rope(plain.rms_norm(q, w[p + "attn.q_norm.weight"], eps), cos[pos], sin[pos])
        k = plain.apply_rope(plain.rms_norm(k, w[p + "attn.k_norm.weight"], eps), cos[pos], sin[pos])
        o = reference_window_attention(q, k, v, d ** -0.5, window)
        a = plain.linear(o.reshape(T, nq * d), w[p + "attn.o_proj.weight"])
        x, residual = plain.add_rms_norm(a, residual, w[p + "norm2.weight"], eps)
        h = plain.swiglu_mlp(x, w, p + "ffn.")
    x, _ = plain.add_rms_norm(h, residual, w["final_norm.weight"], eps)
    return plain.linear(x, w["embed.weight"])


def reference_window_attention(q, k, v, scale, window):
    T, nq, d = q.shape
    G = nq // k.shape[1]
    out = torch.empty(T, nq, d)
    for t in range(T):
        lo = max(0, t - window + 1) if window else 0
        for h in range(nq):
            s = (k[lo:t + 1, h // G].float() @ q[t, h].float()) * scale
            out[t, h] = torch.softmax(s, 0) @ v[lo:t + 1, h // G].float()
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_a_window_have_pages_of_their_own_and_give_them_back(tmp_path, dtype):
    """Three attention layers, the middle one sees only the last 11 keys: its group releases pages while the
    request runs, the freed pages go to another request at once, and the logits stay those of the plain model."""
    from safetensors.torch import load_file
    from nanohybrid_vlm_b200.config import ARCHITECTURES, Config
    from nanohybrid_vlm_b200.engine import ModelRunner, StepItem
    from nanohybrid_vlm_b200.weights import write_random_model
    register_window_toy()
    try:
        d = write_random_model(str(tmp_path / "win"), WINDOW, seed=4)
        w = load_file(f"{d}/model.safetensors")
        runner = ModelRunner(Config(d, dtype=dtype, kvcache_block_size=4, num_kvcache_blocks=30, max_num_seqs=2,
                                    max_num_batched_tokens=64, max_model_len=96, enforce_eager=True))
        cache = runner.cache
        assert [g.window for g in runner.layout.groups] == [None, 11] and runner.layout.run_group == [0, 1, 0]
        rng = np.random.default_rng(1)
        toks = {"a": rng.integers(0, 120, 70).tolist(), "b": rng.integers(0, 120, 37).tolist()}
        ref = {r: window_plain_logits(w, t) for r, t in toks.items()}
        got = {"a": [], "b": []}
        at = {"a": 0, "b": 0}
        cuts = {"a": [30, 1, 1, 17, 2, 19], "b": [0, 0, 9, 1, 26, 1]}
        for step in range(6):
            items = []
            for r in ("a", "b"):
                n = cuts[r][step]
                if n == 0:
                    continue
                cache.allocate(r, at[r] + n)
                items.append(StepItem(r, toks[r][at[r]:at[r] + n], at[r], list(range(n))))
                at[r] += n
            logits = runner.step(items).cpu()
            k = 0
            for it in items:
                got[it.req_id].append(logits[k:k + len(it.tokens)])
                k += len(it.tokens)
                cache.release_behind_window(it.req_id, at[it.req_id])
            cache.check()
        # request a: 70 tokens computed, the windowed group keeps only the pages of keys 60..69
        table = cache.block_table("a", 1)
        assert table[:15] == [-1] * 15 and all(p >= 0 for p in table[15:])
        assert all(p >= 0 for p in cache.block_table("a", 0))
        assert cache.pools[1].num_used < cache.pools[0].num_used
        for r in toks:
            g = torch.cat(got[r])
            if dtype == "float32":
                torch.testing.assert_close(g, ref[r], rtol=1e-4, atol=2e-5)
            else:
                assert (g - ref[r]).abs().max() <= 0.06 * ref[r].std()
    finally:
        ARCHITECTURES.unregister("ToyWindowLM")


# ------------------------------------------------------------------------------------------------ routing and another position encoding

ROUTED = dict(architectures=["ToyRoutedLM"], model_type="toy_routed", hidden_size=40, vocab_size=83, num_experts=3,
              expert_size=24, num_attention_heads=2, num_key_value_heads=2, head_dim=16, intermediate_size=56,
              rms_norm_eps=1e-5, max_position_embeddings=96, torch_dtype="float32")


def register_routed_toy():
    """A feed-forward that routes every token to one of its experts, and a position encoding with a learnt table
    that is added to the embedded tokens (the attention layers then rotate nothing): both defined here."""
    from nanohybrid_vlm_b200.config import ModelConfig, register_architecture
    from nanohybrid_vlm_b200.parts import (BLOCKS, FEED_FORWARDS, NORMS, POSITIONS, Block, FeedForward, LayerRun,
                                           LayerSpec, ModelSpec, Norm, ParamDecl, PartUse, PositionEncoding, part)

    class TopOneExperts(FeedForward):
        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.E, self.I = int(spec["num_experts"]), int(spec["expert_size"])

        def params(self):
            H = self.env.hidden_size
            return [ParamDecl("router.weight", (self.E, H)), ParamDecl("up.weight", (self.E * self.I, H)),
                    ParamDecl("down.weight", (self.E * H, self.I))]

        def forward(self, x, batch):
            H = self.env.hidden_size
            prob = torch.softmax(x.float() @ self.w_router_weight.float().t(), -1)     # router logits in fp32
            best = prob.argmax(-1)
            up = self.w_up_weight.float().view(self.E, self.I, H)
            down = self.w_down_weight.float().view(self.E, H, self.I)
            hidden = torch.relu(torch.einsum("tih,th->ti", up[best], x.float()))
            y = torch.einsum("thi,ti->th", down[best], hidden) * prob.gather(1, best[:, None])
            return y.to(x.dtype)

    class LearntPositions(PositionEncoding):
        def params(self):
            return [ParamDecl("weight", (int(self.spec["max_position"]), self.env.hidden_size))]

        def add_to_embeddings(self, h, batch):
            return (h.float() + self.w_weight.float()[batch.positions.long()]).to(h.dtype)

    class MeanCentredNorm(Norm):
        """A LayerNorm without bias: mean and variance over the row, times a weight (another norm than the
        engine's own), with the residual add that the block arrangement asks of every norm."""

        def params(self):
            return [ParamDecl("weight", (int(self.spec["width"]),), init="norm")]

        def _norm(self, s):
            s = s - s.mean(-1, keepdim=True)
            return s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + float(self.spec["eps"])) * self.w_weight.float()

        def forward(self, x):
            return self._norm(x.float()).to(x.dtype)

        def forward_add(self, x, residual):
            s = x.float() + residual.float()
            residual.copy_(s.to(residual.dtype))
            return self._norm(s).to(x.dtype)

        def forward_add_rows(self, x, residual, rows):
            r = rows.long()
            return self._norm(x[r].float() + residual[r].float()).to(x.dtype)

    class ParallelBlock(Block):
        """Another arrangement of the same four parts: mixer and feed-forward both read one norm of the stream
        and their outputs are added together (the second norm of the layer goes unused, with its tensor)."""

        def forward(self, hidden, residual, batch, cache):
            if residual is None:
                residual = hidden
                x = self.mixer_norm.forward(hidden)
            else:
                x = self.mixer_norm.forward_add(hidden, residual)
            return self.mixer.forward(x, batch, cache) + self.ffn.forward(x, batch), residual

    FEED_FORWARDS.register("top_one_experts", TopOneExperts, replace=True)
    POSITIONS.register("learnt", LearntPositions, replace=True)
    NORMS.register("mean_centred", MeanCentredNorm, replace=True)
    BLOCKS.register("parallel", ParallelBlock, replace=True)

    def parse(raw):
        cfg = ModelConfig(architecture="ToyRoutedLM", model_type=raw["model_type"], vocab_size=raw["vocab_size"],
                          hidden_size=raw["hidden_size"], max_position_embeddings=raw["max_position_embeddings"],
                          dtype=torch.float32, eos_token_id=None)
        object.__setattr__(cfg, "raw", raw)
        return cfg

    def build(cfg):
        raw = cfg.raw
        H = raw["hidden_size"]
        norm = part("rmsnorm", width=H, eps=raw["rms_norm_eps"])
        attn = part("gqa_attention", num_heads=raw["num_attention_heads"], num_kv_heads=raw["num_key_value_heads"],
                    head_dim=raw["head_dim"])                           # no q/k norm, nothing rotated
        experts = part("top_one_experts", num_experts=raw["num_experts"], expert_size=raw["expert_size"])
        dense = part("swiglu", intermediate_size=raw["intermediate_size"])

        centred = part("mean_centred", width=H, eps=raw["rms_norm_eps"])

        def layer(i, ffn, block="prenorm_residual", layer_norm=norm):
            return LayerSpec(part(block), PartUse(attn, f"layers.{i}.attn."), PartUse(layer_norm, f"layers.{i}.norm1."),
                             PartUse(ffn, f"layers.{i}.ffn."), PartUse(layer_norm, f"layers.{i}.norm2."))

        return ModelSpec(architecture="ToyRoutedLM", hidden_size=H, vocab_size=raw["vocab_size"],
                         max_position=raw["max_position_embeddings"],
                         embedding=PartUse(part("token_embedding", vocab_size=raw["vocab_size"]), "embed."),
                         positions=(PartUse(part("learnt", max_position=raw["max_position_embeddings"]), "positions."),),
                         # a routed and a dense feed-forward; then a layer in another arrangement with another norm
                         layers=(layer(0, experts), layer(1, dense), layer(2, dense, "parallel", centred)),
                         order=(LayerRun(0), LayerRun(1), LayerRun(2)),
                         final_norm=PartUse(norm, "final_norm."),
                         head=PartUse(part("lm_head", vocab_size=raw["vocab_size"], tied=False), "head."))

    register_architecture("ToyRoutedLM", model_types=("toy_routed",), parse_config=parse, build_spec=build, replace=True)


def routed_plain_logits(w, tokens):
    raw, T = ROUTED, len(tokens)
    nq, nkv, d, eps, H = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], raw["rms_norm_eps"], raw["hidden_size"]
    E, I = raw["num_experts"], raw["expert_size"]
    h = w["embed.weight"][torch.tensor(tokens)] + w["positions.weight"][:T]
    residual = None
    for i in range(2):
        p = f"layers.{i}."
        if residual is None:
            residual, x = h, plain.rms_norm(h, w[p + "norm1.weight"], eps)
        else:
            x, residual = plain.add_rms_norm(h, residual, w[p + "norm1.weight"], eps)
        q = plain.linear(x, w[p + "attn.q_proj.weight"]).view(T, nq, d)
        k = plain.linear(x, w[p + "attn.k_proj.weight"]).view(T, nkv, d)
        v = plain.linear(x, w[p + "attn.v_proj.weight"]).view(T, nkv, d)
        o = plain.causal_attention(q, k, v, d ** -0.5)
        a = plain.linear(o.reshape(T, nq * d), w[p + "attn.o_proj.weight"])
        x, residual = plain.add_rms_norm(a, residual, w[p + "norm2.weight"], eps)
        if i == 0:
            rows = []
            for t in range(T):
                prob = torch.softmax(w[p + "ffn.router.weight"] @ x[t], 0)
                e = int(prob.argmax())
                up = w[p + "ffn.up.weight"][e * I:(e + 1) * I]
                down = w[p + "ffn.down.weight"][e * H:(e + 1) * H]
                rows.append(prob[e] * (down @ torch.relu(up @ x[t])))
            h = torch.stack(rows)
        else:
            h = plain.swiglu_mlp(x, w, p + "ffn.")
    # layer 2: the parallel arrangement behind a mean-centred norm
    residual = h + residual
    c = residual - residual.mean(-1, keepdim=True)
    x = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * w["layers.2.norm1.weight"]
    q = plain.linear(x, w["layers.2.attn.q_proj.weight"]).view(T, nq, d)
    k = plain.linear(x, w["layers.2.attn.k_proj.weight"]).view(T, nkv, d)
    v = plain.linear(x, w["layers.2.attn.v_proj.weight"]).view(T, nkv, d)
    o = plain.causal_attention(q, k, v, d ** -0.5)
    h = plain.linear(o.reshape(T, nq * d), w["layers.2.attn.o_proj.weight"]) + plain.swiglu_mlp(x, w, "layers.2.ffn.")
    x, _ = plain.add_rms_norm(h, residual, w["final_norm.weight"], eps)
    return plain.linear(x, w["head.weight"])


def test_routing_learnt_positions_another_norm_and_another_block_register_build_and_step(tmp_path):
    from safetensors.torch import load_file
    from nanohybrid_vlm_b200.config import ARCHITECTURES, Config
    from nanohybrid_vlm_b200.engine import ModelRunner, StepItem
    from nanohybrid_vlm_b200.parts import BLOCKS, FEED_FORWARDS, NORMS, POSITIONS
    from nanohybrid_vlm_b200.weights import write_random_model
    register_routed_toy()
    try:
        d = write_random_model(str(tmp_path / "routed"), ROUTED, seed=11)
        w = load_file(f"{d}/model.safetensors")
        assert w["positions.weight"].shape == (96, 40) and w["layers.0.ffn.router.weight"].shape == (3, 40)
        assert "layers.1.ffn.gate_proj.weight" in w and "layers.0.attn.q_norm.weight" not in w
        runner = ModelRunner(Config(d, kvcache_block_size=8, num_kvcache_blocks=24, max_num_seqs=3,
                                    max_num_batched_tokens=64, max_model_len=96, enforce_eager=True))
        rng = np.random.default_rng(3)
        reqs = {"a": rng.integers(0, 83, 50).tolist(), "b": rng.integers(0, 83, 23).tolist()}
        ref = {r: routed_plain_logits(w, t) for r, t in reqs.items()}
        experts_used = {int(torch.softmax(w["layers.0.ffn.router.weight"] @ x, 0).argmax())
                        for x in torch.randn(64, 40, generator=torch.Generator().manual_seed(0))}
        assert len(experts_used) > 1, "the router of the random model should not send everything to one expert"
        cuts = {"a": [31, 1, 18], "b": [2, 20, 1]}
        at, got = {"a": 0, "b": 0}, {"a": [], "b": []}
        for step in range(3):
            items = []
            for r in reqs:
                n = cuts[r][step]
                runner.cache.allocate(r, at[r] + n)
                items.append(StepItem(r, reqs[r][at[r]:at[r] + n], at[r], list(range(n))))
                at[r] += n
            logits = runner.step(items).cpu()
            k = 0
            for it in items:
                got[it.req_id].append(logits[k:k + len(it.tokens)])
                k += len(it.tokens)
        for r in reqs:
            torch.testing.assert_close(torch.cat(got[r]), ref[r], rtol=1e-4, atol=2e-5)
        runner.cache.check()
    finally:
        ARCHITECTURES.unregister("ToyRoutedLM")
        FEED_FORWARDS.unregister("top_one_experts")
        POSITIONS.unregister("learnt")
        NORMS.unregister("mean_centred")
        BLOCKS.unregister("parallel")


# ------------------------------------------------------------------------------------------------ another block, embedding, head, positions and checkpoint layout

SANDWICH = dict(architectures=["ToySandwichLM"], model_type="toy_sandwich", hidden_size=40, vocab_size=71,
                num_attention_heads=4, num_key_value_heads=2, head_dim=16, expert_size=24, num_experts=3,
                rms_norm_eps=1e-5, rope_theta=500.0, max_position_embeddings=96, logit_cap=0.3, torch_dtype="float32")


def register_sandwich_toy():
    """Parts that the engine's own files know nothing of, all defined here: a block kind with four norms (one
    before and one behind each sub-block) and no residual carried apart; an embedding with a scale; a head with
    a bias and a soft cap; a position table with two axes whose positions the caller gives; a feed-forward whose
    checkpoint stores its matrices transposed, split by columns, and one tensor per expert."""
    from nanohybrid_vlm_b200.config import ModelConfig, register_architecture
    from nanohybrid_vlm_b200.parts import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block,
                                           Embedding, FeedForward, Head, LayerRun, LayerSpec, ModelSpec, ParamDecl,
                                           PartUse, PositionEncoding, Source, part)
    from nanohybrid_vlm_b200.weights.random_init import register_init

    class SandwichBlock(Block):
        SLOTS = {"mixer": MIXERS, "mixer_norm": NORMS, "mixer_post_norm": NORMS,
                 "ffn": FEED_FORWARDS, "ffn_norm": NORMS, "ffn_post_norm": NORMS}
        OPTIONAL = ("ffn", "ffn_norm", "ffn_post_norm")              # a layer may be a mixer alone

        def forward(self, hidden, residual, batch, cache):
            stream = hidden if residual is None else residual + hidden
            a = self.mixer_post_norm.forward(self.mixer.forward(self.mixer_norm.forward(stream), batch, cache))
            if "ffn" not in self.parts:
                return a, stream
            stream = stream + a
            return self.ffn_post_norm.forward(self.ffn.forward(self.ffn_norm.forward(stream), batch)), stream

    class ScaledEmbedding(Embedding):
        def params(self):
            return [ParamDecl("weight", (int(self.spec["vocab_size"]), self.env.hidden_size))]

        def forward(self, token_ids, batch):
            return self.w_weight[token_ids.long()] * float(self.spec["scale"])

    class CappedHead(Head):
        def params(self):
            V = int(self.spec["vocab_size"])
            return [ParamDecl("weight", (V, self.env.hidden_size)), ParamDecl("bias", (V,), init="tenths")]

        def forward(self, rows_hidden):
            cap = float(self.spec["cap"])
            return cap * torch.tanh((rows_hidden.float() @ self.w_weight.float().t() + self.w_bias.float()) / cap)

    class TwoAxisPositions(PositionEncoding):
        def params(self):
            n = int(self.spec["max_position"])
            return [ParamDecl("rows.weight", (n, self.env.hidden_size)), ParamDecl("cols.weight", (n, self.env.hidden_size))]

        def add_to_embeddings(self, h, batch):
            assert batch.position_axes.shape == (2, h.shape[0])
            return h + self.w_rows_weight[batch.position_axes[0].long()] + self.w_cols_weight[batch.position_axes[1].long()]

    class StackedExperts(FeedForward):
        """Every token goes to the expert with the largest router score.  The up matrices are one parameter
        [E, I, H] filled from one checkpoint tensor per expert, each stored transposed ([H, I]); the down matrices
        one parameter [H, E * I] filled column block by column block."""
        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.E, self.I = int(spec["num_experts"]), int(spec["expert_size"])

        def params(self):
            H, E, I = self.env.hidden_size, self.E, self.I
            return [ParamDecl("router.weight", (E, H)),
                    ParamDecl("up", (E, I, H), sources=tuple(Source(f"experts.{e}.up_t", e, 1, transpose=True, squeeze=True) for e in range(E))),
                    ParamDecl("down", (H, E * I), sources=tuple(Source(f"experts.{e}.down", e * I, I, 1) for e in range(E)))]

        def forward(self, x, batch):
            xf = x.float()
            e = (xf @ self.w_router_weight.float().t()).argmax(-1)                    # [T]
            up = torch.einsum("tih,th->ti", self.w_up.float()[e], xf)
            down = self.w_down.float().view(-1, self.E, self.I).permute(1, 0, 2)[e]    # [T, H, I]
            return torch.einsum("thi,ti->th", down, torch.relu(up)).to(x.dtype)

    register_init("tenths", lambda shape, gen, device: torch.empty(shape, dtype=torch.float32, device=device).uniform_(-0.1, 0.1, generator=gen))
    BLOCKS.register("sandwich", SandwichBlock, replace=True)
    EMBEDDINGS.register("scaled_embedding", ScaledEmbedding, replace=True)
    HEADS.register("capped_head", CappedHead, replace=True)
    POSITIONS.register("two_axis", TwoAxisPositions, replace=True)
    FEED_FORWARDS.register("stacked_experts", StackedExperts, replace=True)

    def parse(raw):
        cfg = ModelConfig(architecture="ToySandwichLM", model_type=raw["model_type"], vocab_size=raw["vocab_size"],
                          hidden_size=raw["hidden_size"], max_position_embeddings=raw["max_position_embeddings"],
                          dtype=torch.float32, eos_token_id=None)
        object.__setattr__(cfg, "raw", raw)
        return cfg

    def build(cfg):
        raw = cfg.raw
        H, V = raw["hidden_size"], raw["vocab_size"]
        norm = part("rmsnorm", width=H, eps=raw["rms_norm_eps"])
        rope = part("rope", theta=raw["rope_theta"], rotary_dim=raw["head_dim"], max_position=raw["max_position_embeddings"])
        attn = part("gqa_attention", num_heads=raw["num_attention_heads"], num_kv_heads=raw["num_key_value_heads"],
                    head_dim=raw["head_dim"], qk_norm_eps=raw["rms_norm_eps"], position=rope)
        ffn = part("stacked_experts", num_experts=raw["num_experts"], expert_size=raw["expert_size"])

        def use(p, i, name):
            return PartUse(p, f"layers.{i}.{name}.")

        full = LayerSpec(part("sandwich"), mixer=use(attn, 0, "attn"), mixer_norm=use(norm, 0, "pre_attn"),
                         mixer_post_norm=use(norm, 0, "post_attn"), ffn=use(ffn, 0, "ffn"),
                         ffn_norm=use(norm, 0, "pre_ffn"), ffn_post_norm=use(norm, 0, "post_ffn"))
        mixer_only = LayerSpec(part("sandwich"), mixer=use(attn, 1, "attn"), mixer_norm=use(norm, 1, "pre_attn"),
                               mixer_post_norm=use(norm, 1, "post_attn"))
        return ModelSpec(architecture="ToySandwichLM", hidden_size=H, vocab_size=V, max_position=raw["max_position_embeddings"],
                         embedding=PartUse(part("scaled_embedding", vocab_size=V, scale=H ** 0.5), "embed."),
                         positions=(PartUse(part("two_axis", max_position=raw["max_position_embeddings"]), "positions."),),
                         position_axes=2, layers=(full, mixer_only), order=(LayerRun(0), LayerRun(1)),
                         final_norm=PartUse(norm, "final_norm."),
                         head=PartUse(part("capped_head", vocab_size=V, cap=raw["logit_cap"]), "head."))

    register_architecture("ToySandwichLM", model_types=("toy_sandwich",), parse_config=parse, build_spec=build, replace=True)


def sandwich_plain_logits(w, tokens, rows, cols):
    raw, T = SANDWICH, len(tokens)
    nq, nkv, d, eps, H = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], raw["rms_norm_eps"], raw["hidden_size"]
    cos, sin = plain.rope_table(d, raw["max_position_embeddings"], raw["rope_theta"])
    rows, cols = torch.tensor(rows), torch.tensor(cols)
    stream = w["embed.weight"][torch.tensor(tokens)] * H ** 0.5 + w["positions.rows.weight"][rows] + w["positions.cols.weight"][cols]

    def attention(x, p):
        q = plain.linear(x, w[p + "q_proj.weight"]).view(T, nq, d)
        k = plain.linear(x, w[p + "k_proj.weight"]).view(T, nkv, d)
        v = plain.linear(x, w[p + "v_proj.weight"]).view(T, nkv, d)
        q = plain.apply_rope(plain.rms_norm(q, w[p + "q_norm.weight"], eps), cos[rows], sin[rows])
        k = plain.apply_rope(plain.rms_norm(k, w[p + "k_norm.weight"], eps), cos[rows], sin[rows])
        return plain.linear(plain.causal_attention(q, k, v, d ** -0.5).reshape(T, nq * d), w[p + "o_proj.weight"])

    a = plain.rms_norm(attention(plain.rms_norm(stream, w["layers.0.pre_attn.weight"], eps), "layers.0.attn."),
                       w["layers.0.post_attn.weight"], eps)
    stream = stream + a
    x = plain.rms_norm(stream, w["layers.0.pre_ffn.weight"], eps)
    out = []
    for t in range(T):
        e = int((w["layers.0.ffn.router.weight"] @ x[t]).argmax())
        up = w[f"layers.0.ffn.experts.{e}.up_t"].t()                  # stored [H, I]
        out.append(w[f"layers.0.ffn.experts.{e}.down"] @ torch.relu(up @ x[t]))
    stream = stream + plain.rms_norm(torch.stack(out), w["layers.0.post_ffn.weight"], eps)
    a = plain.rms_norm(attention(plain.rms_norm(stream, w["layers.1.pre_attn.weight"], eps), "layers.1.attn."),
                       w["layers.1.post_attn.weight"], eps)
    x = plain.rms_norm(a + stream, w["final_norm.weight"], eps)
    cap = raw["logit_cap"]
    return cap * torch.tanh((x @ w["head.weight"].t() + w["head.bias"]) / cap)


def test_a_block_with_post_norms_a_scaled_embedding_a_capped_head_given_positions_and_another_checkpoint_layout(tmp_path):
    from safetensors.torch import load_file
    from nanohybrid_vlm_b200.config import ARCHITECTURES, Config
    from nanohybrid_vlm_b200.engine import ModelRunner, StepItem
    from nanohybrid_vlm_b200.parts import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, POSITIONS
    from nanohybrid_vlm_b200.weights import WeightError, write_random_model
    register_sandwich_toy()
    try:
        raw = SANDWICH
        d = write_random_model(str(tmp_path / "sandwich"), raw, seed=13)
        w = load_file(f"{d}/model.safetensors")
        # the file is written in the checkpoint's own layout: transposed up matrices, one pair of tensors per expert
        assert w["layers.0.ffn.experts.2.up_t"].shape == (raw["hidden_size"], raw["expert_size"])
        assert w["layers.0.ffn.experts.0.down"].shape == (raw["hidden_size"], raw["expert_size"])
        assert "layers.1.ffn.router.weight" not in w and "layers.1.post_attn.weight" in w and w["head.bias"].abs().max() <= 0.1
        runner = ModelRunner(Config(d, kvcache_block_size=8, num_kvcache_blocks=24, max_num_seqs=3,
                                    max_num_batched_tokens=64, max_model_len=96, enforce_eager=True))
        assert runner.builder.n_axes == 2
        rng = np.random.default_rng(5)
        reqs = {"a": rng.integers(0, raw["vocab_size"], 37).tolist(), "b": rng.integers(0, raw["vocab_size"], 20).tolist()}
        # positions that are not the index in the request: a grid walked row by row, and an offset start
        rows = {"a": [3 + i // 6 for i in range(37)], "b": [50 + i for i in range(20)]}
        cols = {"a": [i % 6 for i in range(37)], "b": [7] * 20}
        ref = {r: sandwich_plain_logits(w, reqs[r], rows[r], cols[r]) for r in reqs}
        used = {int((w["layers.0.ffn.router.weight"] @ x).argmax()) for x in torch.randn(64, raw["hidden_size"], generator=torch.Generator().manual_seed(0))}
        assert len(used) > 1
        cuts = {"a": [19, 1, 17], "b": [2, 17, 1]}
        at, got = {"a": 0, "b": 0}, {"a": [], "b": []}
        for step in range(3):
            items = []
            for r in reqs:
                n = cuts[r][step]
                runner.cache.allocate(r, at[r] + n)
                items.append(StepItem(r, reqs[r][at[r]:at[r] + n], at[r], list(range(n)),
                                      positions=[rows[r][at[r]:at[r] + n], cols[r][at[r]:at[r] + n]]))
                at[r] += n
            logits = runner.step(items).cpu()
            k = 0
            for it in items:
                got[it.req_id].append(logits[k:k + len(it.tokens)])
                k += len(it.tokens)
        for r in reqs:
            torch.testing.assert_close(torch.cat(got[r]), ref[r], rtol=1e-4, atol=2e-5)
        with pytest.raises(ValueError, match="positions must be"):
            runner.cache.allocate("c", 3)
            runner.step([StepItem("c", [1, 2, 3], 0, [], positions=[[0, 1, 2]] * 3)])
        # a checkpoint tensor in another layout than the declared one is a wrong shape, named with both
        from safetensors.torch import save_file
        w["layers.0.ffn.experts.1.up_t"] = w["layers.0.ffn.experts.1.up_t"].t().contiguous()
        save_file(w, f"{d}/model.safetensors")
        with pytest.raises(WeightError, match=r"experts\.1\.up_t: checkpoint \(24, 40\) but the model wants \(40, 24\)"):
            ModelRunner(Config(d, kvcache_block_size=8, num_kvcache_blocks=24, max_num_seqs=3, max_num_batched_tokens=64,
                               max_model_len=96, enforce_eager=True))
        with pytest.raises(ValueError, match="arranges"):
            from nanohybrid_vlm_b200.engine.model import CausalLM
            from nanohybrid_vlm_b200.parts import LayerSpec, PartUse, part
            spec = ARCHITECTURES.resolve(raw).build_spec(ARCHITECTURES.resolve(raw).parse_config(raw))
            bad = LayerSpec(part("prenorm_residual"), mixer=spec.layers[0].mixer, mixer_norm=spec.layers[0].mixer_norm,
                            gate=spec.layers[0].ffn_norm)
            import dataclasses
            CausalLM(dataclasses.replace(spec, layers=(bad,), order=spec.order[:1]), torch.float32, "cuda")
    finally:
        ARCHITECTURES.unregister("ToySandwichLM")
        BLOCKS.unregister("sandwich")
        EMBEDDINGS.unregister("scaled_embedding")
        HEADS.unregister("capped_head")
        POSITIONS.unregister("two_axis")
        FEED_FORWARDS.unregister("stacked_experts")
