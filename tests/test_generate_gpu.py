"""Generation through the Python entry point against the plain implementation: greedy tokens, long
decoding, the first tokens of a sequence, prompts cut into portions beside decoding requests, a pool
so small that requests are preempted and recomputed, seeded temperature sampling."""
import numpy as np
import pytest

import plain_qwen3 as plain
from conftest import TINY

pytestmark = pytest.mark.gpu


def make_llm(model_dir, name, dtype="float32", **kw):
    from nanohybrid_vlm_b200 import LLM
    opts = dict(dtype=dtype, kvcache_block_size=16 if name == "A" else 8, num_kvcache_blocks=128, max_num_seqs=8,
                max_num_batched_tokens=64, max_model_len=TINY[name][0]["max_position_embeddings"],
                poison_cache=True)            # the pools start as NaN: a read of a slot that no step wrote shows
    opts.update(kw)
    return LLM(model_dir, **opts)


def prompts_for(name, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, TINY[name][0]["vocab_size"], n).tolist() for n in lengths]


def assert_greedy_follows(plain_model, prompt, tokens, slack):
    """Each generated token is the plain implementation's best token for the same prefix, or within
    `slack` of it (two logits that close may swap under bfloat16)."""
    seq = list(prompt)
    for t in tokens:
        lg = plain_model.logits(seq)[-1]
        assert lg[t] >= lg.max() - slack, f"token {t} at position {len(seq)}: logit {lg[t]:.4f} vs best {lg.max():.4f}"
        seq.append(t)


@pytest.mark.parametrize("name,lengths,new", [("A", (5, 17, 33), 8), ("B", (1, 9, 40, 71), 12)])
def test_greedy_matches_plain_in_float32(name, lengths, new, model_dirs, plain_models):
    from nanohybrid_vlm_b200 import SamplingParams
    prompts = prompts_for(name, lengths)
    want = [plain_models[name].greedy(p, new) for p in prompts]
    for eager in (True, False):
        llm = make_llm(model_dirs[name], name, enforce_eager=eager)
        out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new, ignore_eos=True), use_tqdm=False)
        assert [o["token_ids"] for o in out] == want, f"enforce_eager={eager}"
        assert all(o["text"] == "" for o in out)
        llm.model_runner.cache.check()
        assert llm.model_runner.cache.num_live() == 0
        del llm


@pytest.mark.parametrize("name", list(TINY))
def test_greedy_in_bfloat16_follows_plain(name, model_dirs, plain_models):
    from nanohybrid_vlm_b200 import SamplingParams
    prompts = prompts_for(name, (3, 20, 45), seed=1)
    llm = make_llm(model_dirs[name], name, dtype="bfloat16")
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True), use_tqdm=False)
    for p, o in zip(prompts, out):
        assert len(o["token_ids"]) == 10
        assert_greedy_follows(plain_models[name], p, o["token_ids"], slack=0.03)


def test_long_decoding_and_first_tokens(model_dirs, plain_models):
    """One- and two-token prompts decoded for 150 tokens: every page edge of a short context is crossed
    token by token, through captured graphs."""
    from nanohybrid_vlm_b200 import SamplingParams
    prompts = prompts_for("A", (1, 2, 3), seed=2)
    llm = make_llm(model_dirs["A"], "A")
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=150, ignore_eos=True), use_tqdm=False)
    for p, o in zip(prompts, out):
        assert o["token_ids"] == plain_models["A"].greedy(p, 150)


def test_portions_beside_decoding_and_preemption_leave_tokens_unchanged(model_dirs, plain_models):
    """Tiny B's workload: prompts of 1, 9, 40 and 71 tokens prefilled in portions of 13 mixed with
    decoding requests; then the same with so few pages that requests are preempted and recomputed."""
    from nanohybrid_vlm_b200 import SamplingParams
    prompts = prompts_for("B", (1, 9, 40, 71), seed=3)
    want = [plain_models["B"].greedy(p, 12) for p in prompts]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    llm = make_llm(model_dirs["B"], "B", max_portion=13)
    assert [o["token_ids"] for o in llm.generate(prompts, sp, use_tqdm=False)] == want
    del llm
    # the prompts take 1 + 2 + 5 + 9 = 17 pages of 8 tokens, so all four are admitted into 19 pages; twelve
    # tokens later they would hold 23, so decoding runs out of pages on the way
    llm = make_llm(model_dirs["B"], "B", num_kvcache_blocks=19, max_portion=13)
    assert [o["token_ids"] for o in llm.generate(prompts, sp, use_tqdm=False)] == want
    assert llm.scheduler.num_preemptions > 0
    llm.model_runner.cache.check()
    assert all(p.num_free == p.num_pages for p in llm.model_runner.cache.pools)


def test_eos_stops_a_request(model_dirs, plain_models):
    from nanohybrid_vlm_b200 import SamplingParams
    prompt = prompts_for("B", (12,), seed=4)[0]
    ref = plain_models["B"].greedy(prompt, 12)
    llm = make_llm(model_dirs["B"], "B", eos=ref[4])
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=12), use_tqdm=False)[0]["token_ids"]
    stop = ref.index(ref[4])
    assert out == ref[:stop + 1]


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(model_dirs, plain_models):
    """Temperature 0.8 with per-request seeds: a request draws the same tokens alone, in a batch, with
    its prompt cut into portions, and they are the tokens the plain sampler draws from the plain
    implementation's logits."""
    from nanohybrid_vlm_b200 import SamplingParams
    prompts = prompts_for("B", (1, 9, 40, 71), seed=5)
    sps = [SamplingParams(temperature=0.8, max_tokens=12, ignore_eos=True, seed=100 + i) for i in range(4)]
    llm = make_llm(model_dirs["B"], "B", max_portion=13)
    together = [o["token_ids"] for o in llm.generate(prompts, sps, use_tqdm=False)]
    alone = [llm.generate([p], sp, use_tqdm=False)[0]["token_ids"] for p, sp in zip(prompts, sps)]
    assert together == alone
    other = llm.generate([prompts[2]], SamplingParams(temperature=0.8, max_tokens=12, ignore_eos=True, seed=7),
                         use_tqdm=False)[0]["token_ids"]
    assert other != together[2]
    for p, sp, got in zip(prompts, sps, together):
        seq = list(p)
        for t in got:
            lg = plain_models["B"].logits(seq)[-1]
            assert t == plain.sample(lg, 0.8, sp.seed, len(seq))
            seq.append(t)


def test_entry_point_checks_its_input(model_dirs):
    from nanohybrid_vlm_b200 import SamplingParams
    llm = make_llm(model_dirs["A"], "A")
    sp = SamplingParams(temperature=0.0, max_tokens=2)
    for bad, exc in (([], ValueError), ([1, -2], ValueError), ([1, True], TypeError), ((1, 2), TypeError),
                     ([1, 256], ValueError), ("text", ValueError)):
        with pytest.raises(exc):
            llm.add_request(bad, sp)
    with pytest.raises(TypeError, match="unknown engine options"):
        make_llm(model_dirs["A"], "A", no_such_option=1)
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1.0)
    with pytest.raises(ValueError):
        SamplingParams(temperature=float("nan"))


def test_prefix_reuse_leaves_tokens_unchanged(model_dirs, plain_models):
    """Requests that share leading pages with an earlier request compute only what is new, and generate the
    same tokens as the plain implementation (which knows nothing of pages)."""
    from nanohybrid_vlm_b200 import SamplingParams
    stem = prompts_for("B", (50,), seed=9)[0]
    prompts = [stem, stem[:33] + [5, 6, 7], stem, stem[:8]]
    want = [plain_models["B"].greedy(p, 6) for p in prompts]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    llm = make_llm(model_dirs["B"], "B")
    assert llm.config.enable_prefix_cache is True
    first = llm.generate(prompts[:1], sp, use_tqdm=False)
    assert llm.model_runner.cache.prefix_hits == 0
    rest = llm.generate(prompts[1:], sp, use_tqdm=False)
    assert [o["token_ids"] for o in first + rest] == want
    # pages of 8 tokens: 33 shared tokens -> 4 pages, the whole 50-token stem -> 6 pages, 8 tokens -> none (its only page is its last)
    assert llm.model_runner.cache.prefix_hits == 4 + 6 + 0
    llm.model_runner.cache.check()
    off = make_llm(model_dirs["B"], "B", enable_prefix_cache=False)
    assert [o["token_ids"] for o in off.generate(prompts, sp, use_tqdm=False)] == want
    assert off.model_runner.cache.prefix_hits == 0


def test_prefill_first_with_a_pool_smaller_than_the_work(model_dirs, plain_models):
    """"prefill_first" with more requests than places and a pool that holds two of them: the head of the
    queue waits for room while the running requests decode on; every request gets the plain model's tokens."""
    from nanohybrid_vlm_b200 import SamplingParams
    prompts = prompts_for("B", (30, 41, 9, 25, 1, 38), seed=11)
    want = [plain_models["B"].greedy(p, 9) for p in prompts]
    sp = SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True)
    # pages of 8 tokens: the longest request ends with 49 tokens = 7 pages; 12 pages hold two requests at most
    llm = make_llm(model_dirs["B"], "B", num_kvcache_blocks=12, max_num_seqs=3, scheduler_policy="prefill_first",
                   max_portion=13, enable_prefix_cache=False)
    assert [o["token_ids"] for o in llm.generate(prompts, sp, use_tqdm=False)] == want
    llm.model_runner.cache.check()
    assert all(p.num_free == p.num_pages for p in llm.model_runner.cache.pools)


@pytest.mark.parametrize("name", list(TINY))
def test_decode_steps_launched_ahead_give_the_same_tokens(name, model_dirs, plain_models):
    """``async_decode``: a decode step is launched before the tokens of the one before have been read.  Greedy and
    seeded sampling give the same tokens as with every step read at once, also when requests end at different
    lengths, when one meets its end-of-sequence token in the middle, and when pages run out (preemption)."""
    from nanohybrid_vlm_b200 import SamplingParams
    prompts = prompts_for(name, (5, 17, 33, 2), seed=21)
    ref = [plain_models[name].greedy(p, 14) for p in prompts]
    eos = ref[1][6]                                           # request 1 stops at its 7th token (or earlier, if it repeats)
    sps = [SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=i != 1) for i, n in enumerate((14, 14, 9, 3))]
    want = [r[:sp.max_tokens] for r, sp in zip(ref, sps)]
    want[1] = ref[1][:ref[1].index(eos) + 1]
    for async_decode in (True, False):
        llm = make_llm(model_dirs[name], name, eos=eos, async_decode=async_decode)
        assert llm.async_decode == async_decode
        out = llm.generate(prompts, sps, use_tqdm=False)
        assert [o["token_ids"] for o in out] == want, f"async_decode={async_decode}"
        llm.model_runner.cache.check()
        assert all(p.num_free == p.num_pages for p in llm.model_runner.cache.pools)
        done = {m.seq_id: m.num_completion_tokens for m in llm.get_completed_request_metrics()}
        assert sorted(done.values()) == sorted(len(w) for w in want)
        del llm
    # temperature sampling with seeds, and a pool so small that decoding requests are preempted
    sps = [SamplingParams(temperature=0.8, max_tokens=12, ignore_eos=True, seed=50 + i) for i in range(4)]
    prompts = prompts_for(name, (15, 16, 31, 8), seed=22)        # every one of them needs another page on the way
    outs = []
    for async_decode in (True, False):
        page = 16 if name == "A" else 8
        llm = make_llm(model_dirs[name], name, async_decode=async_decode, num_kvcache_blocks=sum(-(-len(p) // page) for p in prompts))
        outs.append([o["token_ids"] for o in llm.generate(prompts, sps, use_tqdm=False)])
        assert llm.scheduler.num_preemptions > 0
        del llm
    assert outs[0] == outs[1]


def test_profile_ranges_leave_tokens_unchanged(model_dirs, plain_models):
    """``profile_ranges``: the step, the layer runs and the head stand in NVTX ranges; the numbers are the same."""
    from nanohybrid_vlm_b200 import SamplingParams
    prompts = prompts_for("B", (9, 21), seed=31)
    llm = make_llm(model_dirs["B"], "B", profile_ranges=True)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True), use_tqdm=False)
    assert [o["token_ids"] for o in out] == [plain_models["B"].greedy(p, 5) for p in prompts]


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_requests_arriving_while_others_run_give_the_same_tokens_launched_ahead_or_not(seed, model_dirs, plain_models):
    """Random lives: requests of random lengths arrive between steps, with random limits, some stopping at an
    end-of-sequence token, some sampled with a temperature, prompts that share leading pages, in a pool so small
    that requests wait and are preempted.  With decode steps launched ahead of the read and with every step read at
    once the same tokens come out, and the greedy ones are the plain model's."""
    import random
    from nanohybrid_vlm_b200 import SamplingParams
    name = "B"
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(seed)
    stem = [rng.randrange(vocab) for _ in range(40)]
    jobs = []
    for i in range(14):
        n = rng.choice((1, 2, 7, 8, 9, 23, 40, 57))
        prompt = (stem[:n] if rng.random() < 0.4 else [rng.randrange(vocab) for _ in range(n)])
        greedy = rng.random() < 0.6
        sp = SamplingParams(temperature=0.0 if greedy else 0.9, max_tokens=rng.choice((1, 2, 5, 11, 16)),
                            ignore_eos=rng.random() < 0.5, seed=1000 + i)
        jobs.append((rng.randrange(0, 30), prompt, sp))            # (the step before which it arrives, prompt, params)
    ref0 = plain_models[name].greedy(jobs[0][1], 4)
    eos = ref0[-1]
    results = []
    for async_decode in (True, False):
        llm = make_llm(model_dirs[name], name, eos=eos, async_decode=async_decode, num_kvcache_blocks=22, max_num_seqs=5,
                       max_portion=13, max_num_batched_tokens=48)
        ids, done, step = {}, {}, 0
        todo = sorted(range(len(jobs)), key=lambda j: jobs[j][0])
        while todo or not llm.is_finished():
            while todo and (jobs[todo[0]][0] <= step or llm.is_finished()):
                j = todo.pop(0)
                ids[llm.add_request(list(jobs[j][1]), jobs[j][2])] = j
            finished, _ = llm.step()
            for seq_id, tokens in finished:
                assert ids[seq_id] not in done
                done[ids[seq_id]] = tokens
            step += 1
            assert step < 2000
        assert len(done) == len(jobs)
        llm.model_runner.cache.check()
        assert all(p.num_free == p.num_pages for p in llm.model_runner.cache.pools)
        results.append(done)
        del llm
    assert results[0] == results[1]
    for j, (_, prompt, sp) in enumerate(jobs):
        got = results[0][j]
        assert 1 <= len(got) <= sp.max_tokens
        if sp.temperature == 0.0:
            want = plain_models[name].greedy(prompt, sp.max_tokens)
            if not sp.ignore_eos and eos in want:
                want = want[:want.index(eos) + 1]
            assert got == want, f"job {j}"
