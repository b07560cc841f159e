"""Logits of decode steps whose block-table rows the batch builder kept from the step before, against the
plain implementation: a finished request's row taken by another with an equal table length, a change of
batch-size bucket and back, a mixed step in between, a request that was given up and comes back.  Eagerly
and through the captured graphs, in 32-bit (tight tolerance: a wrong page shows)."""
import numpy as np
import pytest

from conftest import TINY

pytestmark = pytest.mark.gpu

TOL = 2e-5


class Driver:
    """Teacher-forced requests through ``ModelRunner.run`` (the call generation makes), with the cache manager
    driven by hand as ``bin/trace_run`` does."""

    def __init__(self, model_dir, plain, eager, **kw):
        from nanohybrid_vlm_b200.config import Config
        from nanohybrid_vlm_b200.engine.runner import ModelRunner
        opts = dict(dtype="float32", kvcache_block_size=4, num_kvcache_blocks=80, max_num_seqs=8,
                    max_num_batched_tokens=128, max_model_len=64, enforce_eager=eager, enable_prefix_cache=False)
        opts.update(kw)
        self.runner = ModelRunner(Config(model_dir, **opts))
        self.plain = plain
        self.tokens: dict[str, list[int]] = {}
        self.ref: dict[str, np.ndarray] = {}
        self.held: dict[str, int] = {}
        self.rng = np.random.default_rng(5)
        self.checked = 0

    def new(self, rid, length, vocab):
        self.tokens[rid] = self.rng.integers(0, vocab, length).tolist()
        self.ref[rid] = self.plain.logits(self.tokens[rid]).numpy()
        self.held[rid] = 0

    def step(self, *parts):
        """parts: (request, number of tokens); the last token's logits of every part are checked."""
        from nanohybrid_vlm_b200.engine.batch import StepItem
        items, sampling = [], []
        for rid, n in parts:
            at = self.held[rid]
            self.runner.cache.allocate(rid, at + n)
            items.append(StepItem(rid, self.tokens[rid][at:at + n], at, [n - 1]))
            sampling.append((0.0, 1, at + n))
            self.held[rid] = at + n
        chosen = self.runner.run(items, sampling)
        logits = self.runner.last_logits.cpu().numpy()
        for i, (rid, n) in enumerate(parts):
            want = self.ref[rid][self.held[rid] - 1]
            err = np.abs(logits[i] - want).max()
            assert err <= TOL, f"request {rid!r} position {self.held[rid] - 1}: error {err:.3e}"
            assert chosen[i] == int(want.argmax())
            self.checked += 1

    def end(self, rid):
        self.runner.cache.free(rid)
        self.held[rid] = 0


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("name", list(TINY))
def test_logits_over_kept_block_table_rows(name, eager, model_dirs, plain_models):
    cfg, _ = TINY[name]
    d = Driver(model_dirs[name], plain_models[name], eager)
    V = cfg["vocab_size"]
    for rid, n in (("a", 40), ("b", 30), ("c", 44), ("d", 30), ("e", 36), ("f", 33)):
        d.new(rid, n, V)
    d.step(("a", 5), ("b", 6), ("c", 9))               # a mixed step of prompts
    for _ in range(6):
        d.step(("a", 1), ("b", 1), ("c", 1))           # rows kept; a and b cross page edges on the way
    # b (12 tokens, 3 pages) ends; d takes its row with 3 pages of its own
    d.end("b")
    d.step(("d", 10))
    for _ in range(3):
        d.step(("a", 1), ("d", 1), ("c", 1))
    # a larger bucket and back
    d.step(("e", 7), ("f", 3))
    for _ in range(3):
        d.step(("a", 1), ("d", 1), ("c", 1), ("e", 1), ("f", 1))
    d.end("e"); d.end("f")
    for _ in range(2):
        d.step(("a", 1), ("d", 1), ("c", 1))
    # a mixed step in between two decode steps of the same requests
    d.step(("a", 1), ("e", 11), ("d", 1), ("c", 1))
    d.step(("a", 1), ("d", 1), ("c", 1))
    d.end("e")
    # a is given up and recomputed to where it was: the same name at the same row, the same table length, other pages
    n = d.held["a"]
    d.end("a")
    d.runner.cache.allocate("hold", 7)                 # takes pages from the head of the free list first
    d.step(("a", n))
    for _ in range(4):
        d.step(("a", 1), ("d", 1), ("c", 1))
    # another order of the same requests
    for _ in range(2):
        d.step(("c", 1), ("a", 1), ("d", 1))
    d.runner.cache.check()
    assert d.checked > 60
