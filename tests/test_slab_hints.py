"""Which copy a decode product names as "read next" (``kernels/ops.py:_slab_product``): learnt from the order of the
products before, only within one model's copies, never a copy that is gone.  The launches are recorded, not run."""
import gc

import pytest
import torch

from nanohybrid_vlm_b200.kernels import ops


class Recorder:
    def __init__(self):
        self.calls = []

    def __call__(self, name, *args):
        self.calls.append((name, args))


@pytest.fixture()
def recorded(monkeypatch):
    rec = Recorder()
    monkeypatch.setattr(ops, "call", rec)
    monkeypatch.setattr(ops, "stream_ptr", lambda: 0)
    monkeypatch.setattr(ops, "SLAB_HINT_BYTES", 65536)
    monkeypatch.setattr(ops, "_slab_after", {})
    monkeypatch.setattr(ops, "_slab_blocks", {})
    monkeypatch.setattr(ops, "_slab_family", {})
    monkeypatch.setattr(ops, "_slab_last", None)
    return rec


def make_copy(family, blocks=4, bytes_per_block=256):
    copy = torch.zeros(blocks * bytes_per_block // 2, dtype=torch.bfloat16)
    ops._slab_blocks[copy.data_ptr()] = blocks
    ops._slab_family[copy.data_ptr()] = family
    return copy


def run(copy):
    out, x = torch.zeros(1, 8, dtype=torch.bfloat16), torch.zeros(1, 16, dtype=torch.bfloat16)
    ops._slab_product(out, x, copy, 1, 8, 16, 0, 148)


def hinted(call):
    """The pointer of the copy that the launch names as next, or None."""
    name, args = call
    return args[10] if name == "nhv_gemm_slab_hint" else None


def test_the_order_of_one_pass_is_the_hint_of_the_next(recorded):
    a, b, c = (make_copy(1) for _ in range(3))
    for copy in (a, b, c):
        run(copy)
    assert [hinted(x) for x in recorded.calls] == [None, None, None]          # nothing is known in the first pass
    for copy in (a, b, c):
        run(copy)
    assert [hinted(x) for x in recorded.calls[3:]] == [b.data_ptr(), c.data_ptr(), a.data_ptr()]   # c was followed by a
    name, args = recorded.calls[3]
    assert args[11:14] == (256, 65536, 4)          # the next copy's bytes per block, what is asked for of them, its blocks


def test_no_hint_across_models_and_none_to_a_copy_that_is_gone(recorded):
    a, b = make_copy(1), make_copy(2)                                          # two models' copies, run in turn
    for _ in range(3):
        run(a)
        run(b)
    assert all(hinted(x) is None for x in recorded.calls)
    c, d = make_copy(3), make_copy(3)
    run(c); run(d); run(c)
    assert hinted(recorded.calls[-1]) == d.data_ptr()
    del d
    gc.collect()
    run(c)
    assert hinted(recorded.calls[-1]) is None
    e = make_copy(3)                                                           # may well lie where d lay: it was not learnt
    run(c)
    assert hinted(recorded.calls[-1]) is None
    run(e); run(c)
    assert hinted(recorded.calls[-1]) == e.data_ptr()                          # now it was


def test_hints_can_be_switched_off(recorded, monkeypatch):
    monkeypatch.setattr(ops, "SLAB_HINT_BYTES", 0)
    a, b = make_copy(1), make_copy(1)
    for _ in range(3):
        run(a)
        run(b)
    assert all(name == "nhv_gemm_slab" for name, _ in recorded.calls)
