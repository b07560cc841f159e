"""A bounded wait that runs out reaches the host.  Nothing here faults or hangs: a test build of the decode
product (``csrc/gemm_slab.cu`` compiled into a library of its own with a wait limit of 4,096 polls and a switch
by which its producer leaves one unit of the ring unsent) lets the consumers' wait run out; the kernel sets its
error word, waits for copies in flight and returns in the ordinary way."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

P, I = ctypes.c_void_p, ctypes.c_int


@pytest.fixture(scope="module")
def starved():
    """The test build, its error word registered with the step's health word like any other kernel's."""
    from nanohybrid_vlm_b200.csrc.build import ensure_variant
    from nanohybrid_vlm_b200.kernels import ops
    lib = ctypes.CDLL(ensure_variant("gemm_slab.cu", {"NHV_WAIT_LIMIT": 4096, "NHV_TEST_DROP_UNIT": 0,
                                                        "NHV_OWN_ERROR_TEXT": 1}, folder=""))
    lib.nhv_gemm_slab.argtypes = [P, P, P, I, I, I, I, I, I, I, P]
    lib.nhv_gemm_slab.restype = I
    lib.nhv_gemm_slab_error.restype = I
    lib.nhv_gemm_slab_error_word.restype = P
    lib.nhv_last_error.restype = ctypes.c_char_p
    ops.register_wait_error_source("gemm_slab (test build)", lib.nhv_gemm_slab_error_word, lib.nhv_gemm_slab_error)
    return lib


def run_product(lib, starve: bool):
    """y = x W^T for one token and a 384 x 96 matrix through ``lib`` (or the engine's own library)."""
    from nanohybrid_vlm_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(384, 96, generator=g) * 0.1).to(torch.bfloat16).cuda()
    x = torch.randn(1, 96, generator=g).to(torch.bfloat16).cuda()
    y = torch.zeros(1, 384, dtype=torch.bfloat16, device="cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    slabs = ops.slab_weight(w, 0, sms)
    if starve:
        rc = lib.nhv_gemm_slab(y.data_ptr(), x.data_ptr(), slabs.data_ptr(), 1, 384, 96, x.stride(0), 384, 0, sms,
                               torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.nhv_last_error()
    else:
        ops.linear_slab(y, x, slabs, 384, 0, sms)
    torch.cuda.synchronize()
    return y, (x.float() @ w.float().t())


def test_a_wait_that_runs_out_sets_the_error_word_and_the_kernel_returns(starved):
    from nanohybrid_vlm_b200.kernels import ops
    y, ref = run_product(starved, starve=True)
    assert starved.nhv_gemm_slab_error() == 2             # the consumers' wait for the unsent unit
    assert starved.nhv_gemm_slab_error() == 0             # reading it cleared it
    # the device is as usable as before: the engine's own build of the same kernel gives the product
    y, ref = run_product(None, starve=False)
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    assert ops.take_wait_errors() == []


def test_the_sampler_hands_the_error_word_to_the_host_and_the_runner_raises(starved):
    from nanohybrid_vlm_b200.engine.runner import ModelRunner
    from nanohybrid_vlm_b200.kernels import KernelError, ops
    logits = torch.randn(3, 50, device="cuda")
    temps = torch.zeros(3, device="cuda")
    seeds = torch.zeros(3, dtype=torch.int64, device="cuda")
    pos = torch.zeros(3, dtype=torch.int32, device="cuda")
    out = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    ops.sample(out, logits, temps, seeds, pos)
    host = out.tolist()
    assert host[3] == 0 and host[:3] == logits.argmax(1).tolist()
    assert ModelRunner._checked(host) == host[:3]
    run_product(starved, starve=True)
    ops.sample(out, logits, temps, seeds, pos)
    host = out.tolist()
    assert host[3] != 0 and host[:3] == logits.argmax(1).tolist()
    with pytest.raises(KernelError, match=r"gemm_slab \(test build\) \(code 2\)"):
        ModelRunner._checked(host)
    ops.sample(out, logits, temps, seeds, pos)            # taken by the raise: the next step is healthy again
    assert out.tolist()[3] == 0


@pytest.mark.parametrize("eager", [True, False])
def test_generation_stops_with_the_kernels_name(starved, eager, model_dirs):
    """Through the entry point, eagerly and through a captured decode graph: the step that reads the tokens of
    the step in which a wait ran out raises instead of handing them out (with decode steps launched ahead of the
    read that is the call after next)."""
    from nanohybrid_vlm_b200 import LLM, SamplingParams
    from nanohybrid_vlm_b200.kernels import KernelError
    llm = LLM(model_dirs["A"], dtype="bfloat16", kvcache_block_size=16, num_kvcache_blocks=32, max_num_seqs=4,
              max_num_batched_tokens=64, max_model_len=128, enforce_eager=eager)
    llm.add_request([1, 2, 3, 4, 5], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    llm.step()
    llm.step()                                            # a decode step (captures the graph when not eager)
    run_product(starved, starve=True)
    with pytest.raises(KernelError, match="a bounded wait ran out in gemm_slab"):
        llm.step()
        llm.step()
    llm.abort_all()                                       # the requests of a failed step are given up
    llm.add_request([1, 2, 3], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    while not llm.is_finished():                          # the word was taken: the engine goes on
        llm.step()


def test_replay_checks_every_step(starved, model_dirs):
    from nanohybrid_vlm_b200.config import Config
    from nanohybrid_vlm_b200.engine.batch import StepItem
    from nanohybrid_vlm_b200.engine.runner import ModelRunner
    from nanohybrid_vlm_b200.kernels import KernelError
    runner = ModelRunner(Config(model_dirs["A"], dtype="float32", kvcache_block_size=16, num_kvcache_blocks=8,
                                max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64))
    runner.cache.allocate("a", 3)
    runner.step([StepItem("a", [1, 2, 3], 0, [2])])
    runner.check_kernels()
    run_product(starved, starve=True)
    with pytest.raises(KernelError, match="gemm_slab"):
        runner.check_kernels()
    runner.check_kernels()
