"""The library's one entry point that allocates nothing, called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory: a program that gave the whole GPU to
its own pool, code on a latency budget that a device-wide synchronisation inside cudaMalloc would break,
a plugin whose host forbids allocations after start-up.  For them ``nhv_gemm_stream_k_no_alloc`` does the
decode step's matrix product with scratch memory that is built into the library, where the ordinary
entry point ``nhv_gemm_stream_k`` takes scratch buffers from its caller.  This test calls both on the
same inputs, twice in a row (the built-in scratch is shared by all calls and keeps the last call's
contents), and checks that the results agree.  It runs last so that a failure here hides no other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

P, I = ctypes.c_void_p, ctypes.c_int


@pytest.fixture(scope="module")
def lib():
    from nanohybrid_vlm_b200.kernels.library import load_library
    lib = load_library()
    lib.nhv_gemm_stream_k_no_alloc.argtypes = [P, P, P, I, I, I, I, I, I, I, P]
    lib.nhv_gemm_stream_k_no_alloc.restype = I
    return lib


def existing(lib, y, x, w, mode, up):
    """The ordinary entry point, with scratch buffers made by the caller."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    scratch = torch.zeros(sms * 2 * 64 * 16, dtype=torch.float32, device="cuda")
    counters = torch.zeros(8192, dtype=torch.int32, device="cuda")
    M, K = x.shape
    rc = lib.nhv_gemm_stream_k(y.data_ptr(), x.data_ptr(), w.data_ptr(), M, y.shape[1], K, x.stride(0), y.shape[1], mode, up,
                               scratch.data_ptr(), counters.data_ptr(), 8192, sms, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.nhv_last_error()
    assert int(counters.sum()) == 0


def no_alloc(lib, y, x, w, mode, up):
    M, K = x.shape
    rc = lib.nhv_gemm_stream_k_no_alloc(y.data_ptr(), x.data_ptr(), w.data_ptr(), M, y.shape[1], K, x.stride(0), y.shape[1],
                                        mode, up, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.nhv_last_error()


@pytest.mark.parametrize("M,N,K,mode", [(8, 4096, 4096, 0), (3, 1000, 264, 0), (16, 384, 96, 1), (5, 2048, 512, 2)])
def test_no_alloc_entry_point_matches_the_existing_one(lib, M, N, K, mode):
    g = torch.Generator().manual_seed(40 + M)
    rows = 2 * N if mode == 2 else N
    w = (torch.randn(rows, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    out_dtype = torch.float32 if mode == 1 else torch.bfloat16
    for call in range(2):                                    # two calls in a row share the built-in scratch
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
        want = torch.full((M, N), float("nan"), dtype=out_dtype, device="cuda")
        got = torch.full((M, N), float("nan"), dtype=out_dtype, device="cuda")
        existing(lib, want, x, w, mode, N if mode == 2 else 0)
        # the device's own count of free memory sees every allocation, whoever makes it (the framework's
        # counters would not see a cudaMalloc inside the library); the ordinary entry point has run the same
        # kernel just before, so nothing is loaded lazily in between
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        no_alloc(lib, got, x, w, mode, N if mode == 2 else 0)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated during the call"
        torch.testing.assert_close(got.float().cpu(), want.float().cpu(), rtol=2e-2, atol=2e-2)
        ref = x.double().cpu() @ w.double().cpu().t()
        if mode == 2:
            gate, up = ref[:, :N], ref[:, N:]
            ref = gate * torch.sigmoid(gate) * up
        torch.testing.assert_close(got.double().cpu(), ref, rtol=3e-2, atol=3e-2 * ref.abs().max().item() / 4 + 1e-3)
    assert lib.nhv_gemm_stream_k_error() == 0


def test_no_alloc_entry_point_refuses_what_its_scratch_cannot_hold(lib):
    x = torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8, 64, dtype=torch.bfloat16, device="cuda")       # never read: the size check comes first
    y = torch.zeros(1, 8, dtype=torch.bfloat16, device="cuda")
    too_wide = 4096 * 64 + 1
    rc = lib.nhv_gemm_stream_k_no_alloc(y.data_ptr(), x.data_ptr(), w.data_ptr(), 1, too_wide, 64, 64, too_wide, 0, 0,
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 1 and b"4096" in lib.nhv_last_error()
    rc = lib.nhv_gemm_stream_k_no_alloc(y.data_ptr(), x.data_ptr(), w.data_ptr(), 17, 8, 64, 64, 8, 0, 0,
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 1 and b"16 tokens" in lib.nhv_last_error()
