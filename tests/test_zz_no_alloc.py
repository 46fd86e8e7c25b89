"""The allocation-free entry point (ldn_inf_dist_forward_nograd_noalloc) against the regular one and the CPU checker.

Callers that may not allocate device memory while they run -- a server that gave its memory to its own pool
at start-up, a runtime that forbids cudaMalloc after initialisation -- use this variant, whose scratch is a
fixed array inside the library.  The results must be the same bits as ldn_inf_dist_forward_nograd and as the CPU
checker's, also on the second of two calls in a row (the array still holds what the first call left); the
second call must leave the amount of free device memory as it found it; its status word must read 0; and a
problem whose scratch would not fit must be refused before anything runs.  The file name sorts last so that a run that
stops at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, x, w, y, G):
    B, CI, HW = x.shape
    CO = w.shape[0]
    return fn(x.data_ptr(), w.data_ptr(), B, CO, CI, G, HW, y.data_ptr(), torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("shape", [(130, 200, 150, 1, 1), (64, 784, 1024, 1, 1), (6, 36, 20, 2, 5), (65, 783, 33, 1, 1)])
def test_noalloc_matches_regular_entry_point_twice(shape):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import oracle
    from l_inf_dist_net_v2_b200._lib import lib
    B, CI, CO, G, HW = shape
    gen = torch.Generator().manual_seed(42)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):  # two calls in a row, different data, same fixed scratch
        x = torch.rand(B, CI, HW, generator=gen).cuda()
        w = torch.randn(CO, CI // G, generator=gen).cuda()
        y_ref = torch.full((B, CO, HW), float("nan"), device="cuda")
        y_new = torch.full((B, CO, HW), float("nan"), device="cuda")
        assert _call(lib.ldn_inf_dist_forward_nograd, x, w, y_ref, G) == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        assert _call(lib.ldn_inf_dist_forward_nograd_noalloc, x, w, y_new, G) == 0
        torch.cuda.synchronize()
        if call == 1:  # (the first call on a device may load the module that holds the array)
            assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free call changed free device memory"
        # p = inf values are exact, so the tolerance the other tests use for them applies: identical bits
        assert torch.equal(y_ref, y_new), (shape, call)
        y_cpu, _ = oracle.inf_dist_forward(x.cpu().numpy(), w.cpu().numpy(), G, want_pos=False)
        assert np.array_equal(y_new.cpu().numpy(), y_cpu), (shape, call)
        assert lib.ldn_noalloc_check_status(stream) == 0


def test_noalloc_refuses_problems_beyond_the_fixed_scratch():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from l_inf_dist_net_v2_b200._lib import lib
    # HW > 1 needs a padded copy of the input: 64 * 64 * 4096 floats = 64 MiB > 32 MiB
    x = torch.rand(64, 4096, 64, device="cuda")
    w = torch.randn(8, 4096, device="cuda")
    y = torch.empty(64, 8, 64, device="cuda")
    status = _call(lib.ldn_inf_dist_forward_nograd_noalloc, x, w, y, 1)
    assert status == 3
    assert b"scratch" in lib.ldn_status_string(status)
    # the regular entry point (which may allocate) still serves it
    assert _call(lib.ldn_inf_dist_forward_nograd, x, w, y, 1) == 0
    torch.cuda.synchronize()
