"""GPU tests of the diagnostic entry points: launch counter, pipe probes, per-CTA trace, scratch release,
status word."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from l_inf_dist_net_v2_b200._lib import lib
    return lib


def _stream():
    return torch.cuda.current_stream().cuda_stream


def test_launch_counter_and_status(lib):
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C
    x = torch.rand(64, 128, 1, device="cuda")
    w = torch.randn(96, 128, device="cuda")
    y = torch.empty(64, 96, 1, device="cuda")
    before = lib.ldn_kernel_launches()
    C.norm_dist_forward(x, w, y, 1, 8.0)
    after = lib.ldn_kernel_launches()
    assert 1 <= after - before <= 3  # tile kernel (+ fix-up)
    assert lib.ldn_check_status(_stream()) == 0


def test_pipe_probes_report_plausible_rates(lib):
    sink = torch.zeros(64, device="cuda")
    ops = ctypes.c_ulonglong(0)
    rates = {}
    for kind, iters in ((0, 2000), (1, 500), (2, 2000), (3, 500), (4, 300), (5, 300)):
        best = float("inf")
        for _ in range(3):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            assert lib.ldn_probe_pipe(kind, iters, sink.data_ptr(), ctypes.byref(ops), _stream()) == 0
            e.record()
            torch.cuda.synchronize()
            best = min(best, s.elapsed_time(e))
        rates[kind] = ops.value / (best * 1e-3) / 1e12
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    nominal_fp32 = sms * 128 * 1.965e9 / 1e12
    assert 0.5 * nominal_fp32 < rates[0] < 1.1 * nominal_fp32
    assert 0.5 * nominal_fp32 < rates[2] < 1.1 * nominal_fp32
    assert 0.5 * nominal_fp32 / 8 < rates[1] < 1.1 * nominal_fp32 / 8
    # general-p instruction streams: between 1 and 5 Tpair/s (1.5 / 1.125 MUFU operations per pair)
    assert 1.0 < rates[4] < 5.0 and 1.0 < rates[5] < 5.0
    assert lib.ldn_probe_pipe(7, 10, sink.data_ptr(), ctypes.byref(ops), _stream()) == 1  # bad kind


def test_trace_buffer_records_every_cta(lib):
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    x = torch.rand(512, 1024, 1, device="cuda")
    w = torch.randn(2048, 1024, device="cuda")
    y = torch.empty(512, 2048, 1, device="cuda")
    trace = torch.zeros(4 * sms, dtype=torch.int64, device="cuda")
    lib.ldn_set_trace_buffer(trace.data_ptr())
    try:
        C.inf_dist_forward_nograd(x, w, y, 1)
        torch.cuda.synchronize()
    finally:
        lib.ldn_set_trace_buffer(None)
    t = trace.cpu().view(sms, 4)
    used = t[:, 3] > 0
    tiles, kt = 4 * 16, 32
    assert int(t[used, 3].sum()) == tiles * kt            # every k-step was taken by exactly one CTA
    assert torch.all(t[used, 2] >= t[used, 1])             # end after start
    assert torch.all(t[used, 0] < sms)


def test_release_scratch_then_reuse(lib):
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C
    x = torch.rand(5, 37, 3, device="cuda")
    w = torch.randn(8, 37, device="cuda")
    y1, y2 = torch.empty(5, 8, 3, device="cuda"), torch.empty(5, 8, 3, device="cuda")
    C.inf_dist_forward_nograd(x, w, y1, 1)
    torch.cuda.synchronize()
    assert lib.ldn_release_scratch() == 0
    C.inf_dist_forward_nograd(x, w, y2, 1)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    C.check_status()


def test_kernel_timing_hook(lib):
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C
    x = torch.rand(256, 512, 1, device="cuda")
    w = torch.randn(512, 512, device="cuda")
    y = torch.empty(256, 512, 1, device="cuda")
    lib.ldn_enable_kernel_timing(1)
    try:
        C.norm_dist_forward(x, w, y, 1, 8.0)
        ms = lib.ldn_last_tile_kernel_ms()
    finally:
        lib.ldn_enable_kernel_timing(0)
    assert 0.0 < ms < 50.0


def test_two_host_threads_on_one_stream(lib):
    """Calls from two host threads that use the same stream share one scratch block; the library serialises such
    calls, so each one's helper kernels and tile kernel stay together in stream order."""
    import threading

    import numpy as np
    import oracle

    rng = np.random.default_rng(7)
    B, CI, CO, HW = 6, 30, 50, 3  # HW > 1 and CI % 4 != 0: both operands go through canonical copies in scratch
    cases = []
    for _ in range(2):
        x = rng.random((B, CI, HW), dtype=np.float32)
        w = rng.standard_normal((CO, CI)).astype(np.float32)
        cases.append((torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), torch.empty(B, CO, HW, device="cuda"),
                      oracle.inf_dist_forward(x, w, 1)[0]))
    stream = _stream()
    errors = []

    def worker(case):
        xd, wd, yd, _ = case
        for _ in range(200):
            st = lib.ldn_inf_dist_forward_nograd(xd.data_ptr(), wd.data_ptr(), B, CO, CI, 1, HW, yd.data_ptr(), stream)
            if st != 0:
                errors.append(st)
                return

    threads = [threading.Thread(target=worker, args=(c,)) for c in cases]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    assert not errors
    for _, _, yd, ref in cases:
        assert np.array_equal(yd.cpu().numpy(), ref)
    assert lib.ldn_check_status(stream) == 0

