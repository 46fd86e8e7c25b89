"""CUDA-graph capture of a layer's forward + backward through the public operator.

The library allocates scratch (cudaMalloc) only when a (device, stream) pair needs more than it has had before, so a
warm-up call on the capture stream makes every later call allocation-free and capturable.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("p", [8.0, 37.5, math.inf])
def test_capture_and_replay_matches_eager(p):
    from l_inf_dist_net_v2_b200 import norm_dist
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C

    torch.manual_seed(0)
    B, CI, CO = 64, 784, 1024
    x = torch.rand(B, CI, 1, device="cuda", requires_grad=True)
    w = torch.randn(CO, CI, device="cuda", requires_grad=True)
    g = torch.randn(B, CO, 1, device="cuda")

    def step():
        x.grad = None
        w.grad = None
        y = norm_dist(x, w, p)
        y.backward(g)
        return y

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):  # warm-up on the capture stream: scratch reaches its final size
            step()
    torch.cuda.current_stream().wait_stream(s)

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        y_static = step()
    gx_static, gw_static = x.grad, w.grad

    for seed in (1, 2):
        torch.manual_seed(seed)
        with torch.no_grad():
            x.copy_(torch.rand(B, CI, 1, device="cuda"))
            w.copy_(torch.randn(CO, CI, device="cuda"))
            g.copy_(torch.randn(B, CO, 1, device="cuda"))
        graph.replay()
        torch.cuda.synchronize()
        y_g, gx_g, gw_g = y_static.detach().clone(), gx_static.clone(), gw_static.clone()
        # eager reference on fresh leaves
        xe = x.detach().clone().requires_grad_(True)
        we = w.detach().clone().requires_grad_(True)
        ye = norm_dist(xe, we, p)
        ye.backward(g)
        assert torch.equal(y_g, ye.detach())
        if math.isinf(p):
            # scatter-add order is free: compare with a tolerance
            assert torch.allclose(gx_g, xe.grad, rtol=1e-5, atol=1e-6)
            assert torch.allclose(gw_g, we.grad, rtol=1e-5, atol=1e-5)
        else:
            assert torch.equal(gx_g, xe.grad) and torch.equal(gw_g, we.grad)
    C.check_status()


def test_graph_stays_valid_when_scratch_grows_later_and_growth_is_refused_during_capture():
    """A captured graph replays with the scratch addresses it was recorded with.  A later, larger eager call on the
    same stream makes the arena grow: the earlier block must stay alive (until ldn_release_scratch), so the replay
    still gives the right result.  And a call that would have to grow the arena while its stream is being captured
    must be refused with status 6 instead of allocating inside the capture."""
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C
    from l_inf_dist_net_v2_b200._lib import lib

    torch.manual_seed(0)
    s = torch.cuda.Stream()

    def small(x, w, y):
        # 2-D problem whose rows are no multiple of 4: operands go through canonical copies in scratch
        C.inf_dist_forward_nograd(x, w, y, 1)

    x = torch.rand(40, 30, 3, device="cuda")
    w = torch.randn(50, 30, device="cuda")
    y = torch.empty(40, 50, 3, device="cuda")
    with torch.cuda.stream(s):
        small(x, w, y)  # warm-up: the arena of this stream now fits the small problem
    s.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        small(x, w, y)
    expected = y.clone()
    # a much larger call on the same stream: the arena has to grow (conv-shaped input whose HW is no multiple of 4
    # cannot be read in place -> canonical copy of 24 MB)
    xb = torch.rand(64, 96, 1022, device="cuda")
    wb = torch.randn(32, 96, device="cuda")
    yb = torch.empty(64, 32, 1022, device="cuda")
    with torch.cuda.stream(s):
        C.inf_dist_forward_nograd(xb, wb, yb, 1)
        # churn the allocator so that a freed block would be reused and overwritten
        junk = [torch.full((1 << 20,), float("nan"), device="cuda") for _ in range(8)]
    s.synchronize()
    y.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, expected)
    del junk
    # growth inside a capture: refused, the capture itself stays usable
    s2 = torch.cuda.Stream()
    with torch.cuda.stream(s2):
        small(x, w, y)
    s2.synchronize()
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2, stream=s2):
        with pytest.raises(RuntimeError, match="status 6"):
            C.inf_dist_forward_nograd(xb, wb, yb, 1)
        small(x, w, y)
    y.fill_(float("nan"))
    g2.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, expected)
    # reserving first makes the large call capturable
    assert lib.ldn_reserve_scratch(s2.cuda_stream, 64 << 20) == 0
    g3 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g3, stream=s2):
        C.inf_dist_forward_nograd(xb, wb, yb, 1)
    ref = yb.clone()
    yb.fill_(float("nan"))
    g3.replay()
    torch.cuda.synchronize()
    assert torch.equal(yb, ref)
    C.check_status()
