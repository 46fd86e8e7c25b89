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
