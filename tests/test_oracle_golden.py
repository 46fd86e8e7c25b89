"""Pin the CPU checker (oracle/ldn_oracle.c) to vectors produced by the reference's own
pure-torch implementation (tests/golden/ref_fallback.npz, made by tests/golden/make_golden.py)."""
import numpy as np
import pytest

import oracle

# The fallback has neither the 1e-10 term of the p > 10 kernel nor the 1.175e-38 floor of the
# p <= 10 kernel; on the golden inputs (distances of order 1) both are far below float32 resolution.
RTOL_FWD = 2e-6
RTOL_BWD = 2e-5


def _cases(golden):
    return [str(c) for c in golden["cases"]]


def _rel(a, b):
    scale = np.maximum(np.abs(b), 1e-30)
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64)) / scale))


def _rel_to_max(a, b):
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))) / max(float(np.max(np.abs(b))), 1e-30))


def test_finite_p_forward_backward(golden):
    for key in _cases(golden):
        B, CI, CO, G, HW = [int(v) for v in golden[f"{key}/dims"]]
        x, w, g = golden[f"{key}/x"], golden[f"{key}/w"], golden[f"{key}/g"]
        for p in golden["powers"]:
            p = float(p)
            y = oracle.norm_dist_forward(x, w, p, G)
            y_ref = golden[f"{key}/p{p}/y"]
            assert y.shape == y_ref.shape
            assert _rel(y, y_ref) < RTOL_FWD, (key, p)
            gx, gw = oracle.norm_dist_backward(g, x, w, y, p, G)
            assert _rel_to_max(gx, golden[f"{key}/p{p}/gx"]) < RTOL_BWD, (key, p)
            assert _rel_to_max(gw, golden[f"{key}/p{p}/gw"]) < RTOL_BWD, (key, p)


def test_inf_forward_bit_exact(golden):
    for key in _cases(golden):
        G = int(golden[f"{key}/dims"][3])
        y, pos = oracle.inf_dist_forward(golden[f"{key}/x"], golden[f"{key}/w"], G)
        assert np.array_equal(y, golden[f"{key}/inf/y"]), key
        assert np.array_equal(pos, golden[f"{key}/inf/pos"]), key
        y2, none = oracle.inf_dist_forward(golden[f"{key}/x"], golden[f"{key}/w"], G, want_pos=False)
        assert none is None and np.array_equal(y2, y)


def test_inf_backward(golden):
    for key in _cases(golden):
        G = int(golden[f"{key}/dims"][3])
        x, w, g = golden[f"{key}/x"], golden[f"{key}/w"], golden[f"{key}/g"]
        gx, gw = oracle.inf_dist_backward(g, golden[f"{key}/inf/pos"], x.shape, w.shape, G)
        assert _rel_to_max(gx, golden[f"{key}/inf/gx"]) < 1e-6, key
        assert _rel_to_max(gw, golden[f"{key}/inf/gw"]) < 1e-6, key


def test_bound_forward_bit_exact_and_backward(golden):
    for key in _cases(golden):
        G = int(golden[f"{key}/dims"][3])
        xL, xU, w = golden[f"{key}/xL"], golden[f"{key}/xU"], golden[f"{key}/w"]
        yL, yU, pL, pU = oracle.bound_inf_dist_forward(xL, xU, w, G)
        assert np.array_equal(yL, golden[f"{key}/bound/yL"]), key
        assert np.array_equal(yU, golden[f"{key}/bound/yU"]), key
        zeros = np.zeros_like(yL)
        g, g2 = golden[f"{key}/g"], golden[f"{key}/g2"]
        gxL, gxU, gw = oracle.bound_inf_dist_backward(g, zeros, pL, pU, xL.shape, w.shape, G)
        assert _rel_to_max(gxL, golden[f"{key}/bound/L_gxL"]) < 1e-6, key
        assert _rel_to_max(gxU, golden[f"{key}/bound/L_gxU"]) < 1e-6, key
        assert _rel_to_max(gw, golden[f"{key}/bound/L_gw"]) < 1e-6, key
        gxL, gxU, gw = oracle.bound_inf_dist_backward(zeros, g2, pL, pU, xL.shape, w.shape, G)
        assert _rel_to_max(gxL, golden[f"{key}/bound/U_gxL"]) < 1e-6, key
        assert _rel_to_max(gxU, golden[f"{key}/bound/U_gxU"]) < 1e-6, key
        assert _rel_to_max(gw, golden[f"{key}/bound/U_gw"]) < 1e-6, key


def test_edge_semantics():
    # value floor and pos = 0 when nothing exceeds 1e-10 (inf_dist_cuda.cu:131-132)
    x = np.zeros((2, 4, 1), np.float32)
    w = np.zeros((3, 4), np.float32)
    y, pos = oracle.inf_dist_forward(x, w)
    assert np.all(y == np.float32(1e-10)) and np.all(pos == 0)
    # first index wins ties, sign flag for negative difference (inf_dist_cuda.cu:173-177)
    x = np.array([[[0.0], [2.0], [0.0], [-2.0]]], np.float32)
    w = np.array([[2.0, 0.0, -2.0, 0.0]], np.float32)
    y, pos = oracle.inf_dist_forward(x, w)
    assert y[0, 0, 0] == 2.0 and pos[0, 0, 0] == np.int32(-2 ** 31)  # index 0, negative
    # bound: xL > xU collapses to the midpoint; posL sentinel when the lower bound is the floor
    xL = np.array([[[1.0], [0.5]]], np.float32)
    xU = np.array([[[0.0], [0.5]]], np.float32)
    w = np.array([[0.5, 0.5]], np.float32)
    yL, yU, pL, pU = oracle.bound_inf_dist_forward(xL, xU, w)
    assert yL[0, 0, 0] == np.float32(1e-10) and yU[0, 0, 0] == np.float32(1e-10)
    assert pL[0, 0, 0] == -1 and pU[0, 0, 0] == 0
    # p <= 10 underflow floor (norm_dist_cuda.cu:230)
    y = oracle.norm_dist_forward(np.zeros((1, 3, 1), np.float32), np.zeros((1, 3), np.float32), 8.0)
    assert np.isclose(y[0, 0, 0], np.float32(1.175494351e-38) ** (1 / 8), rtol=1e-6)
    # p = 1 backward: term is +g where t == 0 (norm_dist_cuda.cu:238-243)
    x = np.array([[[1.0], [3.0]]], np.float32)
    w = np.array([[1.0, 1.0]], np.float32)
    yv = oracle.norm_dist_forward(x, w, 1.0)
    gx, gw = oracle.norm_dist_backward(np.ones((1, 1, 1), np.float32), x, w, yv, 1.0)
    assert gx[0, 0, 0] == 1.0 and gx[0, 1, 0] == 1.0 and gw[0, 0] == -1.0


def test_forward_with_max_matches_plain_forward():
    rng = np.random.default_rng(1)
    x = rng.random((4, 20, 3), dtype=np.float32)
    w = rng.standard_normal((6, 10)).astype(np.float32)
    m, _ = oracle.inf_dist_forward(x, w, 2, want_pos=False)
    y1 = oracle.norm_dist_forward_with_max(x, w, m, 12.0, 2)
    y2 = oracle.norm_dist_forward(x, w, 12.0, 2)
    assert _rel(y1, y2) < 1e-6


def test_torch_port_matches_reference_vectors(golden):
    import torch
    from oracle import torch_port
    for key in _cases(golden):
        G = int(golden[f"{key}/dims"][3])
        x = torch.from_numpy(golden[f"{key}/x"])
        w = torch.from_numpy(golden[f"{key}/w"])
        for p in (3.0, 8.0, 37.5):
            y = torch_port.norm_dist(x.double(), w.double(), p, G)
            assert _rel(y.numpy(), golden[f"{key}/p{p}/y"]) < 1e-12, (key, p)
        y = torch_port.norm_dist(x, w, float("inf"), G)
        assert np.array_equal(y.numpy(), golden[f"{key}/inf/y"]), key
        yL, yU = torch_port.bound_inf_dist(torch.from_numpy(golden[f"{key}/xL"]), torch.from_numpy(golden[f"{key}/xU"]), w, G)
        assert np.array_equal(yL.numpy(), golden[f"{key}/bound/yL"]) and np.array_equal(yU.numpy(), golden[f"{key}/bound/yU"])
        if G == 1:
            g = torch.from_numpy(golden[f"{key}/g"])
            y, gx, gw = torch_port.norm_dist_fwd_bwd(x.double(), w.double(), g.double(), 8.0, chunk=7)
            assert _rel(y.numpy(), golden[f"{key}/p8.0/y"]) < 1e-12
            assert _rel_to_max(gx.numpy(), golden[f"{key}/p8.0/gx"]) < 1e-6
            assert _rel_to_max(gw.numpy(), golden[f"{key}/p8.0/gw"]) < 1e-6
