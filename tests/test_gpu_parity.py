"""GPU parity tests: every entry point of the C ABI (called through the reference-facing module
`l_inf_dist_net_v2_b200.norm_dist_cuda`) against

  * the committed golden vectors made by the reference's pure-torch path (tests/golden/),
  * the CPU checker (oracle/) on seeded inputs, including odd shapes, groups and HW > 1,
  * the reference's own CUDA kernels (oracle/_ref/libldn_ref.so) where that library was built.

Tolerances (relative): p = inf and bounds bit-exact (values and indices); integer p 1e-5; general p 1e-4,
on outputs and on both gradients (gradients relative to the largest gradient magnitude).
"""
import math

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

RTOL_INT = 1e-5
RTOL_GEN = 1e-4


@pytest.fixture(scope="module")
def C():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from l_inf_dist_net_v2_b200 import norm_dist_cuda
    from l_inf_dist_net_v2_b200._lib import lib
    lib.ldn_set_max_ctas(0)
    yield norm_dist_cuda
    lib.ldn_set_max_ctas(0)
    norm_dist_cuda.check_status()


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def is_int_p(p):
    return float(p).is_integer() and 0 <= p <= 8


def rtol_for(p, backward=False):
    e = p - 1 if backward else p
    return RTOL_INT if is_int_p(e) else RTOL_GEN


def rel(a, b):
    a = a.astype(np.float64)
    b = b.astype(np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-30)))


def rel_to_max(a, b):
    a = a.astype(np.float64)
    b = b.astype(np.float64)
    return float(np.max(np.abs(a - b)) / max(float(np.max(np.abs(b))), 1e-30))


def run_forward(C, x, w, p, G):
    y = torch.empty(x.shape[0], w.shape[0], x.shape[2], device="cuda")
    C.norm_dist_forward(dev(x), dev(w), y, G, p)
    return y


def run_backward(C, g, x, w, y, p, G, want_gx=True):
    gx = torch.full(x.shape, float("nan"), device="cuda") if want_gx else None
    gw = torch.full(w.shape, float("nan"), device="cuda")
    C.norm_dist_backward_input_weight(dev(g), dev(x), dev(w), y, gx, gw, G, p)
    return gx, gw


# ------------------------------------------------------------------------------------------------
# golden vectors (reference fallback)
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("max_ctas", [0, 3])
def test_golden_finite_p(C, golden, max_ctas):
    from l_inf_dist_net_v2_b200._lib import lib
    lib.ldn_set_max_ctas(max_ctas)
    for key in [str(c) for c in golden["cases"]]:
        G = int(golden[f"{key}/dims"][3])
        x, w, g = golden[f"{key}/x"], golden[f"{key}/w"], golden[f"{key}/g"]
        for p in [float(v) for v in golden["powers"]]:
            y = run_forward(C, x, w, p, G)
            assert rel(y.cpu().numpy(), golden[f"{key}/p{p}/y"]) < rtol_for(p), (key, p)
            gx, gw = run_backward(C, g, x, w, y, p, G)
            tol = rtol_for(p, backward=True)
            assert rel_to_max(gx.cpu().numpy(), golden[f"{key}/p{p}/gx"]) < tol, (key, p)
            assert rel_to_max(gw.cpu().numpy(), golden[f"{key}/p{p}/gw"]) < tol, (key, p)
            gx2 = torch.full(x.shape, float("nan"), device="cuda")
            C.norm_dist_backward_input(dev(g), dev(x), dev(w), y, gx2, G, p)
            # grad_input alone and the fused grad_input + grad_weight kernel round differently
            assert rel_to_max(gx2.cpu().numpy(), golden[f"{key}/p{p}/gx"]) < tol, (key, p)
    lib.ldn_set_max_ctas(0)
    C.check_status()


@pytest.mark.parametrize("max_ctas", [0, 3])
def test_golden_inf_and_bounds_bit_exact(C, golden, max_ctas):
    from l_inf_dist_net_v2_b200._lib import lib
    lib.ldn_set_max_ctas(max_ctas)
    for key in [str(c) for c in golden["cases"]]:
        G = int(golden[f"{key}/dims"][3])
        x, w, g, g2 = golden[f"{key}/x"], golden[f"{key}/w"], golden[f"{key}/g"], golden[f"{key}/g2"]
        y = torch.empty(golden[f"{key}/inf/y"].shape, device="cuda")
        pos = torch.empty(y.shape, device="cuda", dtype=torch.int32)
        C.inf_dist_forward(dev(x), dev(w), y, pos, G)
        assert np.array_equal(y.cpu().numpy(), golden[f"{key}/inf/y"]), key
        assert np.array_equal(pos.cpu().numpy(), golden[f"{key}/inf/pos"]), key
        y2 = torch.empty_like(y)
        C.inf_dist_forward_nograd(dev(x), dev(w), y2, G)
        assert torch.equal(y, y2)
        gx = torch.full(x.shape, float("nan"), device="cuda")
        gw = torch.full(w.shape, float("nan"), device="cuda")
        C.inf_dist_backward_input_weight(dev(g), pos, gx, gw, G)
        assert rel_to_max(gx.cpu().numpy(), golden[f"{key}/inf/gx"]) < 1e-6, key
        assert rel_to_max(gw.cpu().numpy(), golden[f"{key}/inf/gw"]) < 1e-6, key
        gx2 = torch.full(x.shape, float("nan"), device="cuda")
        C.inf_dist_backward_input(dev(g), pos, gx2, G)
        assert rel_to_max(gx2.cpu().numpy(), golden[f"{key}/inf/gx"]) < 1e-6, key
        # bounds
        xL, xU = golden[f"{key}/xL"], golden[f"{key}/xU"]
        yL = torch.empty_like(y)
        yU = torch.empty_like(y)
        C.bound_inf_dist_forward_nograd(dev(xL), dev(xU), dev(w), yL, yU, G)
        assert np.array_equal(yL.cpu().numpy(), golden[f"{key}/bound/yL"]), key
        assert np.array_equal(yU.cpu().numpy(), golden[f"{key}/bound/yU"]), key
        pL = torch.empty_like(pos)
        pU = torch.empty_like(pos)
        yL2 = torch.empty_like(y)
        yU2 = torch.empty_like(y)
        C.bound_inf_dist_forward(dev(xL), dev(xU), dev(w), yL2, yU2, pL, pU, G)
        assert torch.equal(yL, yL2) and torch.equal(yU, yU2)
        _, _, opL, opU = oracle.bound_inf_dist_forward(xL, xU, w, G)
        assert np.array_equal(pL.cpu().numpy(), opL) and np.array_equal(pU.cpu().numpy(), opU), key
        zeros = torch.zeros_like(y)
        gxl = torch.full(x.shape, float("nan"), device="cuda")
        gxu = torch.full(x.shape, float("nan"), device="cuda")
        gw = torch.full(w.shape, float("nan"), device="cuda")
        C.bound_inf_dist_backward_input_weight(dev(g), zeros, pL, pU, gxl, gxu, gw, G)
        assert rel_to_max(gxl.cpu().numpy(), golden[f"{key}/bound/L_gxL"]) < 1e-6, key
        assert rel_to_max(gxu.cpu().numpy(), golden[f"{key}/bound/L_gxU"]) < 1e-6, key
        assert rel_to_max(gw.cpu().numpy(), golden[f"{key}/bound/L_gw"]) < 1e-6, key
        C.bound_inf_dist_backward_input(zeros, dev(g2), pL, pU, gxl, gxu, G)
        assert rel_to_max(gxl.cpu().numpy(), golden[f"{key}/bound/U_gxL"]) < 1e-6, key
        assert rel_to_max(gxu.cpu().numpy(), golden[f"{key}/bound/U_gxU"]) < 1e-6, key
    lib.ldn_set_max_ctas(0)
    C.check_status()


# ------------------------------------------------------------------------------------------------
# seeded shapes against the CPU checker: odd sizes, groups, HW > 1, several tiles, shared tiles
# ------------------------------------------------------------------------------------------------
SHAPES = [
    # B, CI, CO, G, HW
    (1, 1, 1, 1, 1),
    (3, 17, 10, 1, 1),
    (65, 783, 33, 1, 1),
    (130, 200, 150, 1, 1),
    (64, 784, 1024, 1, 1),
    (37, 96, 40, 4, 1),
    (6, 36, 20, 2, 5),
    (5, 48, 264, 1, 49),
    (300, 260, 10, 1, 1),
    (4, 70, 24, 2, 64),
    # HW >= 96 and a multiple of 4: the input is read in place (k-major operand, one engine group per sample);
    # few outputs per group: 64- and 32-wide tiles
    (3, 40, 24, 2, 100),
    (2, 70, 80, 1, 128),
    (4, 36, 48, 1, 196),
    (2, 33, 130, 1, 260),
]


def make_inputs(shape, seed):
    B, CI, CO, G, HW = shape
    rng = np.random.default_rng(seed)
    x = rng.random((B, CI, HW), dtype=np.float32)
    w = rng.standard_normal((CO, CI // G)).astype(np.float32)
    g = rng.standard_normal((B, CO, HW)).astype(np.float32)
    return x, w, g


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("p", [1.0, 2.0, 3.0, 8.0, 9.0, 2.5, 37.5])
def test_finite_p_against_checker(C, shape, p):
    from l_inf_dist_net_v2_b200._lib import lib
    x, w, g = make_inputs(shape, 1)
    G = shape[3]
    for max_ctas in (0, 5):
        lib.ldn_set_max_ctas(max_ctas)
        y = run_forward(C, x, w, p, G)
        y_ref = oracle.norm_dist_forward(x, w, p, G)
        assert rel(y.cpu().numpy(), y_ref) < rtol_for(p), (shape, p, max_ctas)
        gx, gw = run_backward(C, g, x, w, y, p, G)
        ogx, ogw = oracle.norm_dist_backward(g, x, w, y.cpu().numpy(), p, G)
        tol = rtol_for(p, backward=True)
        assert rel_to_max(gx.cpu().numpy(), ogx) < tol, (shape, p, max_ctas)
        assert rel_to_max(gw.cpu().numpy(), ogw) < tol, (shape, p, max_ctas)
        _, gw_only = run_backward(C, g, x, w, y, p, G, want_gx=False)
        assert rel_to_max(gw_only.cpu().numpy(), ogw) < tol, (shape, p, max_ctas)
        gx_only = torch.full(x.shape, float("nan"), device="cuda")
        C.norm_dist_backward_input(dev(g), dev(x), dev(w), y, gx_only, G, p)
        assert rel_to_max(gx_only.cpu().numpy(), ogx) < tol, (shape, p, max_ctas)
    lib.ldn_set_max_ctas(0)
    C.check_status()


@pytest.mark.parametrize("shape", [(5, 20, 40, 1, 1), (3, 24, 70, 2, 3), (130, 36, 33, 1, 1)])
@pytest.mark.parametrize("p", [60.0, 100.0])
def test_general_p_backward_ragged_large_magnitudes(C, shape, p):
    """Extents that are no multiples of the tile (rows of 128, reduction steps of 32) with |x - w| of 4..8: the
    padding lanes of the general-p backward see |x - 0|^(p-1), which overflows fp32, and must still contribute
    exactly nothing to either gradient."""
    x, w, g = make_inputs(shape, 11)
    x = (4.0 + 4.0 * x).astype(np.float32)
    G = shape[3]
    y = run_forward(C, x, w, p, G)
    y_ref = oracle.norm_dist_forward(x, w, p, G)
    assert rel(y.cpu().numpy(), y_ref) < rtol_for(p)
    ogx, ogw = oracle.norm_dist_backward(g, x, w, y.cpu().numpy(), p, G)
    tol = rtol_for(p, backward=True)
    gx, gw = run_backward(C, g, x, w, y, p, G)
    assert np.isfinite(gx.cpu().numpy()).all() and np.isfinite(gw.cpu().numpy()).all()
    assert rel_to_max(gx.cpu().numpy(), ogx) < tol
    assert rel_to_max(gw.cpu().numpy(), ogw) < tol
    _, gw_only = run_backward(C, g, x, w, y, p, G, want_gx=False)
    assert np.isfinite(gw_only.cpu().numpy()).all() and rel_to_max(gw_only.cpu().numpy(), ogw) < tol
    gx_only = torch.full(x.shape, float("nan"), device="cuda")
    C.norm_dist_backward_input(dev(g), dev(x), dev(w), y, gx_only, G, p)
    assert rel_to_max(gx_only.cpu().numpy(), ogx) < tol
    C.check_status()


@pytest.mark.parametrize("p,tol", [(64.0, 1e-4), (66.0, 1e-4), (300.0, 1e-4), (1000.0, 3e-4)])
def test_large_exponent_gradients(C, p, tol):
    """The reference's schedule raises p to 1000 before switching to p = inf.  Up to p - 1 = 64 the backward folds
    1 / y into the exponent offset; beyond, it takes the logarithm of |t| / y as the reference does.  In fp32 the
    rounding of |t| / y (6e-8) times p - 1 bounds what any implementation can reach: ~1e-4 at p = 1000, hence
    the wider tolerance there; outputs stay within 1e-4 throughout."""
    x, w, g = make_inputs((64, 256, 96, 1, 1), 5)
    y = run_forward(C, x, w, p, 1)
    assert rel(y.cpu().numpy(), oracle.norm_dist_forward(x, w, p, 1)) < RTOL_GEN
    ogx, ogw = oracle.norm_dist_backward(g, x, w, y.cpu().numpy(), p, 1)
    gx, gw = run_backward(C, g, x, w, y, p, 1)
    assert rel_to_max(gx.cpu().numpy(), ogx) < tol
    assert rel_to_max(gw.cpu().numpy(), ogw) < tol
    C.check_status()


@pytest.mark.parametrize("shape", [(700, 96, 40, 1, 1), (300, 64, 48, 2, 1), (9, 24, 16, 1, 100)])
@pytest.mark.parametrize("p", [8.0, 37.5])
def test_fused_backward_in_row_chunks(C, shape, p):
    """With the scratch limit of the fused backward lowered to two row tiles' worth, the batch is processed in
    chunks of whole samples: the input gradient is written chunk by chunk, the weight gradient accumulates."""
    from l_inf_dist_net_v2_b200._lib import lib
    x, w, g = make_inputs(shape, 21)
    B, CI, CO, G, HW = shape
    y = run_forward(C, x, w, p, G)
    ogx, ogw = oracle.norm_dist_backward(g, x, w, y.cpu().numpy(), p, G)
    whole = run_backward(C, g, x, w, y, p, G)
    lib.ldn_set_fused_scratch_limit(2 * CO * (CI // G) * 4)
    try:
        before = lib.ldn_kernel_launches()
        chunked = run_backward(C, g, x, w, y, p, G)
        launches = lib.ldn_kernel_launches() - before
    finally:
        lib.ldn_set_fused_scratch_limit(0)
    rows_per_chunk = max(1, 2 * 128 // HW) * HW
    assert launches >= 3 * -(-B * HW // rows_per_chunk)  # coefficients, tile kernel, column-sum reduction per chunk
    tol = rtol_for(p, backward=True)
    for got, ref_ in ((chunked[0], ogx), (chunked[1], ogw)):
        assert rel_to_max(got.cpu().numpy(), ref_) < tol
    # same terms, but the reduction over outputs may be split between CTAs at other places, and for general p a
    # row's position inside its tile decides which of its exponentials take the polynomial (2.7e-6) path
    same = 1e-6 if is_int_p(p - 1) else 2e-5
    assert rel_to_max(chunked[0].cpu().numpy(), whole[0].cpu().numpy()) < same
    assert rel_to_max(chunked[1].cpu().numpy(), whole[1].cpu().numpy()) < same
    C.check_status()


@pytest.mark.parametrize("ci,hw", [(1000, 96), (2000, 100), (3100, 96), (5000, 100), (6500, 96)])
def test_index_search_of_inputs_read_in_place(C, ci, hw):
    """x[B, C, HW] read in place: the index search keeps a slab of 32, 16 or 8 positions x all channels in shared
    memory (chosen by the reduction length; beyond 6400 channels the general search runs).  Equal maxima inside a
    stage and across stages must give the first channel (inf_dist_cuda.cu:173-177)."""
    rng = np.random.default_rng(ci)
    B, CO = 2, 12
    x = rng.random((B, ci, hw), dtype=np.float32)
    w = rng.standard_normal((CO, ci)).astype(np.float32)
    # channels 7 and 45 repeat channel 3 (same stage / next stage); make that channel the maximum for some outputs
    for k in (7, 45):
        x[:, k] = x[:, 3]
        w[:, k] = w[:, 3]
    w[::3, 3] = w[::3, 7] = w[::3, 45] = 9.0
    oy, opos = oracle.inf_dist_forward(x, w, 1)
    y = torch.empty(B, CO, hw, device="cuda")
    pos = torch.empty(B, CO, hw, device="cuda", dtype=torch.int32)
    C.inf_dist_forward(dev(x), dev(w), y, pos, 1)
    assert np.array_equal(y.cpu().numpy(), oy)
    assert np.array_equal(pos.cpu().numpy(), opos)
    assert (opos[:, ::3] & 0x7fffffff == 3).all()


@pytest.mark.parametrize("shape", SHAPES)
def test_inf_family_against_checker(C, shape):
    from l_inf_dist_net_v2_b200._lib import lib
    x, w, g = make_inputs(shape, 2)
    B, CI, CO, G, HW = shape
    rng = np.random.default_rng(3)
    g2 = rng.standard_normal(g.shape).astype(np.float32)
    eps = np.float32(8.0 / 255.0)
    xL = np.clip(x - eps, 0, 1).astype(np.float32)
    xU = np.clip(x + eps, 0, 1).astype(np.float32)
    # a few inverted intervals exercise the midpoint rule
    if x.size > 4:
        xL.reshape(-1)[::7], xU.reshape(-1)[::7] = xU.reshape(-1)[::7].copy(), xL.reshape(-1)[::7].copy()
    oy, opos = oracle.inf_dist_forward(x, w, G)
    oyL, oyU, opL, opU = oracle.bound_inf_dist_forward(xL, xU, w, G)
    for max_ctas in (0, 5):
        lib.ldn_set_max_ctas(max_ctas)
        y = torch.empty(B, CO, HW, device="cuda")
        pos = torch.empty(B, CO, HW, device="cuda", dtype=torch.int32)
        C.inf_dist_forward(dev(x), dev(w), y, pos, G)
        assert np.array_equal(y.cpu().numpy(), oy), (shape, max_ctas)
        assert np.array_equal(pos.cpu().numpy(), opos), (shape, max_ctas)
        y2 = torch.empty_like(y)
        C.inf_dist_forward_nograd(dev(x), dev(w), y2, G)
        assert torch.equal(y, y2)
        yL, yU = torch.empty_like(y), torch.empty_like(y)
        C.bound_inf_dist_forward_nograd(dev(xL), dev(xU), dev(w), yL, yU, G)
        assert np.array_equal(yL.cpu().numpy(), oyL) and np.array_equal(yU.cpu().numpy(), oyU), (shape, max_ctas)
        for one_pass_limit in (-1, 0):  # one pass for both bounds (default); one pass per bound (very long reductions)
            lib.ldn_set_bound_one_pass_limit(one_pass_limit)
            pL, pU = torch.empty_like(pos), torch.empty_like(pos)
            yL2, yU2 = torch.empty_like(y), torch.empty_like(y)
            C.bound_inf_dist_forward(dev(xL), dev(xU), dev(w), yL2, yU2, pL, pU, G)
            assert torch.equal(yL, yL2) and torch.equal(yU, yU2)
            assert np.array_equal(pL.cpu().numpy(), opL) and np.array_equal(pU.cpu().numpy(), opU), (shape, max_ctas)
        lib.ldn_set_bound_one_pass_limit(-1)
    lib.ldn_set_max_ctas(0)
    # scatters
    gx = torch.full(x.shape, float("nan"), device="cuda")
    gw = torch.full(w.shape, float("nan"), device="cuda")
    C.inf_dist_backward_input_weight(dev(g), dev(opos), gx, gw, G)
    ogx, ogw = oracle.inf_dist_backward(g, opos, x.shape, w.shape, G)
    assert rel_to_max(gx.cpu().numpy(), ogx) < 1e-5 and rel_to_max(gw.cpu().numpy(), ogw) < 1e-5
    gxl = torch.full(x.shape, float("nan"), device="cuda")
    gxu = torch.full(x.shape, float("nan"), device="cuda")
    C.bound_inf_dist_backward_input_weight(dev(g), dev(g2), dev(opL), dev(opU), gxl, gxu, gw, G)
    ol, ou, ow = oracle.bound_inf_dist_backward(g, g2, opL, opU, x.shape, w.shape, G)
    assert rel_to_max(gxl.cpu().numpy(), ol) < 1e-5 and rel_to_max(gxu.cpu().numpy(), ou) < 1e-5
    assert rel_to_max(gw.cpu().numpy(), ow) < 1e-5
    C.check_status()


def test_edge_semantics_on_device(C):
    # floor and pos = 0 when nothing exceeds 1e-10; ties resolve to the first index; sign flag
    x = torch.zeros(2, 8, 1, device="cuda")
    w = torch.zeros(3, 8, device="cuda")
    y = torch.empty(2, 3, 1, device="cuda")
    pos = torch.empty(2, 3, 1, device="cuda", dtype=torch.int32)
    C.inf_dist_forward(x, w, y, pos, 1)
    assert torch.all(y == 1e-10) and torch.all(pos == 0)
    x = torch.tensor([[0.0, 2.0, 0.0, -2.0, 0.0, 2.0]], device="cuda").unsqueeze(-1)
    w = torch.tensor([[2.0, 0.0, -2.0, 0.0, 2.0, 0.0]], device="cuda")
    y = torch.empty(1, 1, 1, device="cuda")
    pos = torch.empty(1, 1, 1, device="cuda", dtype=torch.int32)
    C.inf_dist_forward(x, w, y, pos, 1)
    assert y.item() == 2.0 and pos.item() == -2 ** 31
    # bound: inverted interval collapses to the midpoint, sentinel values of posL / posU
    xL = torch.tensor([[1.0, 0.5]], device="cuda").unsqueeze(-1)
    xU = torch.tensor([[0.0, 0.5]], device="cuda").unsqueeze(-1)
    w = torch.tensor([[0.5, 0.5]], device="cuda")
    yL, yU = torch.empty(1, 1, 1, device="cuda"), torch.empty(1, 1, 1, device="cuda")
    pL = torch.empty(1, 1, 1, device="cuda", dtype=torch.int32)
    pU = torch.empty_like(pL)
    C.bound_inf_dist_forward(xL, xU, w, yL, yU, pL, pU, 1)
    assert yL.item() == np.float32(1e-10) and yU.item() == np.float32(1e-10)
    assert pL.item() == -1 and pU.item() == 0
    assert xL[0, 0, 0].item() == 1.0  # the caller's tensors are untouched
    # p <= 10 underflow floor
    y = torch.empty(1, 1, 1, device="cuda")
    C.norm_dist_forward(torch.zeros(1, 4, 1, device="cuda"), torch.zeros(1, 4, device="cuda"), y, 1, 8.0)
    assert math.isclose(y.item(), 1.175494351e-38 ** (1 / 8), rel_tol=1e-5)
    # p > 10 with all-zero differences: the 1e-10 term alone
    C.norm_dist_forward(torch.zeros(1, 4, 1, device="cuda"), torch.zeros(1, 4, device="cuda"), y, 1, 20.0)
    assert math.isclose(y.item(), 1e-10, rel_tol=1e-4)
    C.check_status()


def test_forward_with_max(C):
    x, w, _ = make_inputs((9, 40, 12, 2, 3), 5)
    m, _ = oracle.inf_dist_forward(x, w, 2, want_pos=False)
    y = torch.empty(9, 12, 3, device="cuda")
    for p in (8.0, 12.0, 37.5):
        C.norm_dist_forward_with_max(dev(x), dev(w), dev(m), y, 2, p)
        assert rel(y.cpu().numpy(), oracle.norm_dist_forward_with_max(x, w, m, p, 2)) < RTOL_GEN, p
    C.check_status()


def test_bad_arguments_raise_before_launch(C):
    x = torch.rand(2, 6, 1, device="cuda")
    w = torch.randn(3, 6, device="cuda")
    y = torch.empty(2, 3, 1, device="cuda")
    with pytest.raises(RuntimeError, match="status 1"):
        C.norm_dist_forward(x, w, y, 1, -1.0)
    with pytest.raises(RuntimeError, match="status 1"):
        C.norm_dist_forward(x, w, y, 4, 8.0)  # CI not divisible by G
    with pytest.raises(RuntimeError, match="contiguous"):
        C.norm_dist_forward(x.transpose(0, 1), w, y, 1, 8.0)
    with pytest.raises(RuntimeError, match="Float"):
        C.norm_dist_forward(x.double(), w, y, 1, 8.0)
    C.check_status()


# ------------------------------------------------------------------------------------------------
# operator / module level (autograd)
# ------------------------------------------------------------------------------------------------
def test_autograd_operator_and_modules(C):
    import l_inf_dist_net_v2_b200 as ldn
    torch.manual_seed(0)
    x_np, w_np, g_np = make_inputs((12, 40, 24, 2, 3), 7)
    for p in (8.0, 37.5, math.inf):
        x = dev(x_np).requires_grad_()
        w = dev(w_np).requires_grad_()
        y = ldn.norm_dist(x, w, p, 2)
        y.backward(dev(g_np))
        if math.isinf(p):
            oy, opos = oracle.inf_dist_forward(x_np, w_np, 2)
            assert np.array_equal(y.detach().cpu().numpy(), oy)
            ogx, ogw = oracle.inf_dist_backward(g_np, opos, x_np.shape, w_np.shape, 2)
            tol = 1e-5
        else:
            oy = oracle.norm_dist_forward(x_np, w_np, p, 2)
            assert rel(y.detach().cpu().numpy(), oy) < rtol_for(p)
            ogx, ogw = oracle.norm_dist_backward(g_np, x_np, w_np, y.detach().cpu().numpy(), p, 2)
            tol = rtol_for(p, True)
        assert rel_to_max(x.grad.cpu().numpy(), ogx) < tol and rel_to_max(w.grad.cpu().numpy(), ogw) < tol
        # weights frozen (the PGD attack path): only grad_input
        x2 = dev(x_np).requires_grad_()
        ldn.norm_dist(x2, dev(w_np), p, 2).backward(dev(g_np))
        assert rel_to_max(x2.grad.cpu().numpy(), ogx) < tol
        # input without grad (first layer): only grad_weight
        w2 = dev(w_np).requires_grad_()
        ldn.norm_dist(dev(x_np), w2, p, 2).backward(dev(g_np))
        assert rel_to_max(w2.grad.cpu().numpy(), ogw) < tol
    with pytest.raises(NotImplementedError):
        ldn.norm_dist(dev(x_np), dev(w_np), 0.0, 2)
    # no-grad path picks the no-grad kernels and gives the same values
    with torch.no_grad():
        y0 = ldn.norm_dist(dev(x_np), dev(w_np), math.inf, 2)
    assert np.array_equal(y0.cpu().numpy(), oracle.inf_dist_forward(x_np, w_np, 2)[0])

    # modules: FC layer with identity init, eval-mode certification triple, conv layer
    layer = ldn.NormDist(40, 64, bias=True, identity_val=10.0, mean_shift=True).cuda()
    xin = dev(x_np[:, :, 0])
    layer.train()
    layer.p = 8.0
    out, lo, up = layer(xin, None, None)
    assert out.shape == (12, 64) and lo is None and up is None
    out.sum().backward()
    assert layer.weight.grad is not None and torch.isfinite(layer.weight.grad).all()
    layer.eval()
    layer.p = math.inf
    with torch.no_grad():
        out, lo, up = layer(xin, (xin - 0.03).clamp(0, 1), (xin + 0.03).clamp(0, 1))
    assert torch.all(lo <= out) and torch.all(out <= up)
    conv = ldn.NormDistConv(4, 8, 3, padding=1, groups=2, bias=True, mean_shift=False).cuda()
    conv.p = math.inf
    img = torch.rand(3, 4, 6, 6, device="cuda")
    with torch.no_grad():
        o, _, _ = conv(img, None, None)
    assert o.shape == (3, 8, 6, 6)
    un = torch.nn.functional.unfold(img, (3, 3), 1, 1, 1)
    oy, _ = oracle.inf_dist_forward(un.cpu().numpy(), conv.weight.detach().cpu().numpy(), 2, want_pos=False)
    assert np.array_equal((o.view(3, 8, 36) - conv.bias.detach().view(1, -1, 1)).cpu().numpy(), oy)
    C.check_status()


# ------------------------------------------------------------------------------------------------
# full benchmark size: subset of rows against the checker + size-independent properties
# ------------------------------------------------------------------------------------------------
def test_full_size_layer(C):
    B, CI, CO = 512, 3072, 5120
    gen = torch.Generator().manual_seed(0)
    x = torch.rand(B, CI, generator=gen)
    w = torch.randn(CO, CI, generator=gen)
    g = torch.randn(B, CO, generator=gen)
    xd, wd, gd = x.cuda().unsqueeze(-1), w.cuda(), g.cuda().unsqueeze(-1)
    rows = [0, 1, 127, 128, 255, 300, 511]
    cols = [0, 5, 127, 128, 2000, 5119]
    xs, ws = x[rows].numpy()[:, :, None], w.numpy()
    # p = inf: bit exact on a row subset; nograd == grad variant everywhere; pos consistent with y everywhere
    y = torch.empty(B, CO, 1, device="cuda")
    pos = torch.empty(B, CO, 1, device="cuda", dtype=torch.int32)
    C.inf_dist_forward(xd, wd, y, pos, 1)
    oy, opos = oracle.inf_dist_forward(xs, ws)
    assert np.array_equal(y[rows].cpu().numpy(), oy) and np.array_equal(pos[rows].cpu().numpy(), opos)
    y2 = torch.empty_like(y)
    C.inf_dist_forward_nograd(xd, wd, y2, 1)
    assert torch.equal(y, y2)
    idx = (pos & 0x7fffffff).long().squeeze(-1)
    t = torch.gather(xd.squeeze(-1), 1, idx) - torch.gather(wd, 1, idx.t()).t()
    assert torch.equal(t.abs(), y.squeeze(-1)) and torch.equal(t < 0, pos.squeeze(-1) < 0)
    # bounds with eps = 8/255: bit exact on the subset, and yL <= y <= yU everywhere
    eps = 8.0 / 255.0
    xL, xU = (xd - eps).clamp(0, 1), (xd + eps).clamp(0, 1)
    yL, yU = torch.empty_like(y), torch.empty_like(y)
    C.bound_inf_dist_forward_nograd(xL, xU, wd, yL, yU, 1)
    oyL, oyU, _, _ = oracle.bound_inf_dist_forward(xL[rows].cpu().numpy(), xU[rows].cpu().numpy(), ws, want_pos=False)
    assert np.array_equal(yL[rows].cpu().numpy(), oyL) and np.array_equal(yU[rows].cpu().numpy(), oyU)
    assert torch.all(yL <= y) and torch.all(y <= yU)
    # p = 8 and p = 37.5: forward subset, grad_x subset rows, grad_w subset rows
    for p in (8.0, 37.5):
        C.norm_dist_forward(xd, wd, y, 1, p)
        assert rel(y[rows].cpu().numpy(), oracle.norm_dist_forward(xs, ws, p)) < rtol_for(p)
        gx = torch.empty_like(xd)
        gw = torch.empty_like(wd)
        C.norm_dist_backward_input_weight(gd, xd, wd, y, gx, gw, 1, p)
        yh = y.cpu().numpy()
        ogx, _ = oracle.norm_dist_backward(g[rows].numpy()[:, :, None], xs, ws, yh[rows], p, want_gw=False)
        assert rel_to_max(gx[rows].cpu().numpy(), ogx) < rtol_for(p, True)
        _, ogw = oracle.norm_dist_backward(g[:, cols].numpy()[:, :, None], x.numpy()[:, :, None], ws[cols],
                                           yh[:, cols], p, want_gx=False)
        assert rel_to_max(gw[cols].cpu().numpy(), ogw) < rtol_for(p, True)
        # translation invariance: shifting x and w by the same constant leaves the distance unchanged
        # (up to the rounding of the shifted inputs)
        C.norm_dist_forward(xd + 0.5, wd + 0.5, y2, 1, p)
        assert rel(y2.cpu().numpy(), yh) < 1e-4
    C.check_status()


# ------------------------------------------------------------------------------------------------
# the reference's own CUDA kernels, when oracle/_ref was built
# ------------------------------------------------------------------------------------------------
def _ref_lib():
    import ctypes
    import os
    from oracle.build import REF_SO
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libldn_ref.so not built")
    return ctypes.CDLL(REF_SO)


def _ptr(t):
    import ctypes
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("shape", [(64, 784, 1024, 1, 1), (130, 200, 150, 1, 1), (6, 36, 20, 2, 5), (512, 3072, 640, 1, 1),
                                   (512, 3072, 5120, 1, 1)])
def test_against_reference_cuda_kernels(C, shape):
    import ctypes
    ref = _ref_lib()
    B, CI, CO, G, HW = shape
    x_np, w_np, g_np = make_inputs(shape, 11)
    x, w, g = dev(x_np), dev(w_np), dev(g_np)
    cf = ctypes.c_float
    dims = (B, CO, CI, G, HW)
    # p = inf: values and argmax indices bit exact
    y, yr = torch.empty(B, CO, HW, device="cuda"), torch.empty(B, CO, HW, device="cuda")
    pos, posr = torch.empty_like(y, dtype=torch.int32), torch.empty_like(y, dtype=torch.int32)
    C.inf_dist_forward(x, w, y, pos, G)
    assert ref.ldn_ref_inf_dist_forward(_ptr(x), _ptr(w), _ptr(yr), _ptr(posr), *dims) == 0
    torch.cuda.synchronize()
    assert torch.equal(y, yr) and torch.equal(pos, posr)
    assert ref.ldn_ref_inf_dist_forward_nograd(_ptr(x), _ptr(w), _ptr(yr), *dims) == 0
    torch.cuda.synchronize()
    assert torch.equal(y, yr)
    # bounds: values and both index arrays bit exact
    eps = 8.0 / 255.0
    xL, xU = (x - eps).clamp(0, 1), (x + eps).clamp(0, 1)
    yL, yU, yLr, yUr = (torch.empty_like(y) for _ in range(4))
    pL, pU, pLr, pUr = (torch.empty_like(pos) for _ in range(4))
    C.bound_inf_dist_forward(xL, xU, w, yL, yU, pL, pU, G)
    assert ref.ldn_ref_bound_inf_dist_forward(_ptr(xL), _ptr(xU), _ptr(w), _ptr(yLr), _ptr(yUr), _ptr(pLr), _ptr(pUr),
                                              *dims) == 0
    torch.cuda.synchronize()
    assert torch.equal(yL, yLr) and torch.equal(yU, yUr) and torch.equal(pL, pLr) and torch.equal(pU, pUr)
    assert ref.ldn_ref_bound_inf_dist_forward_nograd(_ptr(xL), _ptr(xU), _ptr(w), _ptr(yLr), _ptr(yUr), *dims) == 0
    torch.cuda.synchronize()
    assert torch.equal(yL, yLr) and torch.equal(yU, yUr)
    # p = inf and bound backward: both sides scatter-add with atomics, so sums agree to rounding
    g2 = dev(np.random.default_rng(12).standard_normal(g_np.shape).astype(np.float32))
    gx, gw, gxr, gwr = (torch.full_like(t, float("nan")) for t in (x, w, x, w))
    C.inf_dist_backward_input_weight(g, pos, gx, gw, G)
    assert ref.ldn_ref_inf_dist_backward_input_weight(_ptr(g), _ptr(posr), _ptr(gxr), _ptr(gwr), *dims) == 0
    torch.cuda.synchronize()
    assert rel_to_max(gx.cpu().numpy(), gxr.cpu().numpy()) < 1e-5 and rel_to_max(gw.cpu().numpy(), gwr.cpu().numpy()) < 1e-5
    gx.fill_(float("nan"))
    C.inf_dist_backward_input(g, pos, gx, G)
    assert ref.ldn_ref_inf_dist_backward_input(_ptr(g), _ptr(posr), _ptr(gxr), *dims) == 0
    torch.cuda.synchronize()
    assert rel_to_max(gx.cpu().numpy(), gxr.cpu().numpy()) < 1e-5
    gxl, gxu, gxlr, gxur = (torch.full_like(x, float("nan")) for _ in range(4))
    gw.fill_(float("nan"))
    C.bound_inf_dist_backward_input_weight(g, g2, pL, pU, gxl, gxu, gw, G)
    assert ref.ldn_ref_bound_inf_dist_backward_input_weight(_ptr(g), _ptr(g2), _ptr(pLr), _ptr(pUr), _ptr(gxlr),
                                                            _ptr(gxur), _ptr(gwr), *dims) == 0
    torch.cuda.synchronize()
    for got, want in ((gxl, gxlr), (gxu, gxur), (gw, gwr)):
        assert rel_to_max(got.cpu().numpy(), want.cpu().numpy()) < 1e-5
    gxl.fill_(float("nan"))
    gxu.fill_(float("nan"))
    C.bound_inf_dist_backward_input(g, g2, pL, pU, gxl, gxu, G)
    assert ref.ldn_ref_bound_inf_dist_backward_input(_ptr(g), _ptr(g2), _ptr(pLr), _ptr(pUr), _ptr(gxlr), _ptr(gxur),
                                                     *dims) == 0
    torch.cuda.synchronize()
    for got, want in ((gxl, gxlr), (gxu, gxur)):
        assert rel_to_max(got.cpu().numpy(), want.cpu().numpy()) < 1e-5
    if CO > 1024:
        return  # the finite-p part at the full width is covered by test_full_size_layer
    # finite p: outputs and both gradients within the stated tolerances
    for p in (8.0, 3.0, 9.0, 37.5):
        C.norm_dist_forward(x, w, y, G, p)
        assert ref.ldn_ref_norm_dist_forward(_ptr(x), _ptr(w), _ptr(yr), *dims, cf(p)) == 0
        torch.cuda.synchronize()
        assert rel(y.cpu().numpy(), yr.cpu().numpy()) < rtol_for(p), (shape, p)
        gx, gw, gxr, gwr = torch.empty_like(x), torch.empty_like(w), torch.empty_like(x), torch.empty_like(w)
        C.norm_dist_backward_input_weight(g, x, w, yr, gx, gw, G, p)
        assert ref.ldn_ref_norm_dist_backward_input_weight(_ptr(g), _ptr(x), _ptr(w), _ptr(yr), _ptr(gxr), _ptr(gwr),
                                                           *dims, cf(p)) == 0
        torch.cuda.synchronize()
        tol = rtol_for(p, True)
        assert rel_to_max(gx.cpu().numpy(), gxr.cpu().numpy()) < tol, (shape, p)
        assert rel_to_max(gw.cpu().numpy(), gwr.cpu().numpy()) < tol, (shape, p)
    C.check_status()


def test_empty_batch_is_a_no_op(C):
    # like the reference, whose kernels run with every row masked off: empty outputs, zero weight gradient
    w = torch.randn(6, 8, device="cuda")
    x = torch.empty(0, 8, 1, device="cuda")
    y = torch.empty(0, 6, 1, device="cuda")
    pos = torch.empty(0, 6, 1, device="cuda", dtype=torch.int32)
    C.norm_dist_forward(x, w, y, 1, 8.0)
    C.inf_dist_forward(x, w, y, pos, 1)
    C.bound_inf_dist_forward_nograd(x, x, w, y, y.clone(), 1)
    gw = torch.full_like(w, float("nan"))
    C.norm_dist_backward_input_weight(y, x, w, y, torch.empty_like(x), gw, 1, 8.0)
    assert torch.all(gw == 0)
    gw.fill_(float("nan"))
    C.inf_dist_backward_input_weight(y, pos, torch.empty_like(x), gw, 1)
    assert torch.all(gw == 0)
    C.check_status()


def test_fused_mean_shift_matches_torch_operators(C):
    """The one-kernel training-mode MeanShift of fully connected layers against the torch operators the reference
    composes it from (core/modules/basic_modules.py:104-135): output, running mean and input gradient."""
    import l_inf_dist_net_v2_b200 as ldn
    torch.manual_seed(3)
    for B, Cn in ((512, 5120), (37, 70), (1, 5)):
        fused = ldn.MeanShift(Cn, affine=False).cuda().train()
        plain = ldn.MeanShift(Cn, affine=False).cuda().train()
        plain.fused = False
        start = torch.randn(Cn, device="cuda")
        fused.running_mean.copy_(start)
        plain.running_mean.copy_(start)
        x1 = (torch.randn(B, Cn, 1, device="cuda") * 3 + 1).requires_grad_(True)
        x2 = x1.detach().clone().requires_grad_(True)
        g = torch.randn(B, Cn, 1, device="cuda")
        y1 = fused(x1)[0]
        y2 = plain(x2)[0]
        y1.backward(g)
        y2.backward(g)
        assert torch.allclose(y1, y2, rtol=0, atol=2e-6 * 4)
        assert torch.allclose(fused.running_mean, plain.running_mean, rtol=1e-6, atol=1e-6)
        assert torch.allclose(x1.grad, x2.grad, rtol=0, atol=1e-6)
        # eval mode and the bound triple keep the torch path
        fused.eval()
        plain.eval()
        lo, up = x1.detach() - 0.1, x1.detach() + 0.1
        for a, b in zip(fused(x1.detach(), lo, up), plain(x2.detach(), lo, up)):
            assert torch.allclose(a, b, rtol=0, atol=1e-6)
    C.check_status()


@pytest.mark.parametrize("shape", [(130, 200, 150, 1, 1), (6, 36, 20, 2, 5), (3, 40, 24, 2, 100), (64, 784, 1024, 1, 1)])
def test_eval_layer_in_one_kernel_matches_the_separate_steps(C, shape):
    """Eval-mode p = inf layer: distance / bounds, running-mean subtraction and bias folded into the store must give
    the bits of the unfused module (distance kernel, then two torch elementwise passes)."""
    import l_inf_dist_net_v2_b200 as ldn
    from l_inf_dist_net_v2_b200._lib import lib
    B, CI, CO, G, HW = shape
    torch.manual_seed(4)
    for mean_shift, bias in ((True, True), (True, False), (False, True)):
        layer = ldn.NormDistBase(CI, CO, groups=G, bias=bias, mean_shift=mean_shift).cuda().eval()
        with torch.no_grad():
            if mean_shift:
                layer.mean_shift.running_mean.copy_(torch.randn(CO) * 3)
            if bias:
                layer.bias.copy_(torch.randn(CO))
        x = torch.rand(B, CI, HW, device="cuda")
        lo, up = (x - 0.03).clamp(0, 1), (x + 0.03).clamp(0, 1)
        for max_ctas in (0, 5):
            lib.ldn_set_max_ctas(max_ctas)
            with torch.no_grad():
                layer.fused_eval = True
                fused = layer(x, lo, up)
                fused_x_only = layer(x)[0]
                layer.fused_eval = False
                plain = layer(x, lo, up)
            for a, b in zip(fused, plain):
                assert torch.equal(a, b), (shape, mean_shift, bias, max_ctas)
            assert torch.equal(fused_x_only, plain[0])
        lib.ldn_set_max_ctas(0)
    C.check_status()


@pytest.mark.parametrize("p", [8.0, 9.0, 3.0])
@pytest.mark.parametrize("scale", [1e-6, 1e-4, 1.0, 1e4, 3e5])
def test_integer_p_backward_at_extreme_scales(C, p, scale):
    """The integer-p backward multiplies g / y^(p-1) by |t|^(p-1); for outputs around 1e-5 or 1e5 that product leaves
    the fp32 range although the gradient g (|t| / y)^(p-1) itself is of ordinary size (the reference keeps the
    normalised form, norm_dist_cuda.cu:238-243).  The library detects such outputs and recomputes in the normalised
    form: gradients must stay finite and accurate at every scale.  Targets: float64 evaluation of the definition."""
    shape = (70, 96, 40, 2, 1)
    x, w, g = make_inputs(shape, 9)
    x, w = (x * scale).astype(np.float32), (w * scale).astype(np.float32)
    B, CI, CO, G, HW = shape
    xd = x.astype(np.float64).reshape(B, G, 1, CI // G)
    wd = w.astype(np.float64).reshape(G, CO // G, CI // G)
    t = xd - wd[None]                                         # B, G, COg, CIg
    yd = (np.abs(t) ** p).sum(-1) ** (1.0 / p)                # B, G, COg
    y32 = yd.reshape(B, CO, 1).astype(np.float32)
    term = g.astype(np.float64).reshape(B, G, CO // G, 1) * np.sign(t) * (np.abs(t) / yd[..., None]) ** (p - 1)
    gx_ref = term.sum(2).reshape(B, CI, 1)
    gw_ref = -term.sum(0).reshape(CO, CI // G)
    tol = 1e-5 if scale == 1.0 else 1e-4
    gx, gw = run_backward(C, g, x, w, dev(y32), p, G)
    for got, ref_ in ((gx, gx_ref), (gw, gw_ref)):
        got = got.cpu().numpy()
        assert np.isfinite(got).all(), (p, scale)
        assert rel_to_max(got, ref_) < tol, (p, scale, rel_to_max(got, ref_))
    _, gw_only = run_backward(C, g, x, w, dev(y32), p, G, want_gx=False)
    assert rel_to_max(gw_only.cpu().numpy(), gw_ref) < tol, (p, scale)
    gx_only = torch.full(x.shape, float("nan"), device="cuda")
    C.norm_dist_backward_input(dev(g), dev(x), dev(w), dev(y32), gx_only, G, p)
    assert rel_to_max(gx_only.cpu().numpy(), gx_ref) < tol, (p, scale)
    C.check_status()


@pytest.mark.parametrize("shape", [(130, 200, 150, 1, 1), (64, 784, 1024, 1, 1), (9, 40, 96, 1, 5)])
@pytest.mark.parametrize("p", [8.0, 37.5, 2.0])
def test_backward_in_channel_ranges_matches_whole(C, shape, p):
    """The finite-p backward in ranges of output channels (grad_input accumulated over the ranges, grad_weight written
    range by range) against the whole-layer call and the checker; also at a scale where the integer form's range
    guard switches to the normalised form, which must not be added twice."""
    B, CI, CO, G, HW = shape
    for scale in (1.0, 1e-5):
        x, w, g = make_inputs(shape, 17)
        x, w = (x * scale).astype(np.float32), (w * scale).astype(np.float32)
        if scale == 1.0:
            y = run_forward(C, x, w, p, G)
        else:
            t = x.astype(np.float64).transpose(0, 2, 1)[:, :, None, :] - w.astype(np.float64)[None, None]
            y = dev(((np.abs(t) ** p).sum(-1) ** (1.0 / p)).transpose(0, 2, 1).astype(np.float32))
        whole = run_backward(C, g, x, w, y, p, G)
        gx = torch.full(x.shape, float("nan"), device="cuda")
        gw = torch.full(w.shape, float("nan"), device="cuda")
        bounds = [0, CO // 3, CO // 3 + 1, CO]
        for i in range(3):
            C.norm_dist_backward_channels(dev(g), dev(x), dev(w), y, gx, gw, p, bounds[i], bounds[i + 1] - bounds[i], i > 0)
        tol = 1e-4 if scale != 1.0 else 2e-6
        assert rel_to_max(gx.cpu().numpy(), whole[0].cpu().numpy()) < tol, (shape, p, scale)
        assert rel_to_max(gw.cpu().numpy(), whole[1].cpu().numpy()) < tol, (shape, p, scale)
        if scale == 1.0:
            ogx, ogw = oracle.norm_dist_backward(g, x, w, y.cpu().numpy(), p, G)
            assert rel_to_max(gx.cpu().numpy(), ogx) < rtol_for(p, True)
            assert rel_to_max(gw.cpu().numpy(), ogw) < rtol_for(p, True)
    C.check_status()


@pytest.mark.parametrize("shape", [(70, 96, 40, 2, 1), (3, 40, 24, 2, 100), (130, 200, 150, 1, 1)])
@pytest.mark.parametrize("p", [10.5, 37.5, 100.0])
def test_general_p_forward_when_the_cheap_normaliser_is_too_loose(C, shape, p):
    """For 10 < p <= 100 the forward normalises by max|x| + max|w| per output instead of the exact max |x - w|.  When
    inputs and weights nearly coincide (differences of 1e-3 on values around 5) that bound is thousands of times
    too large, every term underflows, and the library must notice and recompute with the exact maximum."""
    B, CI, CO, G, HW = shape
    rng = np.random.default_rng(23)
    x = (5.0 + 1e-3 * rng.random((B, CI, HW))).astype(np.float32)
    w = (5.0 + 1e-3 * rng.standard_normal((CO, CI // G))).astype(np.float32)
    y = run_forward(C, x, w, p, G)
    ref = oracle.norm_dist_forward(x, w, p, G)
    assert np.isfinite(y.cpu().numpy()).all()
    assert rel(y.cpu().numpy(), ref) < RTOL_GEN, (shape, p)
    # and the ordinary case right behind it on the same stream (the guard word alternates between calls)
    x2, w2, _ = make_inputs(shape, 24)
    y2 = run_forward(C, x2, w2, p, G)
    assert rel(y2.cpu().numpy(), oracle.norm_dist_forward(x2, w2, p, G)) < RTOL_GEN
    C.check_status()
