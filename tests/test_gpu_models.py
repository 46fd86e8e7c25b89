"""Model-level parity on the GPU: this package's MLPModel / HybridModel, loaded from the reference's state_dict,
replay one training step (p = 8, 37.5, inf) and the p = inf certification pass of the fixture that
tests/golden/make_golden_models.py made from the reference's own models (ell_inf_models.py:16-75, losses of
main.py:304-318), on the real kernels.

Tolerances: the operator-level bounds (integer p 1e-5, general p 1e-4 relative) apply per layer; through the two to
three stacked distance layers of these models the outputs are held to 3e-5 (p = 8) / 1e-4 (p = 37.5) / 1e-5 (p = inf in
training mode, where the batch mean of MeanShift is a float32 sum in another order) of the largest magnitude, the
gradients to 3e-5 (p = 8), 3e-4 (p = 37.5: three stacked general-p backward passes of 1e-4 each) and 1e-5 (p = inf).  The eval-mode p = inf MLP is subtract / max / elementwise only: logits and margins are bit-exact.
"""
import math

import pytest
import torch

import model_parity as mp

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def device_ok():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    yield
    from l_inf_dist_net_v2_b200 import norm_dist_cuda
    norm_dist_cuda.check_status()


@pytest.mark.parametrize("kind", mp.KINDS)
@pytest.mark.parametrize("p", mp.POWERS)
def test_training_step_matches_reference_models(kind, p):
    tol_out = 1e-5 if math.isinf(p) else (3e-5 if p == 8.0 else 1e-4)
    tol_grad = 1e-5 if math.isinf(p) else (3e-5 if p == 8.0 else 3e-4)
    mp.check_training_step(kind, p, torch.device("cuda"), tol_out=tol_out, tol_grad=tol_grad)


@pytest.mark.parametrize("kind", mp.KINDS)
def test_certification_matches_reference_models(kind):
    mp.check_certification(kind, torch.device("cuda"), exact=kind.startswith("mlp"))


def test_pgd_matches_reference_attack():
    mp.check_pgd(torch.device("cuda"))


@pytest.mark.parametrize("p,adam_eps", [(8.0, 1e-10), (math.inf, 1e-3)])
def test_whole_training_step_in_a_cuda_graph(p, adam_eps):
    """Forward, loss, backward and the Adam update (step count on the device) of a small hybrid model recorded in one
    CUDA graph: three warm-up steps plus four replays must leave the parameters where seven eager steps leave them.
    (At p = inf the scatter backward adds with atomics, so gradients differ in their last bits from run to run; Adam
    with the reference's eps = 1e-10 turns such noise on near-zero gradients into full-size steps, hence the larger
    eps there: the comparison is about the graph, not about Adam's conditioning.)"""
    import copy
    import l_inf_dist_net_v2_b200 as ldn
    from l_inf_dist_net_v2_b200.optim import FusedAdam
    torch.manual_seed(0)
    net_a = ldn.HybridModel(depth=4, width=64, input_dim=[1, 8, 8], hidden=32, identity_val=None).cuda()
    net_b = copy.deepcopy(net_a)
    loss_fn = ldn.losses.crossentropy()
    gen = torch.Generator().manual_seed(5)
    x = torch.rand(48, 1, 8, 8, generator=gen).cuda()
    t = torch.randint(0, 10, (48,), generator=gen).cuda()

    def make_step(net):
        ldn.set_p_norm(net, p)
        net.train()
        opt = FusedAdam(list(net.parameters()), lr=0.01, betas=(0.9, 0.99), eps=adam_eps, capturable=True)

        def step():
            logits, worst = net(x, targets=t, eps=0.03)
            loss_fn(logits, worst, t).backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
        return step

    eager = make_step(net_b)
    for _ in range(7):
        eager()
    step = make_step(net_a)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        step()
    for _ in range(4):
        graph.replay()
    torch.cuda.synchronize()
    for (name, qa), qb in zip(net_a.named_parameters(), net_b.parameters()):
        # (p = inf: the scatter backward adds with atomics, so sums differ in the last bits between runs)
        assert torch.allclose(qa, qb, rtol=1e-4, atol=1e-5), name
    for ba, bb in zip(net_a.buffers(), net_b.buffers()):
        assert torch.allclose(ba, bb, rtol=1e-5, atol=1e-6)
