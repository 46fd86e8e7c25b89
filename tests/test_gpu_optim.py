"""The one-kernel optimisers (ldn_adam_update / ldn_sgd_update through optim.FusedAdam / FusedSGD) against
torch.optim on the same parameters and gradients, several steps, tensors of odd sizes (vector and tail paths, more
tensors than one launch takes), and updating a subset of the parameters."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [(5120, 3072), (513,), (7, 33), (1,), (10, 5120), (4096 * 8 + 4,)] + [(17 + i,) for i in range(40)]


def _params(seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(*s, generator=g).cuda().requires_grad_() for s in SIZES]


def _set_grads(params, seed):
    g = torch.Generator().manual_seed(seed)
    for q in params:
        q.grad = torch.randn(*q.shape, generator=g).cuda()


@pytest.mark.parametrize("kind", ["adam", "sgd", "sgd_momentum", "sgd_nesterov_wd"])
def test_fused_update_matches_torch_optim(kind):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from l_inf_dist_net_v2_b200.optim import FusedAdam, FusedSGD
    a, b = _params(0), _params(0)
    if kind == "adam":
        fused = FusedAdam(a, lr=0.03, betas=(0.9, 0.99), eps=1e-10)
        ref = torch.optim.Adam(b, lr=0.03, betas=(0.9, 0.99), eps=1e-10)
    elif kind == "sgd":
        fused, ref = FusedSGD(a, lr=0.02), torch.optim.SGD(b, lr=0.02)
    elif kind == "sgd_momentum":
        fused = FusedSGD(a, lr=0.02, momentum=0.9, dampening=0.1)
        ref = torch.optim.SGD(b, lr=0.02, momentum=0.9, dampening=0.1)
    else:
        fused = FusedSGD(a, lr=0.02, momentum=0.9, nesterov=True, weight_decay=1e-3)
        ref = torch.optim.SGD(b, lr=0.02, momentum=0.9, nesterov=True, weight_decay=1e-3)
    for step in range(4):
        _set_grads(a, 10 + step)
        _set_grads(b, 10 + step)
        fused.step()
        ref.step()
        for qa, qb in zip(a, b):
            assert torch.allclose(qa, qb, rtol=2e-6, atol=2e-7), (kind, step, tuple(qa.shape))
    if kind == "adam":
        # state layout of torch.optim.Adam: the reference's checkpoints carry optimizer.state_dict()
        st = fused.state[a[0]]
        assert set(st) == {"step", "exp_avg", "exp_avg_sq"} and st["step"] == 4
        assert torch.allclose(st["exp_avg"], ref.state[b[0]]["exp_avg"], rtol=2e-6, atol=1e-7)
        assert torch.allclose(st["exp_avg_sq"], ref.state[b[0]]["exp_avg_sq"], rtol=2e-6, atol=1e-9)


def test_fused_update_of_a_subset_leaves_the_rest_alone():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from l_inf_dist_net_v2_b200.optim import FusedAdam
    a = _params(1)
    before = [q.detach().clone() for q in a]
    opt = FusedAdam(a, lr=0.01)
    _set_grads(a, 5)
    opt.step(params=[a[1], a[3]])
    for i, (q, q0) in enumerate(zip(a, before)):
        assert torch.equal(q, q0) != (i in (1, 3)), i


def test_capturable_adam_in_a_cuda_graph_matches_torch():
    """FusedAdam(capturable=True) keeps the step count on the device: its step can be recorded in a CUDA graph and
    replayed; four replays must match four eager torch.optim.Adam steps on the same gradients."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from l_inf_dist_net_v2_b200.optim import FusedAdam
    a, b = _params(3), _params(3)
    fused = FusedAdam(a, lr=0.03, betas=(0.9, 0.99), eps=1e-10, capturable=True)
    ref = torch.optim.Adam(b, lr=0.03, betas=(0.9, 0.99), eps=1e-10)
    grads = [torch.zeros_like(q) for q in a]
    for q, g in zip(a, grads):
        q.grad = g
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())

    def load(step):
        gen = torch.Generator().manual_seed(50 + step)
        for g, q in zip(grads, b):
            g.copy_(torch.randn(*g.shape, generator=gen))
            q.grad = g.clone()

    load(0)
    with torch.cuda.stream(s):
        fused.step()           # creates the state; not part of the graph
    torch.cuda.current_stream().wait_stream(s)
    ref.step()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        fused.step()
    for step in range(1, 5):
        load(step)
        graph.replay()
        ref.step()
        torch.cuda.synchronize()
        for qa, qb in zip(a, b):
            assert torch.allclose(qa, qb, rtol=3e-6, atol=3e-7), (step, tuple(qa.shape))
    assert float(fused.state[a[0]]["step"]) == 5.0
