"""Replays the model-level reference fixture (tests/golden/ref_models.npz, made by make_golden_models.py from the
reference's MLPModel / HybridModel) on this package's models and compares.  Shared by the CPU test (host-side
logic with the checker's torch port standing in for the operator) and the GPU test (the real kernels)."""
import math
import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
POWERS = [8.0, 37.5, math.inf]


def load_fixture():
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_models.npz"))


KINDS = ["mlp", "hybrid", "mlp_rand", "hybrid_rand"]


def build(kind, device):
    """mlp / hybrid: identity_val = 10 as the reference's recipes use it; *_rand: plain N(0, 1) weights (the weight
    gradients of the hidden layers are then of ordinary size instead of cancelling to almost nothing)."""
    import l_inf_dist_net_v2_b200 as ldn
    ident = None if kind.endswith("_rand") else 10.0
    if kind.startswith("mlp"):
        net = ldn.MLPModel(depth=3, width=32, input_dim=[1, 4, 4], identity_val=ident)
    else:
        net = ldn.HybridModel(depth=4, width=32, input_dim=[1, 4, 4], hidden=16, identity_val=ident)
    return net.to(device)


def load_state(net, fx, prefix, device):
    """Loads the reference's state_dict as it is (strict): proves that reference checkpoints load."""
    keys = [str(k) for k in fx[f"{prefix}_keys"]]
    state = {k: torch.from_numpy(fx[f"{prefix}/{k}"]).to(device) for k in keys}
    missing = net.load_state_dict(state, strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    assert list(net.state_dict().keys()) == keys


def loss_for(kind):
    from l_inf_dist_net_v2_b200 import losses
    return losses.hinge(mix=0.25) if kind.startswith("mlp") else losses.crossentropy(mix=0)


def rel_to_max(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / max(float(np.max(np.abs(b))), 1e-30))


def check_training_step(kind, p, device, tol_out, tol_grad):
    import l_inf_dist_net_v2_b200 as ldn
    fx = load_fixture()
    net = build(kind, device)
    load_state(net, fx, f"{kind}/state", device)
    ldn.set_p_norm(net, p)
    net.train()
    x = torch.from_numpy(fx[f"{kind}/inputs"]).to(device)
    t = torch.from_numpy(fx[f"{kind}/targets"]).to(device)
    eps = float(fx[f"{kind}/eps_train"])
    logits, worst = net(x, targets=t, eps=eps, up=torch.ones(1, 1, 1, device=device),
                        down=torch.zeros(1, 1, 1, device=device))
    loss = loss_for(kind)(logits, worst, t)
    loss.backward()
    tag = f"{kind}/train/p{p}"
    assert rel_to_max(logits.detach().cpu().numpy(), fx[f"{tag}/logits"]) < tol_out, (tag, "logits")
    assert rel_to_max(worst.detach().cpu().numpy(), fx[f"{tag}/worst"]) < tol_out, (tag, "worst")
    assert abs(loss.item() - float(fx[f"{tag}/loss"])) < tol_out * max(1.0, abs(float(fx[f"{tag}/loss"]))), tag
    # Gradients: per tensor, relative to its largest magnitude, within tol_grad or four times the distance of the
    # reference's own float32 evaluation from the float64 target, whichever is larger; and in any case relative to
    # the largest gradient of the whole model (the identity-initialised hidden layers have weight gradients that
    # cancel to ~1e-5 of the last layer's, in the reference as here).
    names = [n for n, _ in net.named_parameters()]
    whole = max(float(np.max(np.abs(fx[f"{tag}/grad/{n}"]))) for n in names)
    for name, prm in net.named_parameters():
        ref = fx[f"{tag}/grad/{name}"]
        assert prm.grad is not None, (tag, name)
        got = prm.grad.cpu().numpy()
        err_abs = float(np.max(np.abs(got.astype(np.float64) - ref)))
        assert err_abs < tol_grad * whole, (tag, name, err_abs / whole)
        if kind.endswith("_rand"):
            own = float(fx[f"{tag}/ref32_err/grad/{name}"]) if f"{tag}/ref32_err/grad/{name}" in fx.files else 0.0
            err = rel_to_max(got, ref)
            assert err < max(tol_grad, 4 * own), (tag, name, err)
    for name, m in net.named_modules():
        if isinstance(m, ldn.MeanShift):
            ref = fx[f"{tag}/running_mean/{name}"]
            assert rel_to_max(m.running_mean.cpu().numpy(), ref) < tol_out, (tag, name)


def check_certification(kind, device, exact):
    import l_inf_dist_net_v2_b200 as ldn
    fx = load_fixture()
    net = build(kind, device)
    load_state(net, fx, f"{kind}/certify/state", device)
    ldn.set_p_norm(net, math.inf)
    net.eval()
    x = torch.from_numpy(fx[f"{kind}/inputs"]).to(device)
    t = torch.from_numpy(fx[f"{kind}/targets"]).to(device)
    eps = float(fx[f"{kind}/eps_test"])
    with torch.no_grad():
        logits, worst = net(x, targets=t, eps=eps, up=torch.ones(1, 1, 1, device=device),
                            down=torch.zeros(1, 1, 1, device=device))
        plain = net(x)
    for got, name in ((logits, "logits"), (worst, "worst"), (plain, "plain")):
        ref = fx[f"{kind}/certify/{name}"]
        if exact and name == "worst" and got.is_cuda:
            # the margins are divided by 2 eps: torch's CUDA division by a scalar multiplies by the reciprocal, its
            # CPU division (which made the fixture) divides, so the last bit may differ
            assert rel_to_max(got.cpu().numpy(), ref) < 2.5e-7, (kind, name)
        elif exact:
            assert np.array_equal(got.cpu().numpy(), ref), (kind, name)
        else:
            assert rel_to_max(got.cpu().numpy(), ref) < 1e-5, (kind, name)
    # certified: every wrong class' worst case stays below the target's
    assert worst.shape == (x.size(0), 10)


def check_pgd(device):
    import l_inf_dist_net_v2_b200 as ldn
    fx = load_fixture()
    net = build("mlp", device)
    load_state(net, fx, "mlp/certify/state", device)
    ldn.set_p_norm(net, math.inf)
    net.eval()
    x = torch.from_numpy(fx["mlp/inputs"]).to(device)
    t = torch.from_numpy(fx["mlp/targets"]).to(device)
    attacker = ldn.AttackPGD(net, 0.1, step_size=0.025, num_steps=3, up=torch.ones(1, 1, 1, device=device),
                             down=torch.zeros(1, 1, 1, device=device), random_start=False)
    adv = attacker.find(x, t)
    assert all(q.requires_grad for q in net.parameters())  # restored
    assert float((adv - x).abs().max()) <= 0.1 + 1e-6
    # the steps are sign steps: every pixel moves by a multiple of the step size, so a differing sign shows
    # as a difference of at least one step; allow none
    assert float((adv.cpu() - torch.from_numpy(fx["mlp/pgd/adv"])).abs().max()) < 1e-6
