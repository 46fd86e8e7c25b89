"""Generate tests/golden/ref_models.npz from the upstream reference's own model code.

Run once in a container that has the upstream checkout; its location must be given in the environment
variable LDN_REFERENCE_ROOT:

    LDN_REFERENCE_ROOT=/path/to/L_inf-dist-net-v2 python tests/golden/make_golden_models.py

The reference's `MLPModel` and `HybridModel` (ell_inf_models.py:16-75) are built as they are, with the
operator calls inside `core.modules.norm_dist` redirected to the reference's pure-torch path
(`use_custom_cuda_func=False`, core/norm_dist.py:99-103,112-120); the reference module imports its CUDA
extension unconditionally, so an empty stand-in module named `norm_dist_cuda` is registered first and no
reference CUDA code runs.  Recorded per model: the initial state_dict, one batch of inputs and targets,
and for p in {8, 37.5, inf}, in training mode: logits, worst-case outputs (margins for the MLP, worst-case
logit differences for the hybrid model), the loss of main.py:304-318 (hinge(mix=0.25) for the MLP,
crossentropy(mix=0) for the hybrid model), every parameter gradient and every MeanShift running mean after
the forward pass (for finite p also how far the reference's own float32 evaluation is from those float64
targets, per quantity, relative to the largest magnitude); in eval mode at p = inf: the certification outputs with interval bounds propagated from
the input (main.py:182-215).  For the MLP a 3-step PGD attack without random start (attack.py:15-36) is
recorded too.

Finite p runs in float64 from the float32 parameters and inputs (the targets the tolerance checks refer
to); p = inf runs in float32 (sub / max only in the distance layers, so the eval-mode MLP is a bit-exact
target).
"""
import functools
import math
import os
import sys
import types

import numpy as np
import torch

REF = os.environ.get("LDN_REFERENCE_ROOT")
if not REF or not os.path.isdir(os.path.join(REF, "core")):
    sys.exit("set LDN_REFERENCE_ROOT to the upstream checkout")
sys.modules.setdefault("norm_dist_cuda", types.ModuleType("norm_dist_cuda"))
sys.path.insert(0, REF)
import core.norm_dist as ref_op  # noqa: E402
import core.modules  # noqa: E402,F401

# (`core.modules` re-exports the function `norm_dist`, which shadows the submodule of the same name as an attribute)
ref_mod = sys.modules["core.modules.norm_dist"]

ref_mod.norm_dist = functools.partial(ref_op.norm_dist, use_custom_cuda_func=False)
ref_mod.bound_inf_dist = functools.partial(ref_op.bound_inf_dist, use_custom_cuda_func=False)
from ell_inf_models import MLPModel, HybridModel  # noqa: E402
from core.modules import NormDistBase, MeanShift  # noqa: E402
from attack import AttackPGD  # noqa: E402
from torch.nn.functional import cross_entropy  # noqa: E402

INPUT_DIM = [1, 4, 4]
BATCH = 16
POWERS = [8.0, 37.5, math.inf]


def hinge(outputs, worst, targets, mix=0.25):  # main.py:304-310
    res = worst.clamp(min=0)
    return (1 - mix) * res.max(dim=1)[0].mean() + mix * res.mean()


def crossentropy(outputs, worst, targets, mix=0.0):  # main.py:313-318
    return (1 - mix) * cross_entropy(worst, targets) + mix * cross_entropy(outputs, targets)


def set_p(model, p):
    for m in model.modules():
        if isinstance(m, NormDistBase):
            m.p = p


def record(out, key, model_fn, loss_fn, eps_train, eps_test, gen):
    torch.manual_seed(0)
    model = model_fn()
    state = {k: v.clone() for k, v in model.state_dict().items()}
    for k, v in state.items():
        out[f"{key}/state/{k}"] = v.numpy()
    out[f"{key}/state_keys"] = np.array(list(state.keys()))
    x = torch.rand(BATCH, *INPUT_DIM, generator=gen)
    t = torch.randint(0, 10, (BATCH,), generator=gen)
    out[f"{key}/inputs"] = x.numpy()
    out[f"{key}/targets"] = t.numpy()
    up = torch.ones(INPUT_DIM[0], 1, 1)
    down = torch.zeros(INPUT_DIM[0], 1, 1)
    def train_step(p, dt):
        model = model_fn().to(dt)
        model.load_state_dict({k: v.to(dt) for k, v in state.items()})
        set_p(model, p)
        model.train()
        logits, worst = model(x.to(dt), targets=t, eps=eps_train, up=up.to(dt), down=down.to(dt))
        loss = loss_fn(logits, worst, t)
        loss.backward()
        res = {"logits": logits.detach().numpy(), "worst": worst.detach().numpy(),
               "loss": np.array(loss.item(), np.float64)}
        for name, prm in model.named_parameters():
            res[f"grad/{name}"] = prm.grad.numpy()
        for name, m in model.named_modules():
            if isinstance(m, MeanShift):
                res[f"running_mean/{name}"] = m.running_mean.numpy()
        return res

    def rel_to_max(a, b):
        return float(np.max(np.abs(a.astype(np.float64) - b)) / max(float(np.max(np.abs(b))), 1e-30))

    for p in POWERS:
        tag = f"{key}/train/p{p}"
        res = train_step(p, torch.float32 if math.isinf(p) else torch.float64)
        for name, v in res.items():
            out[f"{tag}/{name}"] = v if name in ("logits", "worst", "loss") else v.astype(np.float32)
        if not math.isinf(p):
            # how far the reference's own float32 evaluation is from the float64 targets, per quantity: the
            # weight gradients of layers in front of a MeanShift are sums that cancel to a small remainder
            res32 = train_step(p, torch.float32)
            for name, v in res.items():
                out[f"{tag}/ref32_err/{name}"] = np.array(rel_to_max(np.asarray(res32[name]), np.asarray(v, np.float64)))
    # certification: eval mode, p = inf, bounds from the input interval
    model = model_fn()
    model.load_state_dict(state)
    set_p(model, math.inf)
    # running means as a trained network has them: not all zero
    for i, m in enumerate(m for m in model.modules() if isinstance(m, MeanShift)):
        m.running_mean.copy_(torch.linspace(0.2, 1.0, m.out_channels) * (i + 1))
    out[f"{key}/certify/state_keys"] = np.array(list(model.state_dict().keys()))
    for k, v in model.state_dict().items():
        out[f"{key}/certify/state/{k}"] = v.numpy()
    model.eval()
    with torch.no_grad():
        logits, worst = model(x, targets=t, eps=eps_test, up=up, down=down)
        plain = model(x)
    out[f"{key}/certify/logits"] = logits.numpy()
    out[f"{key}/certify/worst"] = worst.numpy()
    out[f"{key}/certify/plain"] = plain.numpy()
    out[f"{key}/eps_train"] = np.array(eps_train)
    out[f"{key}/eps_test"] = np.array(eps_test)
    return model, x, t, up, down


def main():
    out = {}
    gen = torch.Generator().manual_seed(1)
    mlp, x, t, up, down = record(
        out, "mlp", lambda: MLPModel(depth=3, width=32, input_dim=INPUT_DIM, identity_val=10.0),
        hinge, 8.0 / 255.0, 8.0 / 255.0, gen)
    # PGD without random start on the eval-mode p = inf MLP (weights frozen: the grad_input-only kernels)
    attacker = AttackPGD(mlp, 0.1, step_size=0.025, num_steps=3, up=up, down=down, random_start=False)
    adv = attacker.find(x, t)
    out["mlp/pgd/adv"] = adv.detach().numpy()
    record(out, "hybrid", lambda: HybridModel(depth=4, width=32, input_dim=INPUT_DIM, hidden=16, identity_val=10.0),
           crossentropy, 0.0345, 8.0 / 255.0, gen)
    # The identity initialisation makes every hidden unit follow one input closely, and the MeanShift behind it
    # then cancels the weight gradients of the hidden layers to (almost) nothing.  The same two models with plain
    # N(0, 1) weights give gradients of ordinary size in every layer.
    record(out, "mlp_rand", lambda: MLPModel(depth=3, width=32, input_dim=INPUT_DIM, identity_val=None),
           hinge, 8.0 / 255.0, 8.0 / 255.0, gen)
    record(out, "hybrid_rand", lambda: HybridModel(depth=4, width=32, input_dim=INPUT_DIM, hidden=16,
                                                   identity_val=None),
           crossentropy, 0.0345, 8.0 / 255.0, gen)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_models.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
