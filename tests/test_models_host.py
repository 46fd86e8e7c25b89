"""Host-side logic of the model layer (models.py, bound_modules.py, modules.py, losses.py, attack.py) against the
fixture made from the reference's own MLPModel / HybridModel, on the CPU: the distance operator is replaced by the
checker's torch port (oracle/torch_port.py), so what is tested here is everything around the kernels --
state_dict compatibility, MeanShift, bias, margins, the interval-bound head, the losses and the PGD loop."""
import math

import pytest
import torch

import model_parity as mp
from oracle import torch_port


@pytest.fixture(autouse=True)
def torch_operator(monkeypatch):
    from l_inf_dist_net_v2_b200 import modules
    monkeypatch.setattr(modules, "norm_dist", lambda x, w, p, groups=1, tag=None: torch_port.norm_dist(x, w, p, groups))
    monkeypatch.setattr(modules, "bound_inf_dist",
                        lambda lo, up, w, groups=1, tag=None: torch_port.bound_inf_dist(lo, up, w, groups))


@pytest.mark.parametrize("kind", mp.KINDS)
@pytest.mark.parametrize("p", mp.POWERS)
def test_training_step_matches_reference_models(kind, p):
    tol = 2e-5 if not math.isinf(p) else 1e-5
    mp.check_training_step(kind, p, torch.device("cpu"), tol_out=tol, tol_grad=1e-4)


@pytest.mark.parametrize("kind", mp.KINDS)
def test_certification_matches_reference_models(kind):
    mp.check_certification(kind, torch.device("cpu"), exact=kind.startswith("mlp"))


def test_pgd_matches_reference_attack():
    mp.check_pgd(torch.device("cpu"))
