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
