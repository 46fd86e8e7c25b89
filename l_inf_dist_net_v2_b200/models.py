"""The two fully connected model families of the reference (ell_inf_models.py:16-75) on this package's layers,
with the reference's constructor arguments, sub-module names (`fc_dist`, `fc_linear`, `fc_final`, `scalar`:
its checkpoints load) and forward contract:

    model(x)                                  -> logits
    model(x, targets=t, eps=e, up=u, down=d)  -> (logits, worst)

`worst` is what the losses and the certified accuracy are computed from.  While training, or at finite p,
the distance layers only propagate x and the interval [x - eps, x + eps] is attached to their output (the
network is 1-Lipschitz in the l_inf norm); in eval mode with every distance layer at p = inf and `up` /
`down` given, the input box [max(x - eps, down), min(x + eps, up)] is propagated through every layer
(certification, main.py:182-215).
"""
import math

import torch
import torch.nn as nn

from .bound_modules import BoundFinalLinear, BoundLinear, BoundSequential, BoundTanh
from .modules import NormDist, NormDistBase

__all__ = ["MLPModel", "HybridModel", "check_inf_and_eval", "set_p_norm"]


def check_inf_and_eval(model):
    """True when every distance layer of `model` is at p = inf and in eval mode (ell_inf_models.py:9-13)."""
    return all(math.isinf(m.p) and not m.training for m in model.modules() if isinstance(m, NormDistBase))


def set_p_norm(model, p):
    """Sets the exponent of every distance layer (what the reference's schedule does each minibatch,
    main.py:269-272)."""
    for m in model.modules():
        if isinstance(m, NormDistBase):
            m.p = p


def _flat_triple(x, eps, up, down, certify):
    flat = x.flatten(1)
    if not certify:
        return flat, None, None
    return flat, torch.maximum(x - eps, down).flatten(1), torch.minimum(x + eps, up).flatten(1)


def _dist_stack(sizes, last_bias, std, identity_val):
    layers = []
    for i in range(len(sizes) - 1):
        last = last_bias and i == len(sizes) - 2
        layers.append(NormDist(sizes[i], sizes[i + 1], bias=last, mean_shift=not last, std=std,
                               identity_val=identity_val))
    return BoundSequential(*layers)


class MLPModel(nn.Module):
    """depth distance layers: pixels -> width -> ... -> width -> num_classes; logits are the negated distances of
    the last layer (times `scalar`), worst = margins / (2 eps)."""

    def __init__(self, depth, width, input_dim, num_classes=10, std=1.0, identity_val=None, scalar=False):
        super().__init__()
        pixels = input_dim[0] * input_dim[1] * input_dim[2]
        self.fc_dist = _dist_stack([pixels] + [width] * (depth - 1) + [num_classes], True, std, identity_val)
        self.scalar = nn.Parameter(torch.ones(1)) if scalar else 1

    def forward(self, x=None, targets=None, eps=0, up=None, down=None):
        certify = up is not None and down is not None and check_inf_and_eval(self)
        dist, lower, upper = self.fc_dist(_flat_triple(x, eps, up, down, certify))
        if targets is None:
            return -dist * self.scalar
        if lower is None:
            lower = dist - eps
        if upper is None:
            upper = dist + eps
        # scores are negated distances: the score of class j lies in [-upper_j, -lower_j]
        col = targets.view(-1, 1)
        margin = (-lower) - torch.gather(-upper, 1, col)
        margin = margin.scatter(1, col, 0)
        return -dist * self.scalar, margin / (2 * eps)


class HybridModel(nn.Module):
    """depth - 2 distance layers (all with mean shift, no bias) followed by an interval-bound head
    width -> hidden -> tanh -> num_classes."""

    def __init__(self, depth, width, input_dim, hidden=512, num_classes=10, std=1.0, identity_val=None):
        super().__init__()
        pixels = input_dim[0] * input_dim[1] * input_dim[2]
        self.fc_dist = _dist_stack([pixels] + [width] * (depth - 2), False, std, identity_val)
        self.fc_linear = BoundSequential(BoundLinear(width, hidden, bias=True), BoundTanh())
        self.fc_final = BoundFinalLinear(hidden, num_classes, bias=True)

    def forward(self, x=None, targets=None, eps=0, up=None, down=None):
        certify = up is not None and down is not None and check_inf_and_eval(self)
        dist, lower, upper = self.fc_dist(_flat_triple(x, eps, up, down, certify))
        if targets is not None and (lower is None or upper is None):
            lower, upper = dist - eps, dist + eps
        return self.fc_final(*self.fc_linear((dist, lower, upper)), targets=targets)
