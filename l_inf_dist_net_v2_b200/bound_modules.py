"""Interval-bound layers that follow the distance layers in the reference's hybrid model
(core/modules/basic_modules.py:11-46, :77-101, :138-142): every layer maps the triple (x, lower, upper) to
the triple of its outputs, where [lower, upper] is an elementwise enclosure of the layer's value over the
input enclosure.  Same class names, constructor arguments, parameter names (`weight`, `bias`) and scaling
(`w_scale / sqrt(fan_in)`, `b_scale`) as the reference, so its checkpoints load.

An affine map sends the box with centre c and radius r to the box with centre W c + b and radius |W| r.
The layers work on the doubled centre `lower + upper` and the doubled radius `upper - lower`, so that no
halving happens before the matrix products (this is the arithmetic of the reference, which keeps results
comparable to rounding).  These are small cuBLAS products (512 x 5120 x 512 in the largest benchmark
configuration); the distance kernels of this package are not involved.
"""
import math

import torch
import torch.nn as nn

__all__ = ["BoundSequential", "BoundTanh", "BoundReLU", "BoundLinear", "BoundFinalLinear"]


def _map3(triple, fn):
    return tuple(None if z is None else fn(z) for z in triple)


class BoundSequential(nn.Sequential):
    """Chains layers that take and return (x, lower, upper); called with the triple as one argument."""

    def forward(self, paras):
        for layer in self:
            paras = layer(*paras)
        return paras


class BoundTanh(nn.Tanh):
    """tanh is monotone: the enclosure maps endpoint to endpoint."""

    def forward(self, x=None, lower=None, upper=None):
        return _map3((x, lower, upper), torch.tanh)


class BoundReLU(nn.ReLU):
    def forward(self, x=None, lower=None, upper=None):
        return _map3((x, lower, upper), torch.relu)


def _affine(inp, weight, bias, w_scale, b_scale):
    if bias is None:
        return (inp @ weight.t()) * w_scale
    return torch.addmm(bias, inp, weight.t(), beta=b_scale, alpha=w_scale)


class _ScaledLinear(nn.Linear):
    """nn.Linear with N(0, 1) weights, zero bias and the output scaled by w_scale / sqrt(in_features)."""

    def __init__(self, in_features, out_features, bias=True, w_scale=1.0, b_scale=1.0):
        super().__init__(in_features, out_features, bias=bias)
        with torch.no_grad():
            self.weight.normal_()
            if self.bias is not None:
                self.bias.zero_()
        self.w_scale = w_scale / math.sqrt(in_features)
        self.b_scale = b_scale


class BoundLinear(_ScaledLinear):
    def forward(self, x=None, lower=None, upper=None):
        if x is not None:
            x = _affine(x, self.weight, self.bias, self.w_scale, self.b_scale)
        if lower is not None and upper is not None:
            half = 0.5 * self.w_scale
            centre = _affine(lower + upper, self.weight, self.bias, half, self.b_scale)
            radius = (upper - lower) @ self.weight.abs().t()
            lower = torch.add(centre, radius, alpha=-half)
            upper = torch.add(centre, radius, alpha=half)
        return x, lower, upper


class BoundFinalLinear(_ScaledLinear):
    """Last layer.  With targets it returns (logits, worst) where worst[b, j] is an upper bound of
    logit_j - logit_target(b) over the input enclosure (0 at j = target): the bound is taken on the difference
    of the two weight rows, which is tighter than the difference of the two logits' bounds."""

    def forward(self, x=None, lower=None, upper=None, targets=None):
        if x is not None:
            x = _affine(x, self.weight, self.bias, self.w_scale, self.b_scale)
        if lower is None or upper is None or targets is None:
            return x
        half = 0.5 * self.w_scale
        diff = self.weight.unsqueeze(0) - self.weight[targets].unsqueeze(1)  # (B, classes, features)
        worst = torch.bmm(diff, (lower + upper).unsqueeze(-1)) * half
        if self.bias is not None:
            shift = self.bias.unsqueeze(0) - self.bias[targets].unsqueeze(1)
            worst = torch.add(worst, shift.unsqueeze(-1), alpha=self.b_scale)
        spread = torch.bmm(diff.abs(), (upper - lower).unsqueeze(-1))
        return x, torch.add(worst, spread, alpha=half).squeeze(-1)
