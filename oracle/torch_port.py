"""TEST / BASELINE INFRASTRUCTURE ONLY: the reference's CPU path restated with torch tensor ops.

The reference computes its operators on the CPU (or without its extension) as broadcasts followed by
`torch.norm` (core/norm_dist.py:99-103 for the distance, :112-120 for the interval bounds) and lets
autograd derive the gradients.  This module restates that computation so it can be timed on the host
cores of a box that has no upstream checkout; tests/test_oracle_golden.py checks it against the
committed reference vectors.  The broadcast materialises a (B, G, CO/G, CI/G, HW) tensor, so
`norm_dist_fwd_bwd` walks the output channels in chunks.
"""
import math

import torch


def norm_dist(x, weight, p, groups=1):
    """(B, CI, HW), (CO, CI/G) -> (B, CO, HW); max-normalised p-norm of the broadcast difference."""
    B, HW = x.size(0), x.size(2)
    diff = x.reshape(B, groups, 1, -1, HW) - weight.reshape(groups, -1, weight.size(-1), 1)
    with torch.no_grad():
        scale = diff.abs().amax(dim=3, keepdim=True)
    if math.isinf(p):
        y = (diff / scale).abs().amax(dim=3, keepdim=True) * scale
    else:
        y = torch.linalg.vector_norm(diff / scale, ord=p, dim=3, keepdim=True) * scale
    return y.reshape(B, -1, HW)


def bound_inf_dist(x_lower, x_upper, weight, groups=1):
    B, HW = x_lower.size(0), x_lower.size(2)
    w = weight.reshape(groups, -1, weight.size(-1), 1)
    t1 = w - x_lower.reshape(B, groups, 1, -1, HW)
    t2 = x_upper.reshape(B, groups, 1, -1, HW) - w
    upper = torch.maximum(t1, t2).clamp(min=1e-10).amax(dim=3)
    lower = (-torch.minimum(t1, t2).clamp(max=-1e-10)).amax(dim=3)
    return lower.reshape(B, -1, HW), upper.reshape(B, -1, HW)


def norm_dist_fwd_bwd(x, weight, grad_out, p, chunk=256):
    """Forward plus autograd backward for groups = 1, walking CO in chunks.  Returns (y, grad_x, grad_w)."""
    x = x.detach().requires_grad_()
    ys, gws = [], []
    for c0 in range(0, weight.size(0), chunk):
        wc = weight[c0:c0 + chunk].detach().requires_grad_()
        y = norm_dist(x, wc, p)
        y.backward(grad_out[:, c0:c0 + chunk])
        ys.append(y.detach())
        gws.append(wc.grad)
    return torch.cat(ys, 1), x.grad, torch.cat(gws, 0)
