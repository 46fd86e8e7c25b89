"""Module wrappers with the reference's constructor signatures, parameter names and forward contract
(core/modules/norm_dist.py:13-110): every layer takes and returns the triple (x, lower, upper) of
(B, C, H*W) tensors.  `MeanShift` restates core/modules/basic_modules.py:104-135 because NormDistBase
owns one (parameter / buffer names match, so reference checkpoints load).
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import norm_dist_cuda as _C
from .norm_dist import norm_dist, bound_inf_dist

__all__ = ["NormDistBase", "NormDist", "NormDistConv", "MeanShift", "apply_if_not_none"]


def apply_if_not_none(paras, func):
    return [None if x is None else func(x) for x in paras]


class _MeanShiftRowsF(torch.autograd.Function):
    """x - (mean of x over the batch) for (B, C, 1) inputs, with the running-mean update, as one kernel per pass.
    d(out)/d(x) = I - (1/B) 1 1^T, so the backward pass is the same kernel on the incoming gradient."""

    @staticmethod
    def forward(ctx, x, running_mean, momentum):
        out = torch.empty_like(x)
        _C.mean_shift_rows(x, running_mean, momentum, out)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        grad_output = grad_output.contiguous()
        grad_input = torch.empty_like(grad_output)
        _C.mean_shift_rows(grad_output, None, 0.0, grad_input)
        return grad_input, None, None


class MeanShift(nn.Module):
    """Subtracts the per-channel batch mean (training; running mean updated with `momentum`) or the running
    mean (eval) from x and from both bounds."""

    def __init__(self, out_channels, momentum=0.1, affine=True):
        super().__init__()
        self.out_channels = out_channels
        self.momentum = momentum
        self.affine = affine
        self.fused = True  # use the one-kernel path where it applies (set False for the torch operators)
        self.register_buffer("running_mean", torch.zeros(out_channels))
        if affine:
            self.bias = nn.Parameter(torch.zeros(out_channels))
        else:
            self.register_parameter("bias", None)
        if not hasattr(MeanShift, "tag"):
            MeanShift.tag = 0
        MeanShift.tag += 1
        self.tag = MeanShift.tag

    def forward(self, x=None, lower=None, upper=None):
        if self.training:
            assert x is not None, "Currently not supported"
            if (lower is None and upper is None and self.bias is None and x.is_cuda and x.dtype == torch.float32
                    and x.dim() == 3 and x.size(2) == 1 and x.is_contiguous() and self.fused):
                # fully connected layer: mean, running-mean update and subtraction in one kernel
                return _MeanShiftRowsF.apply(x, self.running_mean, self.momentum), None, None
            mean = x.mean(dim=[0, 2])
            with torch.no_grad():
                self.running_mean.mul_(1 - self.momentum).add_(mean, alpha=self.momentum)
        else:
            mean = self.running_mean
        if self.bias is not None:
            mean = mean - self.bias
        x, lower, upper = apply_if_not_none((x, lower, upper), lambda z: z - mean.unsqueeze(-1))
        return x, lower, upper

    def extra_repr(self):
        return "{out_channels}, affine={affine}".format(**self.__dict__)


class NormDistBase(nn.Module):
    def __init__(self, in_features, out_features, p=float("inf"), groups=1, bias=True, std=1.0, mean_shift=True):
        super().__init__()
        assert in_features % groups == 0
        assert out_features % groups == 0
        self.weight = nn.Parameter(torch.randn(out_features, in_features // groups) * std)
        self.groups = groups
        self.p = p
        self.mean_shift = MeanShift(out_channels=out_features, affine=False) if mean_shift else None
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.fused_eval = True  # eval-mode p = inf layers run as one kernel per tensor (False: the separate steps)
        if not hasattr(NormDistBase, "tag"):
            NormDistBase.tag = 0
        NormDistBase.tag += 1
        self.tag = NormDistBase.tag

    def _eval_layer_fused(self, x, lower, upper):
        """Eval mode, p = inf, nothing needs a gradient: distance (and bounds), running-mean subtraction and bias as
        one kernel each -- the same values, bit for bit, as the separate steps below."""
        sub = self.mean_shift.running_mean if self.mean_shift is not None else None
        if self.mean_shift is not None and self.mean_shift.bias is not None:
            sub = sub - self.mean_shift.bias
        add = self.bias
        out = [None, None, None]
        if x is not None:
            out[0] = torch.empty(x.size(0), self.weight.size(0), x.size(2), device=x.device, dtype=torch.float32)
            _C.inf_dist_forward_nograd_shifted(x, self.weight, out[0], sub, add, self.groups)
        if lower is not None and upper is not None:
            out[1] = torch.empty(lower.size(0), self.weight.size(0), lower.size(2), device=lower.device,
                                 dtype=torch.float32)
            out[2] = torch.empty_like(out[1])
            _C.bound_inf_dist_forward_nograd_shifted(lower, upper, self.weight, out[1], out[2], sub, add, self.groups)
        return out

    def _can_fuse_eval(self, x, lower, upper):
        if self.training or not self.fused_eval or not math.isinf(self.p):
            return False
        tensors = [t for t in (x, lower, upper) if t is not None]
        if (lower is None) != (upper is None) or not tensors:
            return False
        grad = torch.is_grad_enabled() and (self.weight.requires_grad or any(t.requires_grad for t in tensors))
        return not grad and all(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.dim() == 3
                                for t in tensors)

    # x, lower and upper are 3-D tensors of shape (B, C, H*W)
    def forward(self, x=None, lower=None, upper=None):
        if self._can_fuse_eval(x, lower, upper):
            return self._eval_layer_fused(x, lower, upper)
        if x is not None:
            x = norm_dist(x, self.weight, self.p, self.groups, tag=self.tag)
        if lower is not None and upper is not None:
            assert math.isinf(self.p)
            lower, upper = bound_inf_dist(lower, upper, self.weight, self.groups, tag=self.tag)
        if self.mean_shift is not None:
            x, lower, upper = self.mean_shift(x, lower, upper)
        if self.bias is not None:
            x, lower, upper = apply_if_not_none((x, lower, upper), lambda z: z + self.bias.view(1, -1, 1))
        return x, lower, upper


class NormDist(NormDistBase):
    def __init__(self, in_features, out_features, groups=1, bias=True, identity_val=None, **kwargs):
        super().__init__(in_features, out_features, groups=groups, bias=bias, **kwargs)
        self.in_features = in_features
        self.out_features = out_features
        if identity_val is not None and in_features <= out_features:
            with torch.no_grad():
                rows = torch.arange(out_features)
                self.weight[rows, rows % (in_features // groups)] = -identity_val

    def forward(self, x=None, lower=None, upper=None):
        x, lower, upper = apply_if_not_none((x, lower, upper), lambda z: z.unsqueeze(-1))
        x, lower, upper = super().forward(x, lower, upper)
        x, lower, upper = apply_if_not_none((x, lower, upper), lambda z: z.squeeze(-1))
        return x, lower, upper

    def extra_repr(self):
        s = "in_features={}, out_features={}, bias={}"
        if self.groups != 1:
            s += ", groups={groups}"
        return s.format(self.in_features, self.out_features, self.bias is not None, groups=self.groups)


class NormDistConv(NormDistBase):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, identity_val=None, **kwargs):
        if isinstance(kernel_size, int):
            kernel_size = (kernel_size, kernel_size)
        in_features = in_channels * kernel_size[0] * kernel_size[1]
        assert in_channels % groups == 0
        super().__init__(in_features, out_channels, groups=groups, bias=bias, **kwargs)
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = kernel_size
        self.stride = stride
        self.padding = padding
        self.dilation = dilation
        if identity_val is not None and in_channels <= out_channels:
            with torch.no_grad():
                weight = self.weight.view(out_channels, -1, *kernel_size)
                rows = torch.arange(out_channels)
                weight[rows, rows % (in_channels // groups), kernel_size[0] // 2, kernel_size[1] // 2] = -identity_val

    def forward(self, x=None, lower=None, upper=None):
        unfold_paras = self.kernel_size, self.dilation, self.padding, self.stride
        h, w = 0, 0
        if x is not None:
            h, w = x.size(2), x.size(3)
            x = F.unfold(x, *unfold_paras)
        if lower is not None and upper is not None:
            h, w = lower.size(2), lower.size(3)
            lower = F.unfold(lower, *unfold_paras)
            upper = F.unfold(upper, *unfold_paras)
        x, lower, upper = super().forward(x, lower, upper)
        # as in the reference, the output size ignores dilation
        h, w = [(s + 2 * self.padding - k) // self.stride + 1 for s, k in zip((h, w), self.kernel_size)]
        x, lower, upper = apply_if_not_none((x, lower, upper), lambda z: z.view(z.size(0), -1, h, w))
        return x, lower, upper

    def extra_repr(self):
        s = "{in_channels}, {out_channels}, kernel_size={kernel_size}, stride={stride}"
        if self.padding != 0:
            s += ", padding={padding}"
        if self.dilation != 1:
            s += ", dilation={dilation}"
        if self.groups != 1:
            s += ", groups={groups}"
        if self.bias is None:
            s += ", bias=False"
        return s.format(**self.__dict__)
