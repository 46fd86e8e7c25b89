"""Operator API of the reference (core/norm_dist.py:94-121) on the sm_100a kernels.

`norm_dist(input, weight, p, groups=1, use_custom_cuda_func=True, tag=None)` and
`bound_inf_dist(x_lower, x_upper, weight, groups=1, use_custom_cuda_func=True, tag=None)` keep the
reference's signatures, shapes ((B, C, HW) activations, (CO, CI/groups) weight), p dispatch
(inf -> max kernels, p > 0 -> power kernels, otherwise NotImplementedError) and needs_input_grad logic
(core/norm_dist.py:6-51, :54-91).  There is no non-CUDA path: `use_custom_cuda_func=False` raises.
"""
import math

import torch

from . import norm_dist_cuda as _C

__all__ = ["norm_dist", "bound_inf_dist", "NormDistF", "BoundInfDistF"]


class NormDistF(torch.autograd.Function):
    """core/norm_dist.py:6-51.  grad_input is only computed when the input needs it."""

    @staticmethod
    def forward(ctx, x, weight, group, p, need_grad, tag):
        output = torch.empty(x.size(0), weight.size(0), x.size(2), device=x.device, dtype=torch.float32)
        assert weight.size(1) * group == x.size(1)
        ctx.group = group
        ctx.p = p
        ctx.tag = tag
        if math.isinf(p):
            if not need_grad:
                _C.inf_dist_forward_nograd(x, weight, output, group)
            else:
                pos = torch.empty_like(output, dtype=torch.int)
                _C.inf_dist_forward(x, weight, output, pos, group)
                ctx.save_for_backward(x, weight, pos)
        elif p > 0:
            _C.norm_dist_forward(x, weight, output, group, p)
            ctx.save_for_backward(x, weight, output)
        else:
            raise NotImplementedError
        return output

    @staticmethod
    def backward(ctx, grad_output):
        grad_input = grad_weight = None
        grad_output = grad_output.contiguous()
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if math.isinf(ctx.p):
            x, weight, pos = ctx.saved_tensors
            if need_x:
                grad_input = torch.empty_like(x)
            if need_w:
                grad_weight = torch.empty_like(weight)
                _C.inf_dist_backward_input_weight(grad_output, pos, grad_input, grad_weight, ctx.group)
            elif need_x:
                _C.inf_dist_backward_input(grad_output, pos, grad_input, ctx.group)
        else:
            x, weight, output = ctx.saved_tensors
            if need_x:
                grad_input = torch.empty_like(x)
            if need_w:
                grad_weight = torch.empty_like(weight)
                _C.norm_dist_backward_input_weight(grad_output, x, weight, output, grad_input, grad_weight,
                                                   ctx.group, ctx.p)
            elif need_x:
                _C.norm_dist_backward_input(grad_output, x, weight, output, grad_input, ctx.group, ctx.p)
        return grad_input, grad_weight, None, None, None, None


class BoundInfDistF(torch.autograd.Function):
    """core/norm_dist.py:54-91."""

    @staticmethod
    def forward(ctx, x_lower, x_upper, weight, group, need_grad, tag):
        assert x_lower.size() == x_upper.size()
        assert weight.size(1) * group == x_lower.size(1)
        y_lower = torch.empty(x_lower.size(0), weight.size(0), x_lower.size(2), device=x_lower.device,
                              dtype=torch.float32)
        y_upper = torch.empty_like(y_lower)
        ctx.group = group
        ctx.tag = tag
        if not need_grad:
            _C.bound_inf_dist_forward_nograd(x_lower, x_upper, weight, y_lower, y_upper, group)
        else:
            pos_lower = torch.empty_like(y_lower, dtype=torch.int)
            pos_upper = torch.empty_like(pos_lower)
            _C.bound_inf_dist_forward(x_lower, x_upper, weight, y_lower, y_upper, pos_lower, pos_upper, group)
            ctx.save_for_backward(x_lower, x_upper, weight, pos_lower, pos_upper)
        return y_lower, y_upper

    @staticmethod
    def backward(ctx, grad_y_lower, grad_y_upper):
        grad_weight = None
        grad_y_lower = grad_y_lower.contiguous()
        grad_y_upper = grad_y_upper.contiguous()
        x_lower, x_upper, weight, pos_lower, pos_upper = ctx.saved_tensors
        # the kernels zero-fill what they accumulate into; zeros are only needed for the untouched case
        if ctx.needs_input_grad[2]:
            grad_x_lower = torch.empty_like(x_lower)
            grad_x_upper = torch.empty_like(x_upper)
            grad_weight = torch.empty_like(weight)
            _C.bound_inf_dist_backward_input_weight(grad_y_lower, grad_y_upper, pos_lower, pos_upper,
                                                    grad_x_lower, grad_x_upper, grad_weight, ctx.group)
        elif ctx.needs_input_grad[0] and ctx.needs_input_grad[1]:
            grad_x_lower = torch.empty_like(x_lower)
            grad_x_upper = torch.empty_like(x_upper)
            _C.bound_inf_dist_backward_input(grad_y_lower, grad_y_upper, pos_lower, pos_upper,
                                             grad_x_lower, grad_x_upper, ctx.group)
        else:
            grad_x_lower = torch.zeros_like(x_lower)
            grad_x_upper = torch.zeros_like(x_upper)
        if not ctx.needs_input_grad[0]:
            grad_x_lower = None
        if not ctx.needs_input_grad[1]:
            grad_x_upper = None
        return grad_x_lower, grad_x_upper, grad_weight, None, None, None


def norm_dist(input, weight, p, groups=1, use_custom_cuda_func=True, tag=None):
    if not use_custom_cuda_func:
        raise NotImplementedError("this package has no non-CUDA path (use_custom_cuda_func=False)")
    need_grad = torch.is_grad_enabled() and (input.requires_grad or weight.requires_grad)
    return NormDistF.apply(input, weight, groups, p, need_grad, tag)


def bound_inf_dist(x_lower, x_upper, weight, groups=1, use_custom_cuda_func=True, tag=None):
    if not use_custom_cuda_func:
        raise NotImplementedError("this package has no non-CUDA path (use_custom_cuda_func=False)")
    need_grad = torch.is_grad_enabled() and (x_lower.requires_grad or x_upper.requires_grad or weight.requires_grad)
    return BoundInfDistF.apply(x_lower, x_upper, weight, groups, need_grad, tag)
