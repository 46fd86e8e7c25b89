"""The 12-function extension-module interface of the reference (`import norm_dist_cuda as _C`,
core/cuda/norm_dist.cpp:191-204), implemented on the C ABI of libldn_b200.so.

Same names, same argument order, same in-place semantics (the caller allocates every output, nothing is
returned) and the same checks: every tensor must be a contiguous CUDA tensor (core/cuda/norm_dist.cpp:8-10)
of dtype float32 (int32 for pos arrays).  Shapes are read from the tensors exactly as the reference
wrappers do (core/cuda/norm_dist.cpp:44,73,127).  Differences: kernels are launched on the current
stream of the tensors' device instead of the legacy default stream, and a failing launch raises
(RuntimeError).
"""
import torch

from ._lib import lib, check

__all__ = [
    "norm_dist_forward", "norm_dist_forward_with_max", "norm_dist_backward_input",
    "norm_dist_backward_input_weight", "inf_dist_forward", "inf_dist_forward_nograd",
    "inf_dist_backward_input", "inf_dist_backward_input_weight", "bound_inf_dist_forward",
    "bound_inf_dist_forward_nograd", "bound_inf_dist_backward_input", "bound_inf_dist_backward_input_weight",
]


def _f(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != torch.float32:
        raise RuntimeError(f"expected scalar type Float but found {t.dtype} for {name}")
    return t.data_ptr()


def _i(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != torch.int32:
        raise RuntimeError(f"expected scalar type Int but found {t.dtype} for {name}")
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def norm_dist_forward(input, weight, output, G, p):
    a, w, y = _f(input, "input"), _f(weight, "weight"), _f(output, "output")
    B, CO, CI, HW = input.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        check(lib.ldn_norm_dist_forward(a, w, B, CO, CI, G, HW, y, p, _stream()), "norm_dist_forward")


def norm_dist_forward_with_max(input, weight, max_output, output, G, p):
    a, w, m, y = _f(input, "input"), _f(weight, "weight"), _f(max_output, "max_output"), _f(output, "output")
    B, CO, CI, HW = input.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        check(lib.ldn_norm_dist_forward_with_max(a, w, m, B, CO, CI, G, HW, y, p, _stream()),
              "norm_dist_forward_with_max")


def norm_dist_backward_input(grad_output, input, weight, output, grad_input, G, p):
    g, a, w, y = _f(grad_output, "grad_output"), _f(input, "input"), _f(weight, "weight"), _f(output, "output")
    gx = _f(grad_input, "grad_input")
    B, CO, CI, HW = grad_output.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        check(lib.ldn_norm_dist_backward_input(g, a, w, y, B, CO, CI, G, HW, gx, p, _stream()),
              "norm_dist_backward_input")


def norm_dist_backward_input_weight(grad_output, input, weight, output, grad_input, grad_weight, G, p):
    """grad_input may be None when the caller does not need it (an extension of the reference interface)."""
    g, a, w, y = _f(grad_output, "grad_output"), _f(input, "input"), _f(weight, "weight"), _f(output, "output")
    gx = None if grad_input is None else _f(grad_input, "grad_input")
    gw = _f(grad_weight, "grad_weight")
    B, CO, CI, HW = grad_output.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        check(lib.ldn_norm_dist_backward_input_weight(g, a, w, y, B, CO, CI, G, HW, gx, gw, p, _stream()),
              "norm_dist_backward_input_weight")


def inf_dist_forward(input, weight, output, pos, G):
    a, w, y, ps = _f(input, "input"), _f(weight, "weight"), _f(output, "output"), _i(pos, "pos")
    B, CO, CI, HW = input.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        check(lib.ldn_inf_dist_forward(a, w, B, CO, CI, G, HW, y, ps, _stream()), "inf_dist_forward")


def inf_dist_forward_nograd(input, weight, output, G):
    a, w, y = _f(input, "input"), _f(weight, "weight"), _f(output, "output")
    B, CO, CI, HW = input.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        check(lib.ldn_inf_dist_forward_nograd(a, w, B, CO, CI, G, HW, y, _stream()), "inf_dist_forward_nograd")


def inf_dist_backward_input(grad_output, pos, grad_input, G):
    g, ps, gx = _f(grad_output, "grad_output"), _i(pos, "pos"), _f(grad_input, "grad_input")
    B, CO, CI, HW = grad_output.size(0), grad_output.size(1), grad_input.size(1), grad_input.size(2)
    with torch.cuda.device(grad_output.device):
        check(lib.ldn_inf_dist_backward_input(g, ps, B, CO, CI, G, HW, gx, _stream()), "inf_dist_backward_input")


def inf_dist_backward_input_weight(grad_output, pos, grad_input, grad_weight, G):
    """grad_input may be None when the caller does not need it (an extension of the reference interface)."""
    g, ps = _f(grad_output, "grad_output"), _i(pos, "pos")
    gx = None if grad_input is None else _f(grad_input, "grad_input")
    gw = _f(grad_weight, "grad_weight")
    B, CO, CI, HW = grad_output.size(0), grad_output.size(1), grad_weight.size(1) * G, grad_output.size(2)
    with torch.cuda.device(grad_output.device):
        check(lib.ldn_inf_dist_backward_input_weight(g, ps, B, CO, CI, G, HW, gx, gw, _stream()),
              "inf_dist_backward_input_weight")


def bound_inf_dist_forward(inputL, inputU, weight, outputL, outputU, posL, posU, G):
    xl, xu, w = _f(inputL, "inputL"), _f(inputU, "inputU"), _f(weight, "weight")
    yl, yu, pl, pu = _f(outputL, "outputL"), _f(outputU, "outputU"), _i(posL, "posL"), _i(posU, "posU")
    B, CO, CI, HW = inputL.size(0), outputL.size(1), inputL.size(1), inputL.size(2)
    with torch.cuda.device(inputL.device):
        check(lib.ldn_bound_inf_dist_forward(xl, xu, w, B, CO, CI, G, HW, yl, yu, pl, pu, _stream()),
              "bound_inf_dist_forward")


def bound_inf_dist_forward_nograd(inputL, inputU, weight, outputL, outputU, G):
    xl, xu, w = _f(inputL, "inputL"), _f(inputU, "inputU"), _f(weight, "weight")
    yl, yu = _f(outputL, "outputL"), _f(outputU, "outputU")
    B, CO, CI, HW = inputL.size(0), outputL.size(1), inputL.size(1), inputL.size(2)
    with torch.cuda.device(inputL.device):
        check(lib.ldn_bound_inf_dist_forward_nograd(xl, xu, w, B, CO, CI, G, HW, yl, yu, _stream()),
              "bound_inf_dist_forward_nograd")


def bound_inf_dist_backward_input(grad_outputL, grad_outputU, posL, posU, grad_inputL, grad_inputU, G):
    gl, gu = _f(grad_outputL, "grad_outputL"), _f(grad_outputU, "grad_outputU")
    pl, pu = _i(posL, "posL"), _i(posU, "posU")
    gxl, gxu = _f(grad_inputL, "grad_inputL"), _f(grad_inputU, "grad_inputU")
    B, CO, CI, HW = grad_outputL.size(0), grad_outputL.size(1), grad_inputL.size(1), grad_inputL.size(2)
    with torch.cuda.device(grad_outputL.device):
        check(lib.ldn_bound_inf_dist_backward_input(gl, gu, pl, pu, B, CO, CI, G, HW, gxl, gxu, _stream()),
              "bound_inf_dist_backward_input")


def bound_inf_dist_backward_input_weight(grad_outputL, grad_outputU, posL, posU, grad_inputL, grad_inputU,
                                         grad_weight, G):
    gl, gu = _f(grad_outputL, "grad_outputL"), _f(grad_outputU, "grad_outputU")
    pl, pu = _i(posL, "posL"), _i(posU, "posU")
    gxl, gxu, gw = _f(grad_inputL, "grad_inputL"), _f(grad_inputU, "grad_inputU"), _f(grad_weight, "grad_weight")
    B, CO, CI, HW = grad_outputL.size(0), grad_outputL.size(1), grad_weight.size(1) * G, grad_outputL.size(2)
    with torch.cuda.device(grad_outputL.device):
        check(lib.ldn_bound_inf_dist_backward_input_weight(gl, gu, pl, pu, B, CO, CI, G, HW, gxl, gxu, gw,
                                                           _stream()),
              "bound_inf_dist_backward_input_weight")


def mean_shift_rows(x, running_mean, momentum, out):
    """Not part of the reference's extension module: out = x - mean over dim 0 of the (B, C) view of x, and, when
    running_mean is given, running_mean <- (1 - momentum) running_mean + momentum mean, in one kernel."""
    a, y = _f(x, "x"), _f(out, "out")
    rm = None if running_mean is None else _f(running_mean, "running_mean")
    B, C = x.size(0), x.numel() // max(x.size(0), 1)
    with torch.cuda.device(x.device):
        check(lib.ldn_mean_shift_rows(a, B, C, rm, float(momentum), y, None, _stream()), "mean_shift_rows")


def norm_dist_backward_channels(grad_output, input, weight, output, grad_input, grad_weight, p, co_begin, co_count,
                                accumulate_input):
    """Not part of the reference's extension module: the finite-p backward pass of an ungrouped layer restricted to the
    output channels [co_begin, co_begin + co_count); see ldn_norm_dist_backward_channels."""
    g, a, w, y = _f(grad_output, "grad_output"), _f(input, "input"), _f(weight, "weight"), _f(output, "output")
    gx, gw = _f(grad_input, "grad_input"), _f(grad_weight, "grad_weight")
    B, CO, CI, HW = grad_output.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        check(lib.ldn_norm_dist_backward_channels(g, a, w, y, B, CO, CI, HW, co_begin, co_count, gx, gw, p,
                                                  int(bool(accumulate_input)), _stream()),
              "norm_dist_backward_channels")


def inf_dist_forward_nograd_shifted(input, weight, output, sub, add, G):
    """Not part of the reference's extension module: inf_dist_forward_nograd with (y - sub[o]) + add[o] applied in the
    store; sub / add are (CO,) tensors or None."""
    a, w, y = _f(input, "input"), _f(weight, "weight"), _f(output, "output")
    sp = None if sub is None else _f(sub, "sub")
    ap = None if add is None else _f(add, "add")
    B, CO, CI, HW = input.size(0), output.size(1), input.size(1), input.size(2)
    with torch.cuda.device(input.device):
        check(lib.ldn_inf_dist_forward_nograd_shifted(a, w, B, CO, CI, G, HW, y, sp, ap, _stream()),
              "inf_dist_forward_nograd_shifted")


def bound_inf_dist_forward_nograd_shifted(inputL, inputU, weight, outputL, outputU, sub, add, G):
    """Not part of the reference's extension module: bound_inf_dist_forward_nograd with the same epilogue on both
    bounds."""
    xl, xu, w = _f(inputL, "inputL"), _f(inputU, "inputU"), _f(weight, "weight")
    yl, yu = _f(outputL, "outputL"), _f(outputU, "outputU")
    sp = None if sub is None else _f(sub, "sub")
    ap = None if add is None else _f(add, "add")
    B, CO, CI, HW = inputL.size(0), outputL.size(1), inputL.size(1), inputL.size(2)
    with torch.cuda.device(inputL.device):
        check(lib.ldn_bound_inf_dist_forward_nograd_shifted(xl, xu, w, B, CO, CI, G, HW, yl, yu, sp, ap, _stream()),
              "bound_inf_dist_forward_nograd_shifted")


def check_status():
    """Waits for the current stream and raises if a kernel reported a bounded-wait timeout."""
    check(lib.ldn_check_status(_stream()), "device status check")


# The compiled pybind11 / PyTorch binding of the same C ABI (csrc/binding/norm_dist_ext.cpp, built in-tree by
# build.py) replaces the ctypes wrappers above when it is present: same names, same checks, less call overhead.
# Both bindings call the same library; neither computes anything itself.
BINDING = "ctypes"
try:
    from . import _norm_dist_ext as _ext
except ImportError:
    _ext = None
if _ext is not None:
    for _name in __all__ + ["check_status"]:
        globals()[_name] = getattr(_ext, _name)
    BINDING = "pybind11"
