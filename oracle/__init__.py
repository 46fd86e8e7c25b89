"""numpy front end of the CPU checker in oracle/ldn_oracle.c.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline leg of
bench.py.  Nothing in the product package imports it.

Every function takes/returns contiguous numpy arrays with the reference's shapes:
x (B, CI, HW), w (CO, CI/G), y (B, CO, HW); 2-D x / y (fully-connected use) are accepted and
treated as HW = 1.
"""
import ctypes

import numpy as np

from .build import build_oracle

_lib = None


def _get():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(build_oracle())
        lib.ldn_oracle_num_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _i(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _dims(x, w, groups):
    x3 = x if x.ndim == 3 else x.reshape(x.shape[0], x.shape[1], 1)
    B, CI, HW = x3.shape
    CO = w.shape[0]
    assert w.shape[1] * groups == CI, "weight.size(1) * groups must equal x.size(1)"
    assert CO % groups == 0
    return B, CO, CI, HW


def _yshape(x, B, CO, HW):
    return (B, CO, HW) if x.ndim == 3 else (B, CO)


def num_threads():
    return int(_get().ldn_oracle_num_threads())


def norm_dist_forward(x, w, p, groups=1):
    x, w = _f(x), _f(w)
    B, CO, CI, HW = _dims(x, w, groups)
    y = np.empty(_yshape(x, B, CO, HW), np.float32)
    _get().ldn_oracle_norm_dist_forward(_p(x), _p(w), _p(y), B, CO, CI, groups, HW, ctypes.c_float(p))
    return y


def norm_dist_forward_with_max(x, w, mx, p, groups=1):
    x, w, mx = _f(x), _f(w), _f(mx)
    B, CO, CI, HW = _dims(x, w, groups)
    y = np.empty(_yshape(x, B, CO, HW), np.float32)
    _get().ldn_oracle_norm_dist_forward_with_max(_p(x), _p(w), _p(mx), _p(y), B, CO, CI, groups, HW,
                                                 ctypes.c_float(p))
    return y


def norm_dist_backward(go, x, w, y, p, groups=1, want_gx=True, want_gw=True):
    go, x, w, y = _f(go), _f(x), _f(w), _f(y)
    B, CO, CI, HW = _dims(x, w, groups)
    gx = np.empty_like(x) if want_gx else None
    gw = np.empty_like(w) if want_gw else None
    _get().ldn_oracle_norm_dist_backward(_p(go), _p(x), _p(w), _p(y), _p(gx), _p(gw),
                                         B, CO, CI, groups, HW, ctypes.c_float(p))
    return gx, gw


def inf_dist_forward(x, w, groups=1, want_pos=True):
    x, w = _f(x), _f(w)
    B, CO, CI, HW = _dims(x, w, groups)
    y = np.empty(_yshape(x, B, CO, HW), np.float32)
    pos = np.empty(y.shape, np.int32) if want_pos else None
    _get().ldn_oracle_inf_dist_forward(_p(x), _p(w), _p(y), _p(pos), B, CO, CI, groups, HW)
    return y, pos


def inf_dist_backward(go, pos, x_shape, w_shape, groups=1, want_gw=True):
    go, pos = _f(go), _i(pos)
    B, CI = x_shape[0], x_shape[1]
    HW = x_shape[2] if len(x_shape) == 3 else 1
    CO = w_shape[0]
    gx = np.empty(x_shape, np.float32)
    gw = np.empty(w_shape, np.float32) if want_gw else None
    _get().ldn_oracle_inf_dist_backward(_p(go), _p(pos), _p(gx), _p(gw), B, CO, CI, groups, HW)
    return gx, gw


def bound_inf_dist_forward(xL, xU, w, groups=1, want_pos=True):
    xL, xU, w = _f(xL), _f(xU), _f(w)
    B, CO, CI, HW = _dims(xL, w, groups)
    yL = np.empty(_yshape(xL, B, CO, HW), np.float32)
    yU = np.empty_like(yL)
    pL = np.empty(yL.shape, np.int32) if want_pos else None
    pU = np.empty(yL.shape, np.int32) if want_pos else None
    _get().ldn_oracle_bound_inf_dist_forward(_p(xL), _p(xU), _p(w), _p(yL), _p(yU), _p(pL), _p(pU),
                                             B, CO, CI, groups, HW)
    return yL, yU, pL, pU


def bound_inf_dist_backward(goL, goU, posL, posU, x_shape, w_shape, groups=1, want_gw=True):
    goL, goU, posL, posU = _f(goL), _f(goU), _i(posL), _i(posU)
    B, CI = x_shape[0], x_shape[1]
    HW = x_shape[2] if len(x_shape) == 3 else 1
    CO = w_shape[0]
    gxL = np.empty(x_shape, np.float32)
    gxU = np.empty(x_shape, np.float32)
    gw = np.empty(w_shape, np.float32) if want_gw else None
    _get().ldn_oracle_bound_inf_dist_backward(_p(goL), _p(goU), _p(posL), _p(posU),
                                              _p(gxL), _p(gxU), _p(gw), B, CO, CI, groups, HW)
    return gxL, gxU, gw
