"""ctypes binding of libldn_b200.so (the C ABI declared in include/ldn_b200.h).

The library is the only compute path of this package: if it is missing or cannot be loaded the import
fails with instructions, there is no fallback.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libldn_b200.so")

_c_float_p = ctypes.c_void_p
_c_int_p = ctypes.c_void_p
_i = ctypes.c_int
_f = ctypes.c_float
_s = ctypes.c_void_p

# name -> argument types, exactly as declared in include/ldn_b200.h
SIGNATURES = {
    "ldn_norm_dist_forward": [_c_float_p, _c_float_p, _i, _i, _i, _i, _i, _c_float_p, _f, _s],
    "ldn_norm_dist_forward_with_max": [_c_float_p, _c_float_p, _c_float_p, _i, _i, _i, _i, _i, _c_float_p, _f, _s],
    "ldn_norm_dist_backward_input": [_c_float_p] * 4 + [_i] * 5 + [_c_float_p, _f, _s],
    "ldn_norm_dist_backward_input_weight": [_c_float_p] * 4 + [_i] * 5 + [_c_float_p, _c_float_p, _f, _s],
    "ldn_norm_dist_backward_channels": [_c_float_p] * 4 + [_i] * 6 + [_c_float_p, _c_float_p, _f, _i, _s],
    "ldn_inf_dist_forward_nograd": [_c_float_p, _c_float_p] + [_i] * 5 + [_c_float_p, _s],
    "ldn_inf_dist_forward": [_c_float_p, _c_float_p] + [_i] * 5 + [_c_float_p, _c_int_p, _s],
    "ldn_inf_dist_backward_input": [_c_float_p, _c_int_p] + [_i] * 5 + [_c_float_p, _s],
    "ldn_inf_dist_backward_input_weight": [_c_float_p, _c_int_p] + [_i] * 5 + [_c_float_p, _c_float_p, _s],
    "ldn_bound_inf_dist_forward_nograd": [_c_float_p] * 3 + [_i] * 5 + [_c_float_p, _c_float_p, _s],
    "ldn_bound_inf_dist_forward": [_c_float_p] * 3 + [_i] * 5 + [_c_float_p, _c_float_p, _c_int_p, _c_int_p, _s],
    "ldn_bound_inf_dist_backward_input": [_c_float_p, _c_float_p, _c_int_p, _c_int_p] + [_i] * 5 +
                                         [_c_float_p, _c_float_p, _s],
    "ldn_bound_inf_dist_backward_input_weight": [_c_float_p, _c_float_p, _c_int_p, _c_int_p] + [_i] * 5 +
                                                [_c_float_p, _c_float_p, _c_float_p, _s],
    "ldn_inf_dist_forward_nograd_shifted": [_c_float_p, _c_float_p] + [_i] * 5 + [_c_float_p, _c_float_p, _c_float_p, _s],
    "ldn_bound_inf_dist_forward_nograd_shifted": [_c_float_p] * 3 + [_i] * 5 + [_c_float_p] * 4 + [_s],
    "ldn_inf_dist_forward_nograd_noalloc": [_c_float_p, _c_float_p] + [_i] * 5 + [_c_float_p, _s],
    "ldn_mean_shift_rows": [_c_float_p, _i, _i, _c_float_p, _f, _c_float_p, _c_float_p, _s],
    "ldn_adam_update": [_i, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                        _f, _f, _f, _f, _i, _f, _s],
    "ldn_adam_update_device_step": [_i, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                    ctypes.c_void_p, _f, _f, _f, _f, ctypes.c_void_p, _f, _s],
    "ldn_sgd_update": [_i, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                       _f, _f, _f, _f, _i, _i, _f, _s],
    "ldn_check_status": [_s],
    "ldn_noalloc_check_status": [_s],
    "ldn_release_scratch": [],
    "ldn_reserve_scratch": [_s, ctypes.c_ulonglong],
    "ldn_probe_pipe": [_i, _i, _c_float_p, ctypes.c_void_p, _s],
}
OTHER_SYMBOLS = ["ldn_status_string", "ldn_version", "ldn_set_max_ctas", "ldn_kernel_launches", "ldn_set_trace_buffer",
                 "ldn_enable_kernel_timing", "ldn_last_tile_kernel_ms", "ldn_set_fused_scratch_limit", "ldn_set_bound_one_pass_limit"]


class LdnError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def load(path=LIB_PATH):
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python l_inf_dist_net_v2_b200/build.py` "
            "(needs nvcc; there is no CPU or PyTorch fallback for these operators)")
    lib = ctypes.CDLL(path)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int
    lib.ldn_status_string.argtypes = [ctypes.c_int]
    lib.ldn_status_string.restype = ctypes.c_char_p
    lib.ldn_version.argtypes = []
    lib.ldn_version.restype = ctypes.c_char_p
    lib.ldn_set_max_ctas.argtypes = [ctypes.c_int]
    lib.ldn_set_max_ctas.restype = None
    lib.ldn_set_bound_one_pass_limit.argtypes = [ctypes.c_int]
    lib.ldn_set_bound_one_pass_limit.restype = None
    lib.ldn_set_fused_scratch_limit.argtypes = [ctypes.c_ulonglong]
    lib.ldn_set_fused_scratch_limit.restype = None
    lib.ldn_enable_kernel_timing.argtypes = [ctypes.c_int]
    lib.ldn_enable_kernel_timing.restype = None
    lib.ldn_last_tile_kernel_ms.argtypes = []
    lib.ldn_last_tile_kernel_ms.restype = ctypes.c_float
    lib.ldn_set_trace_buffer.argtypes = [ctypes.c_void_p]
    lib.ldn_set_trace_buffer.restype = None
    lib.ldn_kernel_launches.argtypes = []
    lib.ldn_kernel_launches.restype = ctypes.c_ulonglong
    return lib


lib = load()


def check(status, what):
    if status != 0:
        raise LdnError(f"{what} failed with status {status}: {lib.ldn_status_string(status).decode()}")
