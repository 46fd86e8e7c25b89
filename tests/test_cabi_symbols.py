"""CPU checks of the boundary: the library loads, exports every symbol include/ldn_b200.h declares, and the
reference-facing Python layer rejects bad inputs before any launch."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "ldn_b200.h")).read()
    return sorted(set(re.findall(r"LDN_API\s+[\w\s\*]+?\b(ldn_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from l_inf_dist_net_v2_b200 import _lib
    names = _declared()
    assert len(names) >= 17, names
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/ldn_b200.h but not exported"
    # every bound signature is declared
    for n in list(_lib.SIGNATURES) + _lib.OTHER_SYMBOLS:
        assert n in names, n


def test_version_and_status_strings():
    from l_inf_dist_net_v2_b200._lib import lib
    assert b"sm_100a" in lib.ldn_version()
    assert lib.ldn_status_string(0) == b"ok"
    assert b"bad argument" in lib.ldn_status_string(1)


def test_module_exports_the_reference_functions():
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C
    expected = ["norm_dist_forward", "norm_dist_forward_with_max", "norm_dist_backward_input",
                "norm_dist_backward_input_weight", "inf_dist_forward", "inf_dist_forward_nograd",
                "inf_dist_backward_input", "inf_dist_backward_input_weight", "bound_inf_dist_forward",
                "bound_inf_dist_forward_nograd", "bound_inf_dist_backward_input",
                "bound_inf_dist_backward_input_weight"]
    for n in expected:
        assert callable(getattr(C, n))


def test_cpu_tensors_are_rejected_like_the_reference():
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C
    x = torch.rand(2, 4, 1)
    w = torch.randn(3, 4)
    y = torch.empty(2, 3, 1)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        C.norm_dist_forward(x, w, y, 1, 8.0)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        C.inf_dist_forward_nograd(x, w, y, 1)


def test_no_fallback_path():
    import l_inf_dist_net_v2_b200 as m
    with pytest.raises(NotImplementedError):
        m.norm_dist(torch.rand(2, 4, 1), torch.randn(3, 4), 8.0, use_custom_cuda_func=False)
    with pytest.raises(NotImplementedError):
        m.bound_inf_dist(torch.rand(2, 4, 1), torch.rand(2, 4, 1), torch.randn(3, 4), use_custom_cuda_func=False)


def test_module_parameter_names_and_identity_init():
    import l_inf_dist_net_v2_b200 as m
    torch.manual_seed(0)
    layer = m.NormDist(6, 10, bias=False, mean_shift=True, identity_val=10.0, std=1.0)
    assert set(layer.state_dict().keys()) == {"weight", "mean_shift.running_mean"}
    for i in range(10):
        assert layer.weight[i, i % 6].item() == -10.0
    conv = m.NormDistConv(4, 8, 3, padding=1, groups=2, identity_val=5.0)
    assert conv.weight.shape == (8, 2 * 9)
    wv = conv.weight.view(8, 2, 3, 3)
    for i in range(8):
        assert wv[i, i % 2, 1, 1].item() == -5.0


def test_compiled_binding_is_used_when_built():
    import os
    from l_inf_dist_net_v2_b200 import norm_dist_cuda as C
    pkg = os.path.dirname(C.__file__)
    built = any(f.startswith("_norm_dist_ext") and f.endswith(".so") for f in os.listdir(pkg))
    assert C.BINDING == ("pybind11" if built else "ctypes")
