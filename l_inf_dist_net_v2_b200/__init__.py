"""sm_100a (B200) implementation of the L_p-distance operator family of zbh2047/L_inf-dist-net-v2.

Importing this package loads libldn_b200.so (built in-tree by `python l_inf_dist_net_v2_b200/build.py`);
the import fails if the library is missing -- there is no CPU or pure-PyTorch path.
"""
from . import norm_dist_cuda  # noqa: F401  (loads the native library)
from .norm_dist import norm_dist, bound_inf_dist, NormDistF, BoundInfDistF  # noqa: F401
from .modules import NormDistBase, NormDist, NormDistConv, MeanShift, apply_if_not_none  # noqa: F401

from .bound_modules import BoundSequential, BoundTanh, BoundReLU, BoundLinear, BoundFinalLinear  # noqa: F401
from .models import MLPModel, HybridModel, check_inf_and_eval, set_p_norm  # noqa: F401
from .attack import AttackPGD  # noqa: F401
from . import losses  # noqa: F401

__version__ = "0.2"
