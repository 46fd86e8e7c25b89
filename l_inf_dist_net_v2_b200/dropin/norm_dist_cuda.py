"""Drop-in module: put this directory on sys.path (before any installed `norm_dist_cuda`) and the
reference's `core/norm_dist.py` (`import norm_dist_cuda as _C`) runs on the sm_100a kernels unchanged."""
from l_inf_dist_net_v2_b200.norm_dist_cuda import *  # noqa: F401,F403
from l_inf_dist_net_v2_b200.norm_dist_cuda import check_status  # noqa: F401
