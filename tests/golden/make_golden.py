"""Generate tests/golden/ref_fallback.npz from the upstream reference's own pure-torch path.

Run once in a container that has the upstream checkout; its location must be given in the environment
variable LDN_REFERENCE_ROOT:   LDN_REFERENCE_ROOT=/path/to/L_inf-dist-net-v2 python tests/golden/make_golden.py

What it records, per case, are the inputs and the outputs of the reference functions
`core.norm_dist.norm_dist(..., use_custom_cuda_func=False)` and
`core.norm_dist.bound_inf_dist(..., use_custom_cuda_func=False)` and of torch autograd through
them.  The reference module imports its CUDA extension unconditionally, so an empty stand-in
module named `norm_dist_cuda` is registered first; no reference CUDA code runs here.

Finite p: outputs and gradients are computed in float64 (the fallback is dtype agnostic) from the
float32 inputs, so they are the exact targets the tolerance checks refer to (gradients are stored
rounded to float32 to keep the fixture small).
p = inf and bounds: outputs in float32 (only subtract / max are involved, so they are bit-exact
targets).  The argmax index array is not produced by the fallback; it is derived here from the
same difference tensor the fallback forms (index of the maximum of |x - w| and the sign of x - w
there) on inputs without ties.
"""
import math
import os
import sys
import types

import numpy as np
import torch

REF = os.environ.get("LDN_REFERENCE_ROOT")
if not REF or not os.path.isdir(os.path.join(REF, "core")):
    sys.exit("set LDN_REFERENCE_ROOT to the upstream checkout")
sys.modules.setdefault("norm_dist_cuda", types.ModuleType("norm_dist_cuda"))
sys.path.insert(0, REF)
from core.norm_dist import norm_dist, bound_inf_dist  # noqa: E402

# (B, CI, CO, G, HW)
SHAPES = [
    (5, 12, 8, 2, 3),
    (3, 17, 10, 1, 1),
    (7, 32, 33, 1, 1),
    (4, 24, 12, 4, 5),
    (9, 40, 6, 2, 1),
    (2, 64, 130, 1, 7),
]
POWERS = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0, 9.0, 2.5, 10.0, 10.5, 37.5, 100.0]


def main():
    out = {}
    gen = torch.Generator().manual_seed(0)
    cases = []
    for si, (B, CI, CO, G, HW) in enumerate(SHAPES):
        x = torch.rand(B, CI, HW, generator=gen)
        w = torch.randn(CO, CI // G, generator=gen)
        g = torch.randn(B, CO, HW, generator=gen)
        g2 = torch.randn(B, CO, HW, generator=gen)
        eps = 8.0 / 255.0
        xL = (x - eps).clamp(0, 1)
        xU = (x + eps).clamp(0, 1)
        key = f"s{si}"
        cases.append(key)
        out[f"{key}/dims"] = np.array([B, CI, CO, G, HW], np.int64)
        for name, t in (("x", x), ("w", w), ("g", g), ("g2", g2), ("xL", xL), ("xU", xU)):
            out[f"{key}/{name}"] = t.numpy()
        # finite p, float64 targets
        for p in POWERS:
            xd = x.double().requires_grad_()
            wd = w.double().requires_grad_()
            y = norm_dist(xd, wd, p, G, use_custom_cuda_func=False)
            y.backward(g.double())
            out[f"{key}/p{p}/y"] = y.detach().numpy()
            out[f"{key}/p{p}/gx"] = xd.grad.numpy().astype(np.float32)
            out[f"{key}/p{p}/gw"] = wd.grad.numpy().astype(np.float32)
        # p = inf, float32 bit-exact value + gradient through the fallback
        xf = x.clone().requires_grad_()
        wf = w.clone().requires_grad_()
        y = norm_dist(xf, wf, math.inf, G, use_custom_cuda_func=False)
        y.backward(g)
        out[f"{key}/inf/y"] = y.detach().numpy()
        out[f"{key}/inf/gx"] = xf.grad.numpy()
        out[f"{key}/inf/gw"] = wf.grad.numpy()
        diff = x.view(B, G, 1, -1, HW) - w.view(G, -1, w.size(-1), 1)  # same tensor the fallback forms
        idx = diff.abs().argmax(dim=3, keepdim=True)
        sign = torch.gather(diff, 3, idx) < 0
        pos = (idx.int() | (sign.int() << 31)).view(B, CO, HW)
        out[f"{key}/inf/pos"] = pos.numpy().astype(np.int32)
        # bounds, float32 bit-exact values + gradients through the fallback
        lf = xL.clone().requires_grad_()
        uf = xU.clone().requires_grad_()
        wf = w.clone().requires_grad_()
        yL, yU = bound_inf_dist(lf, uf, wf, G, use_custom_cuda_func=False)
        (yL * g).sum().backward(retain_graph=True)
        out[f"{key}/bound/yL"] = yL.detach().numpy()
        out[f"{key}/bound/yU"] = yU.detach().numpy()
        out[f"{key}/bound/L_gxL"] = lf.grad.numpy().copy()
        out[f"{key}/bound/L_gxU"] = uf.grad.numpy().copy()
        out[f"{key}/bound/L_gw"] = wf.grad.numpy().copy()
        lf.grad = None
        uf.grad = None
        wf.grad = None
        (yU * g2).sum().backward()
        out[f"{key}/bound/U_gxL"] = lf.grad.numpy().copy()
        out[f"{key}/bound/U_gxU"] = uf.grad.numpy().copy()
        out[f"{key}/bound/U_gw"] = wf.grad.numpy().copy()
    out["cases"] = np.array(cases)
    out["powers"] = np.array(POWERS, np.float64)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_fallback.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
