"""Optimisers whose update is one kernel over all tensors of a step (csrc/ldn_optim.cu), with torch.optim's
update rules and state layout (`exp_avg` / `exp_avg_sq` / `step`, `momentum_buffer`), so that their state_dict
is interchangeable with torch.optim.Adam / torch.optim.SGD.  The reference trains with
Adam(betas=(0.9, 0.99), eps=1e-10) (main.py:388-392).

`step(params=None)` updates only the given parameters when a list is passed: the data-parallel wrapper
(parallel.OverlappedDataParallel) applies each layer's update just before that layer's next forward pass.
"""
import ctypes

import torch

from ._lib import lib, check

__all__ = ["FusedAdam", "FusedSGD"]


def _ptr_array(tensors):
    return (ctypes.c_void_p * len(tensors))(*[None if t is None else t.data_ptr() for t in tensors])


def _check_tensor(t, what):
    if not (t.is_cuda and t.is_contiguous() and t.dtype == torch.float32):
        raise RuntimeError(f"{what} must be a contiguous float32 CUDA tensor")


class _Fused(torch.optim.Optimizer):
    def _select(self, group, params):
        chosen = []
        for q in group["params"]:
            if q.grad is None:
                continue
            if params is not None and not any(q is r for r in params):
                continue
            _check_tensor(q, "parameter")
            if q.grad.is_sparse:
                raise RuntimeError("sparse gradients are not supported")
            g = q.grad if q.grad.is_contiguous() else q.grad.contiguous()
            _check_tensor(g, "gradient")
            chosen.append((q, g))
        return chosen


class FusedAdam(_Fused):
    """capturable=True keeps the step count in a float tensor on the device (as torch.optim.Adam(capturable=True)
    does), advanced by a tensor operation and read by the update kernel, so that `step()` can be recorded in a CUDA
    graph; run at least one step before capturing (it creates the state)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, grad_scale=1.0, capturable=False):
        if lr < 0 or eps < 0 or not (0 <= betas[0] < 1) or not (0 <= betas[1] < 1):
            raise ValueError("invalid Adam hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, grad_scale=grad_scale, capturable=capturable))

    def _step_capturable(self, group, params):
        by_dev = {}
        for q, g in self._select(group, params):
            st = self.state[q]
            if not st:
                st["step"] = torch.zeros((), dtype=torch.float32, device=q.device)
                st["exp_avg"] = torch.zeros_like(q, memory_format=torch.preserve_format)
                st["exp_avg_sq"] = torch.zeros_like(q, memory_format=torch.preserve_format)
            by_dev.setdefault(q.device, []).append((q, g, st))
        for device, items in by_dev.items():
            # one counter per launch: the tensors updated together share the first one's step tensor
            steps = [st["step"] for _, _, st in items]
            torch._foreach_add_(steps, 1.0)
            ps = [q for q, _, _ in items]
            with torch.cuda.device(device):
                check(lib.ldn_adam_update_device_step(
                    len(items), _ptr_array(ps), _ptr_array([g for _, g, _ in items]),
                    _ptr_array([st["exp_avg"] for _, _, st in items]),
                    _ptr_array([st["exp_avg_sq"] for _, _, st in items]),
                    (ctypes.c_longlong * len(items))(*[q.numel() for q in ps]),
                    group["lr"], group["betas"][0], group["betas"][1], group["eps"], steps[0].data_ptr(),
                    group["grad_scale"], torch.cuda.current_stream().cuda_stream), "adam update")

    @torch.no_grad()
    def step(self, params=None):
        for group in self.param_groups:
            if group.get("capturable"):
                self._step_capturable(group, params)
                continue
            by_step = {}
            for q, g in self._select(group, params):
                st = self.state[q]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(q, memory_format=torch.preserve_format)
                    st["exp_avg_sq"] = torch.zeros_like(q, memory_format=torch.preserve_format)
                st["step"] = int(st["step"]) + 1
                by_step.setdefault((st["step"], q.device), []).append((q, g, st))
            for (step, device), items in by_step.items():
                ps = [q for q, _, _ in items]
                with torch.cuda.device(device):
                    check(lib.ldn_adam_update(
                        len(items), _ptr_array(ps), _ptr_array([g for _, g, _ in items]),
                        _ptr_array([st["exp_avg"] for _, _, st in items]),
                        _ptr_array([st["exp_avg_sq"] for _, _, st in items]),
                        (ctypes.c_longlong * len(items))(*[q.numel() for q in ps]),
                        group["lr"], group["betas"][0], group["betas"][1], group["eps"], step, group["grad_scale"],
                        torch.cuda.current_stream().cuda_stream), "adam update")


class FusedSGD(_Fused):
    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, grad_scale=1.0):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov, grad_scale=grad_scale))

    @torch.no_grad()
    def step(self, params=None):
        for group in self.param_groups:
            fresh, warm = [], []
            for q, g in self._select(group, params):
                buf = None
                first = False
                if group["momentum"] != 0:
                    st = self.state[q]
                    first = "momentum_buffer" not in st
                    if first:
                        st["momentum_buffer"] = torch.empty_like(q, memory_format=torch.preserve_format)
                    buf = st["momentum_buffer"]
                (fresh if first else warm).append((q, g, buf))
            for first, items in ((1, fresh), (0, warm)):
                by_dev = {}
                for it in items:
                    by_dev.setdefault(it[0].device, []).append(it)
                for device, its in by_dev.items():
                    ps = [q for q, _, _ in its]
                    with torch.cuda.device(device):
                        check(lib.ldn_sgd_update(
                            len(its), _ptr_array(ps), _ptr_array([g for _, g, _ in its]),
                            _ptr_array([b for _, _, b in its]),
                            (ctypes.c_longlong * len(its))(*[q.numel() for q in ps]),
                            group["lr"], group["momentum"], group["dampening"], group["weight_decay"],
                            int(group["nesterov"]), first, group["grad_scale"],
                            torch.cuda.current_stream().cuda_stream), "sgd update")
