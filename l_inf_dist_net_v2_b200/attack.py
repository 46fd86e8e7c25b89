"""Projected-gradient l_inf attack with the reference's interface (attack.py:4-36): `AttackPGD(net, eps, step_size,
num_steps, up, down, random_start=True).find(inputs, targets)` returns perturbed inputs inside the eps-ball
around `inputs`, clipped to [down, up].  The weights are frozen while it runs, so the distance layers take the
grad_input-only kernels (norm_dist_backward_input / inf_dist_backward_input).
"""
import torch
import torch.nn.functional as F

__all__ = ["AttackPGD"]


class AttackPGD:
    def __init__(self, net, eps, step_size, num_steps, up, down, random_start=True):
        self.net = net
        self.eps = eps
        self.step_size = step_size
        self.num_steps = num_steps
        self.up = up
        self.down = down
        self.rand = random_start

    def _project(self, x, centre=None):
        if centre is not None:
            x = torch.minimum(torch.maximum(x, centre - self.eps), centre + self.eps)
        return torch.minimum(torch.maximum(x, self.down), self.up)

    def find(self, inputs, targets):
        params = list(self.net.parameters())
        was = [q.requires_grad for q in params]
        for q in params:
            q.requires_grad_(False)
        try:
            x = inputs.detach()
            if self.rand:
                # N(0, eps / 4) noise clipped to half the radius, as in the reference
                noise = torch.empty_like(x).normal_(0, self.eps / 4).clamp_(-self.eps / 2, self.eps / 2)
                x = self._project(x + noise)
            for _ in range(self.num_steps):
                x = x.detach().requires_grad_()
                loss = F.cross_entropy(self.net(x), targets, reduction="sum")
                grad, = torch.autograd.grad(loss, x)
                x = self._project(torch.add(x.detach(), grad.sign(), alpha=self.step_size), inputs)
        finally:
            for q, r in zip(params, was):
                q.requires_grad_(r)
        return x.detach()
