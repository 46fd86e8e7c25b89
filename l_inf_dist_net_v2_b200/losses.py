"""Training losses of the reference driver (main.py:304-330), as callables `loss(outputs, worst_outputs, targets)`
on what the models return: `hinge` and `mixture` act on the margins of `MLPModel`, `crossentropy` on the
worst-case logit differences of `HybridModel`."""
import math

import torch.nn.functional as F

__all__ = ["hinge", "crossentropy", "mixture"]


class hinge:
    """(1 - mix) * mean over samples of the largest positive margin + mix * mean of all positive margins."""

    def __init__(self, mix=0.25):
        self.mix = mix

    def __call__(self, outputs, worst_outputs, targets):
        pos = worst_outputs.clamp(min=0)
        return (1 - self.mix) * pos.max(dim=1)[0].mean() + self.mix * pos.mean()


class crossentropy:
    def __init__(self, mix=0):
        self.mix = mix

    def __call__(self, outputs, worst_outputs, targets):
        robust = F.cross_entropy(worst_outputs, targets)
        if self.mix == 0:
            return robust
        return (1 - self.mix) * robust + self.mix * F.cross_entropy(outputs, targets)


class mixture:
    """Clipped hinge on the margins plus lam * cross-entropy on the logits; lam decays geometrically from lam0 to
    lam_end as `update(ratio)` is called with ratio going from 0 to 1."""

    def __init__(self, lam0=0.1, lam_end=0.001, clip=1):
        self.lam_start = lam0
        self.lam_end = lam_end
        self.lam = lam0
        self.speed = math.log(lam_end / lam0)
        self.clip = clip

    def update(self, ratio):
        self.lam = self.lam_start * math.exp(self.speed * ratio)

    def __call__(self, outputs, worst_outputs, targets):
        pos = worst_outputs.clamp(min=0, max=self.clip)
        return pos.max(dim=1)[0].mean() + self.lam * F.cross_entropy(outputs, targets)
