"""SGD with momentum, Nesterov and L2 weight decay (reference: ``src/optimizers.cpp:156-425``,
``kernel_gen/kernel_gen/kernels/optimizer.py:50-79``)."""
from __future__ import annotations

import torch

from .base import Optimizer


class SgdOptimizer(Optimizer):
    def __init__(self, named_params, prefix: str, lr: float, momentum: float = 0.0, nesterov: bool = False,
                 weight_decay: float = 0.0):
        super().__init__(named_params, prefix)
        self.lr, self.momentum, self.nesterov, self.weight_decay = lr, momentum, nesterov, weight_decay
        if momentum != 0.0:
            for name, p in self.named_params:
                self.state[name]["velocity"] = torch.zeros_like(p, dtype=torch.float32)

    @torch.no_grad()
    def step(self) -> None:
        self.step_count += 1
        for name, p in self.named_params:
            if p.grad is None:
                continue
            w = self._master(name, p)
            g = p.grad.float()
            if self.weight_decay != 0.0:
                g = g + self.weight_decay * w
            if self.momentum != 0.0:
                v = self.state[name]["velocity"]
                v.mul_(self.momentum).add_(g)
                g = g + self.momentum * v if self.nesterov else v
            w.add_(g, alpha=-self.lr)
            self._publish(name, p)
