"""AdamW with decoupled weight decay and fp32 state.

Update rule of the reference kernel (reference: ``kernel_gen/kernel_gen/kernels/optimizer.py:6-45``,
``src/optimizers.cpp:427-823``): ``p -= lr·wd·p``; ``m = β1·m + (1-β1)·g``; ``v = β2·v + (1-β2)·g²``;
``p -= lr · (m / bc1) / (sqrt(v / bc2) + eps)`` with bias corrections ``bc = 1 - β^step`` computed on
the host per step.

When the parameters live in :class:`~fbamtrain_b200.utils.flat.FlatGroup` buffers the state
(``m``, ``v`` and the fp32 master copy) is flat as well, and on CUDA one kernel launch per group
updates state and master and writes the rounded 16-bit parameter.  ``step(shard=(rank, world))``
restricts the update to this rank's contiguous slice of every group (ZeRO-1).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..utils.nvtx import gputx_range

from ..utils.flat import FlatGroup
from .base import Optimizer


class AdamwOptimizer(Optimizer):
    def __init__(self, named_params, prefix: str, lr: float, beta1: float = 0.9, beta2: float = 0.999,
                 eps: float = 1e-8, weight_decay: float = 0.0, groups: Optional[List[FlatGroup]] = None):
        self.groups = groups
        if groups is None:
            super().__init__(named_params, prefix)
            for name, p in self.named_params:
                self.state[name]["m"] = torch.zeros_like(p, dtype=torch.float32)
                self.state[name]["v"] = torch.zeros_like(p, dtype=torch.float32)
        else:
            self.named_params = [(n, p) for g in groups for n, p in g.named_params]
            self.prefix, self.step_count, self.state = prefix, 0, {}
            self.flat_state = []
            for g in groups:
                fs = {"m": torch.zeros(g.numel, dtype=torch.float32, device=g.device),
                      "v": torch.zeros(g.numel, dtype=torch.float32, device=g.device)}
                if g.dtype in (torch.float16, torch.bfloat16):
                    fs["master"] = g.data.float()
                self.flat_state.append(fs)
                for n, _ in g.named_params:
                    self.state[n] = {k: g.view_of(t, n) for k, t in fs.items()}
        self.lr, self.beta1, self.beta2, self.eps, self.weight_decay = lr, beta1, beta2, eps, weight_decay

    def _update_range(self, w, g, m, v, bc1, bc2):
        w.mul_(1.0 - self.lr * self.weight_decay)
        m.mul_(self.beta1).add_(g, alpha=1.0 - self.beta1)
        v.mul_(self.beta2).addcmul_(g, g, value=1.0 - self.beta2)
        denom = (v / bc2).sqrt_().add_(self.eps)
        w.addcdiv_(m / bc1, denom, value=-self.lr)

    def step(self, shard: Optional[Tuple[int, int]] = None, grad_scale: float = 1.0) -> None:
        with gputx_range("fbamtrain::optimizer::adamw_step"):
            return self._step_impl(shard, grad_scale)

    @torch.no_grad()
    def _step_impl(self, shard: Optional[Tuple[int, int]] = None, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        bc1 = 1.0 - self.beta1 ** self.step_count
        bc2 = 1.0 - self.beta2 ** self.step_count
        if self.groups is None:
            if shard is not None:
                raise ValueError("sharded steps need flat parameter groups")
            for name, p in self.named_params:
                if p.grad is None:
                    continue
                st = self.state[name]
                self._update_range(self._master(name, p), p.grad.float() * grad_scale, st["m"], st["v"], bc1, bc2)
                self._publish(name, p)
            return
        for g, fs in zip(self.groups, self.flat_state):
            lo, hi = 0, g.numel
            if shard is not None:
                rank, world = shard
                per = g.numel // world
                lo, hi = rank * per, (rank + 1) * per
            if g.data.is_cuda:
                from ..ops import dispatch
                if dispatch.get_backend() == "auto" and g.data.dtype in (torch.bfloat16, torch.float16, torch.float32):
                    from ..ops.native_ops import adamw_flat
                    adamw_flat(g.data, g.grad, fs["m"], fs["v"], fs.get("master"), lo, hi, self.lr, self.beta1,
                               self.beta2, self.eps, self.weight_decay, bc1, bc2, grad_scale)
                    continue
            w = fs["master"][lo:hi] if "master" in fs else g.data[lo:hi]
            self._update_range(w, g.grad[lo:hi].float() * grad_scale, fs["m"][lo:hi], fs["v"][lo:hi], bc1, bc2)
            if "master" in fs:
                g.data[lo:hi].copy_(w)

    def load_state_tensors(self, tensors) -> None:
        super().load_state_tensors(tensors)

    def _publish(self, name, p) -> None:
        if "master" in self.state[name]:
            p.data.copy_(self.state[name]["master"])
