"""SGD with momentum, Nesterov and L2 weight decay (reference: ``src/optimizers.cpp:156-425``,
``kernel_gen/kernel_gen/kernels/optimizer.py:50-79``)."""
from __future__ import annotations

import torch

from ..utils.nvtx import gputx_range

from .base import Optimizer


class SgdOptimizer(Optimizer):
    def __init__(self, named_params, prefix: str, lr: float, momentum: float = 0.0, nesterov: bool = False,
                 weight_decay: float = 0.0):
        super().__init__(named_params, prefix)
        self.lr, self.momentum, self.nesterov, self.weight_decay = lr, momentum, nesterov, weight_decay
        if momentum != 0.0:
            for name, p in self.named_params:
                self.state[name]["velocity"] = torch.zeros_like(p, dtype=torch.float32)

    def step(self) -> None:
        with gputx_range("fbamtrain::optimizer::sgd_step"):
            return self._step_impl()

    @torch.no_grad()
    def _step_impl(self) -> None:
        self.step_count += 1
        for name, p in self.named_params:
            if p.grad is None:
                continue
            if self._native_step(name, p):
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

    def _native_step(self, name: str, p: torch.Tensor) -> bool:
        """One fused kernel per tensor on a GPU (bf16 / fp16 parameters with an fp32 master, or fp32 parameters)."""
        if not p.is_cuda or p.dtype not in (torch.bfloat16, torch.float16, torch.float32) or p.grad.dtype != p.dtype:
            return False
        from ..ops import dispatch
        if dispatch.get_backend() != "auto" or not p.is_contiguous() or not p.grad.is_contiguous():
            return False
        import ctypes as C
        from ..ops import native as nv
        st = self.state[name]
        master = st.get("master")
        if p.dtype != torch.float32 and master is None:
            return False
        nv.check(nv.lib(p).fbam_sgd(nv.ptr(p.data), nv.ptr(p.grad), nv.ptr(st.get("velocity")), nv.ptr(master),
                                   C.c_longlong(p.numel()), int(p.dtype != torch.float32), C.c_float(self.lr),
                                   C.c_float(self.momentum), int(self.nesterov), C.c_float(self.weight_decay),
                                   nv.stream_ptr()), "fbam_sgd")
        return True
