"""Muon: momentum, Newton–Schulz orthogonalisation of the 2-D update, decoupled weight decay.

Algorithm of the reference (reference: ``src/optimizers.cpp:825-1434``; NS loop ``1320-1367``;
orientation rule ``941-968``; scale ``1044-1054``):

1. the momentum buffer is an exponential moving average, ``buf = μ·buf + (1 − μ)·g`` (``1204-1226``); the update
   is ``(1 − μ)·g + μ·buf`` (the reference's only form; ``nesterov = false`` here takes ``buf`` itself);
2. cast to bf16, divide by ``(‖·‖_F + 1e-7)``;
3. five iterations of ``A = X Xᵀ; B = b·A + c·A A; X = a·X + B X`` with
   ``(a, b, c) = (3.4445, -4.7750, 2.0315)``, run on the orientation with rows ≤ cols;
4. scale by ``sqrt(max(1, rows / cols))`` of the *logical* (``out x in``) orientation;
5. ``p ← p·(1 - lr·wd) - lr·U`` on the fp32 master copy.

Parameters with more than two dimensions (conv weights) are flattened to ``(out, rest)``.
``MuonWithAuxAdam`` sends tensors with ``ndim >= 2`` to Muon and the rest (gains, biases, initial
states) to AdamW, with state name prefixes ``/muon`` and ``/adam`` (reference:
``src/optimizers.cpp:1436-1514``).  ``adam_names`` can force additional parameters — embeddings and the
LM head in the large configurations — onto AdamW.
"""
from __future__ import annotations

from typing import Callable, Iterable, Optional, Tuple

import torch

from ..utils.nvtx import gputx_range

from .adamw import AdamwOptimizer
from .base import Optimizer

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(g: torch.Tensor, steps: int = 5, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Approximate ``U Vᵀ`` of the 2-D matrix ``g``; returns ``dtype``."""
    a, b, c = NS_COEFFS
    x = g.to(dtype)
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t()
    x = x / (x.float().norm() + 1e-7).to(dtype)
    for _ in range(steps):
        aa = x @ x.t()
        bb = b * aa + c * (aa @ aa)
        x = a * x + bb @ x
    return x.t() if transposed else x


def muon_update(grad2d: torch.Tensor, momentum_buf: torch.Tensor, momentum: float, nesterov: bool,
                ns_steps: int = 5, ns: Callable = newton_schulz) -> torch.Tensor:
    momentum_buf.mul_(momentum).add_(grad2d, alpha=1.0 - momentum)
    upd = (1.0 - momentum) * grad2d + momentum * momentum_buf if nesterov else momentum_buf
    u = ns(upd, ns_steps).float()
    rows, cols = grad2d.shape
    return u * max(1.0, rows / cols) ** 0.5


class MuonOptimizer(Optimizer):
    def __init__(self, named_params, prefix: str, lr: float, momentum: float = 0.95, nesterov: bool = True,
                 weight_decay: float = 0.0, ns_steps: int = 5):
        super().__init__(named_params, prefix)
        self.lr, self.momentum, self.nesterov = lr, momentum, nesterov
        self.weight_decay, self.ns_steps = weight_decay, ns_steps
        self.ns_fn: Callable = newton_schulz   # replaced by the fused all-gather → NS path under DP
        for name, p in self.named_params:
            if p.dim() < 2:
                raise ValueError(f"Muon needs tensors with ndim >= 2, got '{name}' with shape {tuple(p.shape)}")
            self.state[name]["momentum"] = torch.zeros_like(p, dtype=torch.float32)

    def _ns(self, device) -> Callable:
        if self.ns_fn is not newton_schulz:
            return self.ns_fn
        if device.type == "cuda":
            from ..ops import dispatch
            if dispatch.get_backend() == "auto":
                from ..ops.native_ops import newton_schulz as native_ns
                return native_ns
        return newton_schulz

    def apply_update(self, name: str, p: torch.nn.Parameter, u2d: torch.Tensor) -> None:
        """``p ← p·(1 − lr·wd) − lr·scale·U`` on the master copy; ``u2d`` is the orthogonalised ``(out, rest)`` update."""
        w = self._master(name, p)
        rows, cols = u2d.shape
        scale = max(1.0, rows / cols) ** 0.5
        w.mul_(1.0 - self.lr * self.weight_decay).add_(u2d.float().view_as(w), alpha=-self.lr * scale)
        self._publish(name, p)

    def step(self) -> None:
        with gputx_range("fbamtrain::optimizer::muon_step"):
            return self._step_impl()

    @torch.no_grad()
    def _step_impl(self) -> None:
        self.step_count += 1
        for name, p in self.named_params:
            if p.grad is None:
                continue
            w = self._master(name, p)
            g2 = p.grad.float().reshape(p.shape[0], -1)
            u = muon_update(g2, self.state[name]["momentum"].view_as(g2), self.momentum, self.nesterov,
                            self.ns_steps, self._ns(p.device))
            w.mul_(1.0 - self.lr * self.weight_decay).add_(u.view_as(w), alpha=-self.lr)
            self._publish(name, p)


class MuonWithAuxAdam(Optimizer):
    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], prefix: str, lr: float,
                 momentum: float, nesterov: bool, weight_decay: float, beta1: float, beta2: float, eps: float,
                 adam_names: Optional[Callable[[str], bool]] = None):
        named = list(named_params)
        force_adam = adam_names or (lambda _n: False)
        muon_params = [(n, p) for n, p in named if p.dim() >= 2 and not force_adam(n)]
        adam_params = [(n, p) for n, p in named if not (p.dim() >= 2 and not force_adam(n))]
        self.named_params = named
        self.prefix = prefix
        self.muon = MuonOptimizer(muon_params, prefix + "/muon", lr, momentum, nesterov, weight_decay)
        self.adam = AdamwOptimizer(adam_params, prefix + "/adam", lr, beta1, beta2, eps, weight_decay)
        self.step_count = 0

    @property
    def state(self):  # merged read-only view, used by shared-state hashing
        merged = {}
        merged.update({("muon/" + k): v for k, v in self.muon.state.items()})
        merged.update({("adam/" + k): v for k, v in self.adam.state.items()})
        return merged

    def set_step(self, step: int) -> None:
        self.step_count = int(step)
        self.muon.set_step(step)
        self.adam.set_step(step)

    def reset_masters_from_params(self) -> None:
        self.muon.reset_masters_from_params()
        self.adam.reset_masters_from_params()

    def step(self) -> None:
        self.step_count += 1
        self.muon.step()
        self.adam.step()

    def state_tensors(self):
        out = self.muon.state_tensors()
        out.pop(f"{self.muon.prefix}/__optimizer/step")
        out.update(self.adam.state_tensors())   # the step counter lives under <prefix>/adam/__optimizer/step
        return out

    def load_state_tensors(self, tensors) -> None:
        self.muon.load_state_tensors(tensors)
        self.adam.load_state_tensors(tensors)
        self.step_count = self.adam.step_count
        self.muon.step_count = self.adam.step_count
