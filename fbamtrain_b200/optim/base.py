"""Optimizer base: named parameters, fp32 master copies for 16-bit parameters, named state.

State naming follows the reference's checkpoint layout (reference: ``src/optimizers.cpp:25-32,
471-483, 872-876, 1472-1481``): ``<prefix>/<param>/{m,v,master,momentum,velocity}`` and
``<prefix>/__optimizer/step`` (a one-element unsigned 64-bit counter).  ``state_tensors()`` returns
that flat name → tensor mapping and ``load_state_tensors()`` restores it with strict dtype/shape
checks (reference: ``src/optimizers.cpp:66-75``).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Tuple

import torch


class Optimizer:
    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], prefix: str):
        self.named_params: List[Tuple[str, torch.nn.Parameter]] = [(n, p) for n, p in named_params]
        self.prefix = prefix
        self.step_count = 0
        self.state: Dict[str, Dict[str, torch.Tensor]] = {}
        for name, p in self.named_params:
            st: Dict[str, torch.Tensor] = {}
            if p.dtype in (torch.float16, torch.bfloat16):
                st["master"] = p.detach().float().clone()
            self.state[name] = st

    # -- helpers ----------------------------------------------------------------------------
    def _master(self, name: str, p: torch.nn.Parameter) -> torch.Tensor:
        return self.state[name].get("master", p.data)

    def _publish(self, name: str, p: torch.nn.Parameter) -> None:
        """Rounds the updated master copy into the parameter."""
        if "master" in self.state[name]:
            p.data.copy_(self.state[name]["master"])

    def zero_grad(self) -> None:
        for _, p in self.named_params:
            if p.grad is not None:
                p.grad.zero_()

    def set_step(self, step: int) -> None:
        self.step_count = int(step)

    @torch.no_grad()
    def reset_masters_from_params(self) -> None:
        """After parameters were overwritten from outside (a model-only checkpoint): the fp32 master copies follow."""
        for name, p in self.named_params:
            master = self.state.get(name, {}).get("master")
            if master is not None:
                master.copy_(p.detach().float())

    def step(self) -> None:
        raise NotImplementedError

    # -- (de)serialisation ------------------------------------------------------------------
    def state_tensors(self) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for name, st in self.state.items():
            for key, t in st.items():
                out[f"{self.prefix}/{name}/{key}"] = t
        out[f"{self.prefix}/__optimizer/step"] = torch.tensor([self.step_count], dtype=torch.int64)
        return out

    def load_state_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        for name, st in self.state.items():
            for key, t in st.items():
                full = f"{self.prefix}/{name}/{key}"
                if full not in tensors:
                    raise KeyError(f"optimizer state '{full}' missing from checkpoint")
                src = tensors[full]
                if src.dtype != t.dtype or tuple(src.shape) != tuple(t.shape):
                    raise ValueError(f"optimizer state '{full}' is {src.dtype}{tuple(src.shape)}, "
                                     f"expected {t.dtype}{tuple(t.shape)}")
                t.copy_(src)
        key = f"{self.prefix}/__optimizer/step"
        if key in tensors:
            self.step_count = int(tensors[key].reshape(-1)[0])
        for name, p in self.named_params:
            self._publish(name, p)
