"""Contiguous parameter / gradient buffers.

All parameters of one scope and dtype are packed into a single flat tensor, each at a
256-byte-aligned offset, and so are their gradients — the arrangement the reference obtains by
running its gradient-allocation graph under a bump allocator (reference: ``src/main.cpp:745-807,
2340-2396``; alignment ``753-779``).  One flat buffer per group means one collective per group, one
fused optimizer launch per group, and shard boundaries that are plain offsets.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Tuple

import torch

ALIGN_BYTES = 256


class FlatGroup:
    """Parameters of one (scope, dtype) packed into ``data`` with gradients in ``grad``."""

    def __init__(self, name: str, named_params: List[Tuple[str, torch.nn.Parameter]], shard_multiple: int = 1):
        if not named_params:
            raise ValueError("empty parameter group")
        self.name = name
        self.named_params = named_params
        p0 = named_params[0][1]
        self.dtype, self.device = p0.dtype, p0.device
        align = ALIGN_BYTES // p0.element_size()
        self.offsets: Dict[str, int] = {}
        off = 0
        for n, p in named_params:
            if p.dtype != self.dtype or p.device != self.device:
                raise ValueError(f"parameter '{n}' does not match group dtype/device")
            self.offsets[n] = off
            off += (p.numel() + align - 1) // align * align
        unit = align * max(1, shard_multiple)
        self.numel = (off + unit - 1) // unit * unit
        self.data = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
        self.grad = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
        for n, p in named_params:
            o = self.offsets[n]
            view = self.data[o:o + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view
            p.grad = self.grad[o:o + p.numel()].view_as(p)

    def view_of(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        """The slice of a same-length flat tensor (e.g. optimizer state) that belongs to ``name``."""
        p = dict(self.named_params)[name]
        o = self.offsets[name]
        return flat[o:o + p.numel()].view_as(p)

    def rebind_grads(self) -> None:
        """Re-points ``p.grad`` at the flat buffer (needed after something set grads to None)."""
        for n, p in self.named_params:
            o = self.offsets[n]
            p.grad = self.grad[o:o + p.numel()].view_as(p)


def build_groups(scope: str, named_params: Iterable[Tuple[str, torch.nn.Parameter]],
                 shard_multiple: int = 1) -> List[FlatGroup]:
    """One group per dtype, in first-appearance order."""
    by_dtype: Dict[torch.dtype, List[Tuple[str, torch.nn.Parameter]]] = {}
    for n, p in named_params:
        by_dtype.setdefault(p.dtype, []).append((n, p))
    return [FlatGroup(f"{scope}/{str(dt).replace('torch.', '')}", ps, shard_multiple) for dt, ps in by_dtype.items()]
