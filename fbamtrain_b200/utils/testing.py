"""Tensor comparison helpers used by the tests and by ``tenscmp``.

``assert_similar`` mirrors the acceptance rule of the reference's test helper (reference:
``tensorlib/src/testing.cpp:8-137``): element-wise absolute tolerance; for 16-bit floating types
an element also passes when it is within one unit in the last place of the expected value; any
non-finite value in either tensor fails; shapes must match (strides need not).
"""
from __future__ import annotations

import torch


def _ulp(expected: torch.Tensor) -> torch.Tensor:
    mant = {torch.bfloat16: 7, torch.float16: 10}[expected.dtype]
    e = expected.float().abs().clamp_min(torch.finfo(expected.dtype).tiny)
    return torch.exp2(torch.floor(torch.log2(e)) - mant)


def max_abs_diff(a: torch.Tensor, b: torch.Tensor) -> float:
    if a.numel() == 0:
        return 0.0
    return float((a.double().cpu() - b.double().cpu()).abs().max())


def assert_similar(expected: torch.Tensor, actual: torch.Tensor, tol: float, name: str = "tensor") -> None:
    if tuple(expected.shape) != tuple(actual.shape):
        raise AssertionError(f"{name}: shape {tuple(actual.shape)} != expected {tuple(expected.shape)}")
    e, a = expected.detach().cpu(), actual.detach().cpu()
    if e.is_floating_point() and not (torch.isfinite(e.float()).all() and torch.isfinite(a.float()).all()):
        raise AssertionError(f"{name}: non-finite values present")
    diff = (e.double() - a.double()).abs()
    ok = diff <= tol
    if e.dtype in (torch.bfloat16, torch.float16) and a.dtype == e.dtype:
        ok |= diff <= _ulp(e).double() * 1.0000001
    if not bool(ok.all()):
        idx = int(torch.argmax(diff.flatten() * (~ok).flatten()))
        raise AssertionError(f"{name}: {int((~ok).sum())} of {ok.numel()} elements differ by more than {tol}; "
                             f"worst at flat index {idx}: expected {float(e.flatten()[idx])}, "
                             f"got {float(a.flatten()[idx])}")
