"""Building blocks shared by the frame head and the action model.

``Linear`` keeps its weight as ``(out, in)`` — the K-major operand layout of the GEMM kernels —
and the checkpoint layer transposes to the reference's ``(in, out)`` storage (reference:
``tensorlib/include/linear.h:30-33``).  ``FullMhaAttention`` is a fused-QKV projection, a split
into strided q/k/v views, scaled-dot-product attention and an output projection (reference:
``tensorlib/include/attention.h:95-114``); the block wiring ``x += attn(norm(x)); x += mlp(norm(x))``
follows ``src/framehead_model.cpp:339-398``.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from .init_utils import SeedSequence, fill_uniform_fan_


class RmsNorm(nn.Module):
    def __init__(self, dim: int, eps: float, dtype: torch.dtype):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps)


class LayerNorm(nn.Module):
    """Forward-complete LayerNorm (the reference ships it but no model uses it;
    reference: ``tensorlib/include/layer_norm.h:12-78``)."""

    def __init__(self, dim: int, eps: float, dtype: torch.dtype, bias: bool = True):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype)) if bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.layer_norm(x, self.weight, self.bias, self.eps)


class Linear(nn.Module):
    def __init__(self, fan_in: int, fan_out: int, bias: bool, dtype: torch.dtype, seeds: SeedSequence,
                 act: str = "none"):
        super().__init__()
        self.act = act
        self.weight = nn.Parameter(torch.empty(fan_out, fan_in, dtype=dtype))
        fill_uniform_fan_(self.weight.data, fan_in, seeds)
        if bias:
            self.bias = nn.Parameter(torch.empty(fan_out, dtype=dtype))
            fill_uniform_fan_(self.bias.data, fan_in, seeds)
        else:
            self.bias = None

    def forward(self, x: torch.Tensor, residual: torch.Tensor = None) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias, self.act, residual)


class Embedding(nn.Module):
    """Row lookup ``weight[ids]`` with N(0, 1) initialisation; ids outside ``[0, rows)`` give a zero row, as in the
    cell-embedding kernel (reference: ``tensorlib/include/embedding.h:16-85`` — forward only there; here the
    gradient is a scatter-add into the table)."""

    def __init__(self, rows: int, dim: int, dtype: torch.dtype, seeds: SeedSequence):
        super().__init__()
        from .init_utils import fill_normal_
        self.weight = nn.Parameter(torch.empty(rows, dim, dtype=dtype))
        fill_normal_(self.weight.data, seeds)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        rows = self.weight.shape[0]
        valid = (ids >= 0) & (ids < rows)
        out = torch.nn.functional.embedding(ids.clamp(0, rows - 1).long(), self.weight)
        return out * valid.unsqueeze(-1).to(out.dtype)


class Mean(nn.Module):
    """Mean over one dimension with fp32 accumulation (reference: ``tensorlib/include/mean.h:13-138``)."""

    def __init__(self, dim: int, keepdim: bool = False):
        super().__init__()
        self.dim, self.keepdim = dim, keepdim

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x.float().mean(dim=self.dim, keepdim=self.keepdim).to(x.dtype)


class MlpBlock(nn.Module):
    def __init__(self, dim: int, hidden: int, bias: bool, dtype: torch.dtype, seeds: SeedSequence):
        super().__init__()
        self.fc1 = Linear(dim, hidden, bias, dtype, seeds, act="gelu")
        self.fc2 = Linear(hidden, dim, bias, dtype, seeds)

    def forward(self, x: torch.Tensor, residual: torch.Tensor = None) -> torch.Tensor:
        return self.fc2(self.fc1(x), residual)


class FullMhaAttention(nn.Module):
    def __init__(self, dim: int, n_head: int, bias: bool, causal: bool, dtype: torch.dtype, seeds: SeedSequence):
        super().__init__()
        if dim % n_head != 0:
            raise ValueError("n_embed must be divisible by n_head")
        self.n_head, self.causal = n_head, causal
        self.qkv = Linear(dim, 3 * dim, bias, dtype, seeds)
        self.proj = Linear(dim, dim, bias, dtype, seeds)

    def forward(self, x: torch.Tensor, residual: torch.Tensor = None) -> torch.Tensor:
        b, t, e = x.shape
        d = e // self.n_head
        qkv = self.qkv(x.reshape(b * t, e)).view(b, t, 3, self.n_head, d)
        o = ops.attention_qkv(qkv, self.causal)
        res = None if residual is None else residual.reshape(b * t, e)
        return self.proj(o.reshape(b * t, e), res).view(b, t, e)


class AttentionBlock(nn.Module):
    def __init__(self, dim: int, n_head: int, mlp_dim: int, bias: bool, causal: bool, eps: float,
                 dtype: torch.dtype, seeds: SeedSequence):
        super().__init__()
        self.ln1 = RmsNorm(dim, eps, dtype)
        self.attn = FullMhaAttention(dim, n_head, bias, causal, dtype, seeds)
        self.ln2 = RmsNorm(dim, eps, dtype)
        self.mlp = MlpBlock(dim, mlp_dim, bias, dtype, seeds)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # the residual additions ride in the epilogues of the output-projection and second MLP GEMMs
        x = self.attn(self.ln1(x), residual=x)
        b, t, e = x.shape
        x2 = x.reshape(b * t, e)
        return self.mlp(self.ln2(x).reshape(b * t, e), residual=x2).view(b, t, e)
