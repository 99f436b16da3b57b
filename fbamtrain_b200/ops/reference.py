"""Plain-PyTorch definitions of every op.  They are the numerics oracle for the CUDA kernels
(tests run them in fp32) and the execution path on CPU, where autograd differentiates them.

Layouts: activations NHWC / token-major, conv weights OHWI, linear weights ``(out, in)``, LSTM
weights ``(4H, in)`` with gate order i, f, g, o, time-major LSTM sequences ``(T, B, ·)``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def cell_embed(cells: torch.Tensor, cp_embed: torch.Tensor, pos_embed: torch.Tensor, colour_embed: torch.Tensor,
               out_dtype: torch.dtype) -> torch.Tensor:
    """``cells`` int32 ``(N, P, 3)`` → ``(N, P, E)``.

    ``out[n, p] = cp_embed[cp] (zero when cp is outside the table) + pos_embed[p mod P]
    + Σ_c (channel_c / 255) · colour_embed[c]`` with c over fg r,g,b then bg r,g,b, accumulated in
    fp32 (reference: ``kernel_gen/kernel_gen/kernels/build_cell_embeds.py:74-134``)."""
    n, p, _ = cells.shape
    cp = cells[..., 0].long()
    valid = (cp >= 0) & (cp < cp_embed.shape[0])
    e = cp_embed.float()[cp.clamp(0, cp_embed.shape[0] - 1)] * valid.unsqueeze(-1)
    e = e + pos_embed.float()[torch.arange(p, device=cells.device) % pos_embed.shape[0]].unsqueeze(0)
    fg, bg = cells[..., 1].long(), cells[..., 2].long()
    chans = torch.stack([(fg >> 16) & 255, (fg >> 8) & 255, fg & 255,
                         (bg >> 16) & 255, (bg >> 8) & 255, bg & 255], dim=-1).float() / 255.0
    e = e + chans @ colour_embed.float()
    return e.to(out_dtype)


def conv2d_nhwc(x: torch.Tensor, w_ohwi: torch.Tensor, stride: int, padding: int, dilation: int) -> torch.Tensor:
    y = F.conv2d(x.permute(0, 3, 1, 2), w_ohwi.permute(0, 3, 1, 2), None, stride, padding, dilation)
    return y.permute(0, 2, 3, 1).contiguous()


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return y.to(x.dtype)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps).to(x.dtype)


def gelu(x: torch.Tensor) -> torch.Tensor:
    """Exact (erf) GELU (reference: ``kernel_gen/kernel_gen/kernels/act.py:43-63``)."""
    return F.gelu(x.float(), approximate="none").to(x.dtype)


def gelu_grad(x: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    return 0.5 * (1.0 + torch.erf(xf / math.sqrt(2.0))) + xf * torch.exp(-0.5 * xf * xf) / math.sqrt(2.0 * math.pi)


def geglu(x: torch.Tensor) -> torch.Tensor:
    """Channel-split gated GELU: first half is the value, second half the gate."""
    v, g = x.chunk(2, dim=-1)
    return (v.float() * F.gelu(g.float())).to(x.dtype)


def avg_pool2x2_nhwc(x: torch.Tensor) -> torch.Tensor:
    n, h, w, c = x.shape
    return x.float().reshape(n, h // 2, 2, w // 2, 2, c).mean(dim=(2, 4)).to(x.dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], act: str = "none") -> torch.Tensor:
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    if act == "gelu":
        y = F.gelu(y)
    elif act == "relu":
        y = F.relu(y)
    return y.to(x.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool) -> torch.Tensor:
    """``q, k, v``: ``(B, T, H, D)`` (possibly strided views of a fused qkv buffer); returns ``(B, T, H, D)``."""
    d = q.shape[-1]
    s = torch.einsum("bthd,bshd->bhts", q.float(), k.float()) / math.sqrt(d)
    if causal:
        t = q.shape[1]
        mask = torch.ones(t, k.shape[1], dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhts,bshd->bthd", p, v.float()).to(q.dtype)


def lstm_cell(gates: torch.Tensor, c_prev: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``gates`` fp32 ``(B, 4H)`` pre-activations in order i, f, g, o → ``(h, c)`` fp32."""
    i, f, g, o = gates.float().chunk(4, dim=-1)
    c = torch.sigmoid(f) * c_prev.float() + torch.sigmoid(i) * torch.tanh(g)
    h = torch.sigmoid(o) * torch.tanh(c)
    return h, c


def lstm_sequence(x: torch.Tensor, w_ih: torch.Tensor, w_hh: torch.Tensor, b_ih: torch.Tensor, b_hh: torch.Tensor,
                  h0: torch.Tensor, c0: torch.Tensor, compute_dtype: torch.dtype):
    """Time-major LSTM.  ``x`` ``(T, B, I)``; weights fp32 ``(4H, I)``/``(4H, H)`` cast to
    ``compute_dtype`` for the matrix products; gates and cell state in fp32; ``h`` is rounded to
    ``compute_dtype`` between steps, as the reference does (reference:
    ``tensorlib/include/streaming_lstm.h:60-75``, ``kernel_gen/kernel_gen/kernels/lstm_cell.py:126-144``).
    ``h0``/``c0`` are ``(H,)`` and broadcast over the batch.  Returns ``(y (T,B,H), h_T, c_T)``."""
    t_len, b, _ = x.shape
    hdim = w_hh.shape[1]
    wi, wh = w_ih.to(compute_dtype), w_hh.to(compute_dtype)
    bias = (b_ih.float() + b_hh.float())
    h = h0.to(compute_dtype).unsqueeze(0).expand(b, hdim)
    c = c0.float().unsqueeze(0).expand(b, hdim)
    xg = (x.to(compute_dtype).reshape(t_len * b, -1) @ wi.t()).float().reshape(t_len, b, 4 * hdim)
    ys = []
    for t in range(t_len):
        gates = xg[t] + (h @ wh.t()).float() + bias
        hf, c = lstm_cell(gates, c)
        h = hf.to(compute_dtype)
        ys.append(h)
    return torch.stack(ys, 0), h, c


def cross_entropy_sum(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    return F.cross_entropy(logits.float(), targets.long(), reduction="sum")


def lm_head_ce(x: torch.Tensor, w_head: torch.Tensor, targets: torch.Tensor, vocab: int, scale: float) -> torch.Tensor:
    """``x`` ``(rows, H)``, ``w_head`` ``(V_pad, H)``; columns ≥ ``vocab`` are padding and ignored.
    Returns ``scale · Σ_rows CE`` (reference: ``src/main.cpp:1377-1463, 2428``)."""
    logits = (x.float() @ w_head.float().t())[:, :vocab]
    return cross_entropy_sum(logits, targets) * scale
