"""Scaled-dot-product attention over ``(B, T, H, D)`` views on the tcgen05 flash kernels
(``csrc/attention_tcgen05.cu``): causal or not, head dimension 64 or 128, bf16.

q, k and v are normally strided views into one fused-QKV projection output and are consumed in place
(reference layout: ``tensorlib/include/attention.h:95-114``; the reference's kernels cover head
dimension 128 only, ``src/passes/mha_attention_pass.cpp:1017-1124``).  The forward returns the
output and keeps the per-row log-sum-exp for the backward pass.  Other head dimensions run the
library attention.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import torch

import torch.nn.functional as F

from ..utils import flops
from . import native as nv

_warned = set()


def _same_layout(q, k, v) -> bool:
    return q.stride() == k.stride() == v.stride() and q.stride(3) == 1


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal):
        b, t, h, d = q.shape
        if not _same_layout(q, k, v):
            q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out = torch.empty(b, t, h, d, dtype=q.dtype, device=q.device)
        lse = torch.empty(b, h, t, dtype=torch.float32, device=q.device)
        scale = 1.0 / math.sqrt(d)
        sb, st, sh = q.stride(0), q.stride(1), q.stride(2)
        # Two query tiles per CTA (one tile's softmax overlaps the other's MMAs): 0.131 ms against 0.215 ms for one
        # tile per CTA at B8 H8 T1024 D128.  FBAMTRAIN_ATTENTION_FWD2=0 selects the one-tile kernel (same results).
        fwd = nv.lib(q).fbam_attn_fwd if os.environ.get("FBAMTRAIN_ATTENTION_FWD2", "1") == "0" else nv.lib(q).fbam_attn_fwd2
        nv.check(fwd(nv.ptr(q), nv.ptr(k), nv.ptr(v), C.c_longlong(sb), C.c_longlong(st), C.c_longlong(sh),
                     nv.ptr(out), nv.ptr(lse), b, t, h, d, int(causal), C.c_float(scale),
                     nv.ptr(nv.status_word(q.device)), nv.stream_ptr()), "fbam_attn_fwd")
        flops.add(4.0 * b * h * t * t * d * (0.5 if causal else 1.0))
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, d_out, raw_dq=False):
        q, k, v, out, lse = ctx.saved_tensors
        b, t, h, d = q.shape
        if d_out.stride(3) != 1:
            d_out = d_out.contiguous()
        dq32 = torch.zeros(b, t, h, d, dtype=torch.float32, device=q.device)
        dk = torch.empty(b, t, h, d, dtype=q.dtype, device=q.device)
        dv = torch.empty(b, t, h, d, dtype=q.dtype, device=q.device)
        delta = torch.empty(b, h, t, dtype=torch.float32, device=q.device)
        nv.check(nv.lib(q).fbam_attn_bwd(
            nv.ptr(q), nv.ptr(k), nv.ptr(v), C.c_longlong(q.stride(0)), C.c_longlong(q.stride(1)),
            C.c_longlong(q.stride(2)), nv.ptr(out), nv.ptr(d_out), C.c_longlong(d_out.stride(0)),
            C.c_longlong(d_out.stride(1)), C.c_longlong(d_out.stride(2)), nv.ptr(lse), nv.ptr(delta), nv.ptr(dq32),
            nv.ptr(dk), nv.ptr(dv), b, t, h, d, int(ctx.causal), C.c_float(ctx.scale),
            nv.ptr(nv.status_word(q.device)), nv.stream_ptr()), "fbam_attn_bwd")
        flops.add(10.0 * b * h * t * t * d * (0.5 if ctx.causal else 1.0))   # 2.5 x forward
        return (dq32 if raw_dq else dq32.to(q.dtype)), dk, dv, None


class _FlashAttentionQkv(torch.autograd.Function):
    """Attention on the fused projection output ``qkv (B, T, 3, H, D)``: q, k and v are read in place as strided views
    and the three gradients are written into one ``(B, T, 3, H, D)`` buffer, so autograd sees a single tensor in and
    a single gradient out (separate q / k / v selections would each materialise a zero-filled full-size gradient)."""

    @staticmethod
    def forward(ctx, qkv, causal):
        out = _FlashAttention.forward(ctx, qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal)
        ctx.qkv_shape = qkv.shape
        return out

    @staticmethod
    def backward(ctx, d_out):
        dq, dk, dv, _ = _FlashAttention.backward(ctx, d_out, raw_dq=True)
        dqkv = torch.empty(ctx.qkv_shape, dtype=dk.dtype, device=d_out.device)
        dqkv[:, :, 0].copy_(dq)            # fp32 accumulator -> 16-bit, straight into its slice
        dqkv[:, :, 1].copy_(dk)
        dqkv[:, :, 2].copy_(dv)
        return dqkv, None


def flash_attention_qkv(qkv, causal):
    """``qkv`` bf16 or fp16 ``(B, T, 3, H, D)`` contiguous → ``(B, T, H, D)``."""
    d = qkv.shape[-1]
    if qkv.dtype in nv.ELEM_DTYPES and d in (64, 128) and qkv.is_contiguous() and (3 * qkv.shape[3] * d * 2) % 16 == 0:
        return _FlashAttentionQkv.apply(qkv, bool(causal))
    return flash_attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal)


def flash_attention(q, k, v, causal):
    d = q.shape[-1]
    if q.dtype in nv.ELEM_DTYPES and q.dtype == k.dtype == v.dtype and d in (64, 128) and (q.stride(0) * 2) % 16 == 0 and (q.stride(1) * 2) % 16 == 0:
        return _FlashAttention.apply(q, k, v, bool(causal))
    if d not in _warned:
        _warned.add(d)
        from ..utils.logging import LOG
        LOG("WARN", f"attention with head dimension {d} runs the library kernel (native kernels cover 64 and 128)")
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal)
    return o.transpose(1, 2).contiguous()
