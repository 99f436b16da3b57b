"""Convolution weight gradient ``dW[o, r, s, c] = Σ_{n,oh,ow} dY[n,oh,ow,o] · X[n, oh·stride + r·dil − pad, …, c]``.

Run as a split-K tensor-core GEMM whose K dimension is the output pixels: both operands are read in
place through 4-D TMA gathers (``dY`` bricks of 64 pixels as the transposed A operand, the input
shifted by the filter tap as the transposed B operand), each CTA accumulates one ``128 x BN`` tile of
``dW`` for one tap over its share of the pixels in tensor memory and writes it to its own fp32 slab; one
small kernel then sums the slabs in a fixed order and rounds to the output type — no atomics anywhere.
(reference: wgrad with accumulate-into-existing and split-K in
``kernel_gen/kernel_gen/kernels/conv2d_bwd.py:120-232`` and the CUTLASS wgrad path of ``src/passes/conv2d_pass.cpp``.)
"""
from __future__ import annotations

import ctypes as C

import torch

from . import native as nv


def wgrad_pass(x, dy, o: int, c: int, taps, stride: int, out_dtype=None, splits: int = 0, bn: int = 0,
               bm: int = 0) -> torch.Tensor:
    """``dW[o, t, c] = Σ_pixels dY[pixel, o] · X[pixel·stride + taps[t], c]`` → ``(O, len(taps)·C)``.  ``taps`` are
    (dh, dw) offsets in input pixels; a single tap ``(0, 0)`` with stride 1 is the plain product ``dYᵀ · X`` over
    all pixels (used for reductions whose K is the number of pixels)."""
    from .native_ops import _brick, _need_elem
    from ..utils import debug, flops
    elem = _need_elem(x, dy)
    out_dtype = out_dtype or elem               # the operands' 16-bit type unless fp32 is asked for
    b, ih, iw, _ = x.shape
    _, oh, ow, _ = dy.shape
    nt = len(taps)
    if c % 64 != 0 or o % 8 != 0 or not 1 <= nt <= 9:
        raise ValueError("native weight gradient needs input channels in multiples of 64, output channels in "
                         "multiples of 8 and 1 to 9 taps")
    # Split-K over the pixels: every split writes its partial (O, taps·C) tile to its own slab of a workspace with
    # plain stores and one reduction sums the slabs — no atomics, deterministic summation order.
    g_tn, g_th, g_tw = _brick(b, oh, ow, 64)
    bricks = -(-b // g_tn) * -(-oh // g_th) * -(-ow // g_tw)
    if splits <= 0:
        tile_n = 256 if nt * c >= 256 else (128 if nt * c >= 128 else 64)
        tile_m = 256 if (o >= 256 and tile_n >= 128 and bm != 128) else 128
        tiles = -(-o // tile_m) * -(-(nt * c) // tile_n)
        sms = torch.cuda.get_device_properties(x.device).multi_processor_count
        # equal-sized work items are scheduled in waves of one per SM: fill (almost) exactly `waves` waves
        waves = 2 if tiles <= sms // 4 else 4
        splits = max(1, min(bricks, waves * sms // tiles))
    splits = min(splits, bricks)
    work = torch.empty(splits, o, nt * c, dtype=torch.float32, device=x.device)
    p = nv.GemmParams()
    g = p.conv
    g.batch, g.grid_h, g.grid_w = b, oh, ow
    g.tn, g.th, g.tw = g_tn, g_th, g_tw
    g.in_mul = stride
    g.num_taps = nt
    for i, (dh, dw_) in enumerate(taps):
        g.tap_dh[i], g.tap_dw[i] = dh, dw_
    p.D, p.ldd = work.data_ptr(), nt * c
    p.split_workspace, p.split_stride = work.data_ptr(), o * nt * c
    p.status = nv.status_word(x.device).data_ptr()
    p.alpha = 1.0
    p.out_fp32 = 1
    p.splits, p.bn, p.bm = splits, bn, bm
    with debug.label(f"wgrad c{c} o{o} taps{nt}"):
        code = nv.lib(dy).fbam_conv_wgrad(nv.ptr(dy), o, nv.ptr(x), ih, iw, c, C.byref(p), nv.stream_ptr())
    nv.check(code, "fbam_conv_wgrad")
    flops.add(2.0 * b * oh * ow * o * nt * c)
    if splits == 1 and out_dtype == torch.float32:
        return work[0]
    out = torch.empty(o, nt * c, dtype=out_dtype, device=x.device)
    if out_dtype not in (torch.float32, elem):
        raise TypeError("weight gradients are written as fp32 or in the operands' 16-bit type")
    nv.check(nv.lib(elem).fbam_slab_reduce(nv.ptr(work), nv.ptr(out), C.c_longlong(o * nt * c), splits,
                                           int(out_dtype == elem), nv.stream_ptr()), "fbam_slab_reduce")
    return out


def conv2d_wgrad(x, dy, w_shape, stride, padding, dilation, out_dtype=None, splits: int = 0, bn: int = 0,
                 bm: int = 0):
    o, _, _, c = w_shape
    if c % 64 != 0 or o % 8 != 0:
        dw = torch.nn.grad.conv2d_weight(x.permute(0, 3, 1, 2), (o, c, 3, 3), dy.permute(0, 3, 1, 2), stride, padding,
                                         dilation)
        return dw.permute(0, 2, 3, 1).contiguous().to(out_dtype)
    taps = [((i // 3) * dilation - padding, (i % 3) * dilation - padding) for i in range(9)]
    return wgrad_pass(x, dy, o, c, taps, stride, out_dtype, splits, bn, bm).view(o, 3, 3, c)
