"""Convolution weight gradient ``dW[o, r, s, c] = Σ_{n,oh,ow} dY[n,oh,ow,o] · X[n, oh·stride + r·dil − pad, …, c]``.

Run as a split-K tensor-core GEMM whose K dimension is the output pixels: both operands are read in
place through 4-D TMA gathers (``dY`` bricks of 64 pixels as the transposed A operand, the input
shifted by the filter tap as the transposed B operand), each CTA accumulates one ``128 x BN`` tile of
``dW`` for one tap over its share of the pixels in tensor memory, and partial tiles are added into an
fp32 ``dW`` with atomics.  (reference: wgrad with accumulate-into-existing and split-K in
``kernel_gen/kernel_gen/kernels/conv2d_bwd.py:120-232`` and the CUTLASS wgrad path of ``src/passes/conv2d_pass.cpp``.)
"""
from __future__ import annotations

import ctypes as C

import torch

from . import native as nv


def conv2d_wgrad(x, dy, w_shape, stride, padding, dilation, out_dtype=torch.bfloat16, splits: int = 0, bn: int = 0,
                 bm: int = 0):
    from .native_ops import _brick
    o, _, _, c = w_shape
    b, ih, iw, _ = x.shape
    _, oh, ow, _ = dy.shape
    if c % 64 != 0 or o % 8 != 0:
        dw = torch.nn.grad.conv2d_weight(x.permute(0, 3, 1, 2), (o, c, 3, 3), dy.permute(0, 3, 1, 2), stride, padding,
                                         dilation)
        return dw.permute(0, 2, 3, 1).contiguous().to(out_dtype)
    # Split-K over the pixels: every split writes its partial (O, 9C) tile to its own slab of a workspace with plain
    # stores and one reduction sums the slabs — no atomics, deterministic summation order.
    g_tn, g_th, g_tw = _brick(b, oh, ow, 64)
    bricks = -(-b // g_tn) * -(-oh // g_th) * -(-ow // g_tw)
    if splits <= 0:
        tile_n = 256 if 9 * c >= 256 else (128 if 9 * c >= 128 else 64)
        tile_m = 256 if (o >= 256 and tile_n >= 128 and bm != 128) else 128
        tiles = -(-o // tile_m) * -(-(9 * c) // tile_n)
        sms = torch.cuda.get_device_properties(x.device).multi_processor_count
        # equal-sized work items are scheduled in waves of one per SM: fill (almost) exactly `waves` waves
        waves = 2 if tiles <= sms // 4 else 4
        splits = max(1, min(bricks, waves * sms // tiles))
    splits = min(splits, bricks)
    work = torch.empty(splits, o, 9 * c, dtype=torch.float32, device=x.device)
    p = nv.GemmParams()
    g = p.conv
    g.batch, g.grid_h, g.grid_w = b, oh, ow
    g.tn, g.th, g.tw = g_tn, g_th, g_tw
    g.in_mul = stride
    g.num_taps = 9
    for i in range(9):
        g.tap_dh[i], g.tap_dw[i] = (i // 3) * dilation - padding, (i % 3) * dilation - padding
    p.D, p.ldd = work.data_ptr(), 9 * c
    p.split_workspace, p.split_stride = work.data_ptr(), o * 9 * c
    p.status = nv.status_word(x.device).data_ptr()
    p.alpha = 1.0
    p.out_fp32 = 1
    p.splits, p.bn, p.bm = splits, bn, bm
    from ..utils import debug
    with debug.label(f"wgrad c{c} o{o}"):
        code = nv.lib().fbam_conv_wgrad_bf16(nv.ptr(dy), o, nv.ptr(x), ih, iw, c, C.byref(p), nv.stream_ptr())
    nv.check(code, "fbam_conv_wgrad_bf16")
    from ..utils import flops
    flops.add(2.0 * b * oh * ow * o * 9 * c)
    dw = work[0] if splits == 1 else work.sum(0)
    return dw.view(o, 3, 3, c).to(out_dtype)
