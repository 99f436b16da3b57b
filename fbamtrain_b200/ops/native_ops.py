"""CUDA implementations of the functional ops: autograd Functions over the native kernels.

Tensor-core work (linear layers, convolutions, LM head) goes through the tcgen05 GEMM /
implicit-GEMM entry points; everything else through the bandwidth-bound kernels.  Model dtype on
this path is bf16 (fp32 parameters — embeddings, LSTM — are handled where noted).

What the reference does in lowering passes over its op graph — fusing bias / GELU / pre-activation output into
the GEMM, choosing transposed-operand variants, splitting convolutions into fprop / dgrad / wgrad kernels
(reference: ``src/passes/matmul_pass.cpp:2783-3689``, ``src/passes/conv2d_pass.cpp``) — happens here at call
time: the autograd Functions pick the epilogue and operand form of each launch.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional, Tuple

import torch

from ..utils import debug, flops
from . import native as nv
from . import tuning

BF16 = torch.bfloat16
# Large problems run on CTA pairs (tcgen05 cta_group::2: two SMs share every B fetch and keep double-buffered
# accumulators).  "auto" picks the pair kernel when there are enough 256-row tiles; False forces single CTAs.
TWO_CTA = "auto"
# Weight-gradient and data-gradient GEMMs read their operands in place through the transposed
# (MN-major) operand form of the tensor-core descriptors.  False = materialise transposes instead.
USE_MN_MAJOR = True


def _need_elem(*ts) -> torch.dtype:
    """All given tensors must share one 16-bit element type (bf16 or half); returns it."""
    dtype = None
    for t in ts:
        if t is None:
            continue
        if t.dtype not in nv.ELEM_DTYPES:
            raise TypeError(f"native kernels take bf16 or fp16 tensors, got {t.dtype}")
        if dtype is not None and t.dtype != dtype:
            raise TypeError(f"native kernels take operands of one 16-bit type, got {dtype} and {t.dtype}")
        dtype = t.dtype
    return dtype


# =================================================================================================
# GEMM
# =================================================================================================
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, bias: Optional[torch.Tensor] = None,
         act: str = "none", residual: Optional[torch.Tensor] = None, preact_out: Optional[torch.Tensor] = None,
         gelu_grad_in: Optional[torch.Tensor] = None, accumulate: int = 0, alpha: float = 1.0,
         bn: int = 0, bm: int = 0, max_ctas: int = 0, ready_flags: Optional[torch.Tensor] = None,
         flag_rows: int = 0, flag_on_b: bool = False, flag_epoch: int = 0, flag_spin_limit: int = 0,
         rs_out=None, rs_rows_per_rank: int = 0, tile_m_rotate: int = 0, two_cta=None,
         rs_slot: int = -1, rs_row_stores: bool = False, ce_stats=None, ce_grad=None, splits: int = 0) -> torch.Tensor:
    """``D[M, N] = epilogue(A · Bᵀ)``.

    ``a``: ``(M, K)`` (or ``(K, M)`` when ``a_mn``); ``b``: ``(N, K)`` (or ``(K, N)`` when ``b_mn``).
    Operands must be bf16 or fp16 (both the same) with unit inner stride; ``out_dtype`` defaults to theirs.  ``accumulate``: 0 overwrite,
    1 read-modify-write ``D +=``, 2 atomic adds (fp32 output only).

    ``ready_flags`` (int32 tensor in local memory, written by peers) gates the loads of A (or B with
    ``flag_on_b``): rows ``[i·flag_rows, (i+1)·flag_rows)`` are read only once ``ready_flags[i] >= flag_epoch``
    (all-gather → GEMM).  ``rs_out`` (list of peer buffer addresses) with ``rs_rows_per_rank`` sends each tile to
    the rank owning its output rows (GEMM → reduce-scatter): with ``rs_slot = s`` as bf16 stores into slot ``s`` of
    the owner's ``[slot][rows][n]`` buffer (the owner sums the slots afterwards), with ``rs_slot = -1`` as fp32
    remote additions into the owner's ``[rows][n]`` buffer; ``out`` is then only used for its shape and pitch.
    ``rs_row_stores`` (slot form): lanes exchange pieces so that each store instruction writes 64 contiguous bytes
    of a row instead of 16 bytes of 32 rows (needs ``M`` and ``rs_rows_per_rank`` in multiples of 32).
    ``two_cta`` selects the CTA-pair kernel (default: automatically for large problems).

    ``splits`` > 1: split-K over that many CTAs per tile (single-CTA kernel); every split writes its fp32 partial tile
    to a slab of a workspace with plain stores and one reduction sums the slabs into the output (no atomics, fixed
    summation order) — for small outputs with a long K, which otherwise occupy a fraction of the SMs.

    Fused LM head + cross-entropy: ``ce_stats = (partial, tgt_logit, targets, vocab)`` stores nothing per element and
    leaves per-row (maximum, sum of exp) pairs of every tile half in ``partial`` ``(M, 2·⌈N/256⌉, 2)`` fp32 and the
    target logits in ``tgt_logit``; ``ce_grad = (lse, targets, vocab, scale)`` writes ``scale·(softmax − onehot)``
    computed from the accumulators and the rows' log-sum-exp instead of the logits."""
    _need_elem(a, b)
    if a.stride(-1) != 1 or b.stride(-1) != 1:
        raise ValueError("GEMM operands need unit inner stride")
    a, b = _tma_pitch(a), _tma_pitch(b)
    m, k = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    n, kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if k != kb:
        raise ValueError(f"inner dimensions differ: {k} vs {kb}")
    if splits > 1:
        if (bias is not None or act != "none" or residual is not None or preact_out is not None or accumulate or
                gelu_grad_in is not None or rs_out is not None or ready_flags is not None or ce_stats or ce_grad
                or alpha != 1.0):
            raise ValueError("split-K takes no epilogue options")
        return _gemm_split_k(a, b, a_mn, b_mn, m, n, k, out, out_dtype or a.dtype, splits, bm, bn)
    if (bm == 0 and bn == 0 and max_ctas == 0 and two_cta is None and ready_flags is None and rs_out is None and
            ce_stats is None and ce_grad is None):
        tuned = tuning.lookup(tuning.gemm_key(m, n, k, a_mn, b_mn), {"m": m, "n": n, "k": k, "a_mn": a_mn, "b_mn": b_mn})
        if tuned is not None:
            bm, bn, max_ctas = tuned.get("bm", 0), tuned.get("bn", 0), tuned.get("max_ctas", 0)
            two_cta = tuned.get("two_cta")
    p = nv.GemmParams()
    if ce_stats is not None:
        partial, tgt_logit, targets, vocab = ce_stats
        slots = 2 * ((n + 255) // 256)
        if partial.shape != (m, slots, 2) or partial.dtype != torch.float32 or not partial.is_contiguous():
            raise ValueError(f"ce_stats partial buffer must be fp32 ({m}, {slots}, 2)")
        p.ce_mode, p.ce_vocab, p.ce_slots = 1, vocab, slots
        p.ce_partial, p.ce_tgt_logit, p.ce_targets = partial.data_ptr(), tgt_logit.data_ptr(), targets.data_ptr()
        out = partial                       # nothing is written through D in this mode
        two_cta = False
    elif out is None:
        out = debug.fresh((m, n), out_dtype or a.dtype, a.device)
    if ce_stats is None and (out.shape != (m, n) or out.stride(1) != 1):
        raise ValueError("output has the wrong shape or layout")
    if ce_grad is not None:
        lse, targets, vocab, scale = ce_grad
        p.ce_mode, p.ce_vocab, p.ce_scale = 2, vocab, scale
        p.ce_lse, p.ce_targets = lse.data_ptr(), targets.data_ptr()
        two_cta = False
    p.D, p.ldd = out.data_ptr(), (n if ce_stats is not None else out.stride(0))
    p.bias = 0 if bias is None else bias.data_ptr()
    p.bias_fp32 = int(bias is not None and bias.dtype == torch.float32)
    if residual is not None:
        _need_elem(residual)
        p.residual, p.ldr = residual.data_ptr(), residual.stride(0)
    if preact_out is not None:
        if preact_out.stride(0) != out.stride(0):
            raise ValueError("preact_out must share the output's row pitch")
        p.preact_out = preact_out.data_ptr()
    if gelu_grad_in is not None:
        if gelu_grad_in.stride(0) != out.stride(0):
            raise ValueError("gelu_grad_in must share the output's row pitch")
        p.gelu_grad_in = gelu_grad_in.data_ptr()
    p.status = nv.status_word(a.device).data_ptr()
    p.alpha = alpha
    p.out_fp32 = int(out.dtype == torch.float32)
    p.act = nv.GEMM_ACT[act]
    p.accumulate = accumulate
    p.bn, p.bm, p.max_ctas = bn, bm, max_ctas
    p.tile_m_rotate = tile_m_rotate
    if ready_flags is not None:
        p.ready_flags = ready_flags.data_ptr()
        p.flag_rows, p.flag_on_b, p.flag_epoch, p.flag_spin_limit = flag_rows, int(flag_on_b), flag_epoch, flag_spin_limit
    if rs_out is not None:
        for i, ptr_ in enumerate(rs_out):
            p.rs_out[i] = ptr_
        p.rs_rows_per_rank = rs_rows_per_rank
        p.rs_slot_plus1 = rs_slot + 1
        p.rs_row_stores = int(rs_row_stores)
    pair = TWO_CTA if two_cta is None else two_cta
    if pair == "auto":
        pair = (n >= 256 and n % 16 == 0 and bm != 128 and
                ((m + 255) // 256) * ((n + 255) // 256) >= 148)
    fn = nv.lib(a).fbam_gemm2 if pair else nv.lib(a).fbam_gemm
    with debug.label(f"gemm{'2' if pair else ''} m{m} n{n} k{k} {'T' if a_mn else 'N'}{'T' if b_mn else 'N'}"):
        code = fn(nv.ptr(a), C.c_longlong(a.stride(0)), int(a_mn), nv.ptr(b), C.c_longlong(b.stride(0)), int(b_mn),
                  m, n, k, C.byref(p), nv.stream_ptr())
    nv.check(code, "fbam_gemm")
    flops.add(2.0 * m * n * k)
    debug.after_launch("gemm", a, b, out)
    return out


def _gemm_split_k(a, b, a_mn, b_mn, m, n, k, out, out_dtype, splits, bm, bn) -> torch.Tensor:
    splits = max(1, min(splits, (k + 63) // 64))
    work = torch.empty(splits, m, n, dtype=torch.float32, device=a.device)
    p = nv.GemmParams()
    p.D, p.ldd = work.data_ptr(), n
    p.split_workspace, p.split_stride = work.data_ptr(), m * n
    p.status = nv.status_word(a.device).data_ptr()
    p.alpha, p.out_fp32, p.splits, p.bn, p.bm = 1.0, 1, splits, bn, bm
    with debug.label(f"gemm m{m} n{n} k{k} {'T' if a_mn else 'N'}{'T' if b_mn else 'N'} split{splits}"):
        code = nv.lib(a).fbam_gemm(nv.ptr(a), C.c_longlong(a.stride(0)), int(a_mn), nv.ptr(b), C.c_longlong(b.stride(0)),
                                   int(b_mn), m, n, k, C.byref(p), nv.stream_ptr())
    nv.check(code, "fbam_gemm")
    flops.add(2.0 * m * n * k)
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    if not out.is_contiguous() or out.dtype not in (torch.float32, a.dtype) or (m * n) % 8:
        out.copy_(work.sum(0))
        return out
    nv.check(nv.lib(a).fbam_slab_reduce(nv.ptr(work), nv.ptr(out), C.c_longlong(m * n), splits,
                                        int(out.dtype != torch.float32), nv.stream_ptr()), "fbam_slab_reduce")
    return out


# FBAMTRAIN_WGRAD_SPLIT_K=0 keeps the weight gradients of the linear layers on single launches without split-K.
WEIGHT_GRAD_SPLIT_K = os.environ.get("FBAMTRAIN_WGRAD_SPLIT_K", "1") != "0"


def weight_grad_splits(m: int, n: int, k: int) -> int:
    """Split-K factor for ``dW = dYᵀ·X`` products whose output is small and whose K (the number of rows of the batch)
    is long: a 1024 x 1024 output is 16 tiles of 256 x 256 — a tenth of the SMs — unless K is divided."""
    tiles = ((m + 255) // 256) * ((n + 255) // 256)
    if not WEIGHT_GRAD_SPLIT_K or k < 4096 or tiles > 48:
        return 0
    return max(1, min(8, 148 // tiles, k // 1024))


def _tma_pitch(t: torch.Tensor) -> torch.Tensor:
    """TMA needs a 16-byte aligned base and row pitch.  An operand that has neither (an inner dimension that is not a
    multiple of 8 elements, a slice that starts at an odd offset) is copied once into a buffer whose rows are padded
    to the next multiple of 8 elements; the returned view has the original shape, so the extent TMA sees is unchanged
    and reads past it are zero-filled.  (The reference keeps separate "unaligned" kernel variants for this:
    ``src/passes/matmul_pass.cpp:3542-3563``.)"""
    if t.data_ptr() % 16 == 0 and (t.stride(0) * t.element_size()) % 16 == 0:
        return t
    rows, cols = t.shape
    per = 16 // t.element_size()
    buf = torch.zeros(rows, (cols + per - 1) // per * per, dtype=t.dtype, device=t.device)
    buf[:, :cols] = t
    return buf[:, :cols]


def _t(x: torch.Tensor) -> torch.Tensor:
    return x.t().contiguous()


def gemm_nt(a, b, **kw):
    """``A (M,K) · B (N,K)ᵀ``."""
    return gemm(a, b, **kw)


def gemm_nn(a, b_kn, **kw):
    """``A (M,K) · B (K,N)``."""
    if USE_MN_MAJOR:
        return gemm(a, b_kn, b_mn=True, **kw)
    return gemm(a, _t(b_kn), **kw)


def gemm_tn(a_km, b_kn, **kw):
    """``A (K,M)ᵀ · B (K,N)`` — weight gradients."""
    if USE_MN_MAJOR:
        return gemm(a_km, b_kn, a_mn=True, b_mn=True, **kw)
    return gemm(_t(a_km), _t(b_kn), **kw)


def _colsum(x2d: torch.Tensor) -> torch.Tensor:
    out = torch.zeros(x2d.shape[1], dtype=torch.float32, device=x2d.device)
    nv.check(nv.lib(x2d).fbam_colsum(nv.ptr(x2d), nv.ptr(out), C.c_longlong(x2d.shape[0]), x2d.shape[1],
                                  nv.stream_ptr()), "fbam_colsum")
    return out


def _gelu_bwd(preact: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(dy)
    nv.check(nv.lib(preact).fbam_gelu(nv.ptr(preact), nv.ptr(dy), nv.ptr(out), C.c_longlong(dy.numel()), 1,
                                nv.stream_ptr()), "fbam_gelu")
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, act, residual=None):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        preact = None
        if act == "gelu" and (x.requires_grad or weight.requires_grad):
            preact = torch.empty((x2.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        res2 = None
        if residual is not None:            # added in the GEMM epilogue, after the activation
            res2 = residual.reshape(-1, weight.shape[0])
            if res2.stride(-1) != 1:
                res2 = res2.contiguous()
        y = gemm(x2, weight, bias=bias, act=act, preact_out=preact, residual=res2)
        if act == "relu":
            preact = y        # the output's sign is all the backward needs
        ctx.save_for_backward(x2, weight, preact)
        ctx.act, ctx.has_bias, ctx.in_shape = act, bias is not None, x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight, preact = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.act == "gelu":
            dy2 = _gelu_bwd(preact, dy2)
        elif ctx.act == "relu":
            dy2 = dy2 * (preact > 0)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm_nn(dy2, weight).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            n_out, n_in = dy2.shape[1], x2.shape[1]
            dw = gemm_tn(dy2, x2, splits=weight_grad_splits(n_out, n_in, dy2.shape[0]) if USE_MN_MAJOR else 0)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _colsum(dy2).to(dy2.dtype)
        d_res = dy if len(ctx.needs_input_grad) > 4 and ctx.needs_input_grad[4] else None
        return dx, dw, db, None, d_res


def linear(x, weight, bias=None, act="none", residual=None):
    _need_elem(x, weight, bias, residual)
    return _Linear.apply(x, weight, bias, act, residual)


# =================================================================================================
# convolution (implicit GEMM)
# =================================================================================================
def _brick(n: int, h: int, w: int, total: int = 128) -> Tuple[int, int, int]:
    """Splits the `total` rows of a tile into (tn, th, tw) positions with the least padding waste."""
    best, best_cost = (1, 1, total), None
    for tw in (1, 2, 4, 8, 16, 32, 64, 128):
        for th in (1, 2, 4, 8, 16, 32, 64, 128):
            if tw * th > total:
                continue
            tn = total // (tw * th)
            cost = (math.ceil(w / tw) * tw) * (math.ceil(h / th) * th) * (math.ceil(n / tn) * tn)
            # prefer wide bricks on ties: longer contiguous runs per TMA box row
            key = (cost, -tw, -th)
            if best_cost is None or key < best_cost:
                best, best_cost = (tn, th, tw), key
    return best


def conv_pass(x: torch.Tensor, wmat: torch.Tensor, n_out: int, out: torch.Tensor, *, grid_hw, in_mul, taps,
              out_mul=1, out_off=(0, 0), accumulate=0, bn: int = 0, act: str = "none",
              preact_out: Optional[torch.Tensor] = None, gelu_grad_in: Optional[torch.Tensor] = None,
              tile_rows: int = 0, two_cta=None, classes=None) -> None:
    """One implicit-GEMM pass (see ``ConvGeom`` in csrc/gemm_tcgen05.h).  ``x`` NHWC bf16 or fp16, ``wmat``
    ``(n_out, taps·C)`` of the same type, ``out`` NHWC with ``n_out`` channels.

    ``classes`` (CTA-pair kernel only): a list of ``(taps, out_off)`` — parity classes of a strided data gradient
    that share the iteration grid.  ``taps`` is then the concatenation of the classes' taps and ``wmat`` holds the
    classes' filter columns side by side in that order; every tile is computed once per class by the same CTA pair,
    so the input tile is read from DRAM once for all classes."""
    b, ih, iw, c = x.shape
    if classes is not None:
        two_cta, tile_rows, bn = True, 0, 0
    elif bn == 0 and tile_rows == 0 and two_cta is None:
        tuned = tuning.lookup(tuning.conv_key(b, grid_hw[0], grid_hw[1], c, n_out, len(taps), in_mul, out_mul),
                              {"batch": b, "in_h": ih, "in_w": iw, "c": c, "n_out": n_out, "grid_hw": list(grid_hw),
                               "in_mul": in_mul, "out_mul": out_mul, "taps": [list(t) for t in taps],
                               "out_off": list(out_off), "out_hw": [out.shape[1], out.shape[2]]})
        if tuned is not None:
            bn, tile_rows, two_cta = tuned.get("bn", 0), tuned.get("tile_rows", 0), tuned.get("two_cta")
    p = nv.GemmParams()
    g = p.conv
    g.batch, g.grid_h, g.grid_w = b, grid_hw[0], grid_hw[1]
    # 256-pixel bricks (two stacked M halves sharing each filter fetch) once there are enough tiles to fill
    # the machine twice; 128-pixel bricks otherwise
    tn, th, tw = _brick(b, grid_hw[0], grid_hw[1], 256)
    tiles256 = math.ceil(b / tn) * math.ceil(grid_hw[0] / th) * math.ceil(grid_hw[1] / tw)
    pair = TWO_CTA if two_cta is None else two_cta
    if pair == "auto":      # pairs pay off only with 256-wide tiles (a 128-wide pair tile fetches as much as one CTA)
        pair = tile_rows == 0 and n_out >= 256 and tiles256 >= 148
    if pair:
        tile_rows = 128          # each CTA of the pair owns one 128-pixel brick
    if tile_rows == 128 or n_out < 128 or (tile_rows == 0 and tiles256 < 2 * 148) or (tw - 1) * in_mul + 1 > 256 \
            or (th - 1) * in_mul + 1 > 256 or tn > 256:
        tn, th, tw = _brick(b, grid_hw[0], grid_hw[1], 128)
    g.tn, g.th, g.tw = tn, th, tw
    g.in_mul, g.out_mul = in_mul, out_mul
    g.out_off_h, g.out_off_w = out_off
    g.out_h, g.out_w = out.shape[1], out.shape[2]
    g.num_taps = len(taps)
    for i, (dh, dw) in enumerate(taps):
        g.tap_dh[i], g.tap_dw[i] = dh, dw
    if classes is not None:
        p.num_classes = len(classes)
        base = 0
        for k, (ctaps, coff) in enumerate(classes):
            cl = p.cls[k]
            cl.num_taps, cl.out_off_h, cl.out_off_w, cl.k_block_base = len(ctaps), coff[0], coff[1], base * (c // 64)
            for i, (dh, dw) in enumerate(ctaps):
                cl.tap_dh[i], cl.tap_dw[i] = dh, dw
            base += len(ctaps)
    p.D, p.ldd = out.data_ptr(), out.shape[3]
    p.status = nv.status_word(x.device).data_ptr()
    p.alpha = 1.0
    p.out_fp32 = int(out.dtype == torch.float32)
    p.accumulate = accumulate
    p.bn = bn
    p.act = nv.GEMM_ACT[act]
    if preact_out is not None:
        p.preact_out = preact_out.data_ptr()
    if gelu_grad_in is not None:
        p.gelu_grad_in = gelu_grad_in.data_ptr()
    fn = nv.lib(x).fbam_conv2 if pair else nv.lib(x).fbam_conv
    with debug.label(f"conv{'2' if pair else ''} c{c} n{n_out} taps{len(taps)} in_mul{in_mul} out_mul{out_mul} {act}"
                     + (f" classes{len(classes)}" if classes is not None else "")):
        code = fn(nv.ptr(x), ih, iw, c, nv.ptr(wmat), C.c_longlong(wmat.stride(0)), n_out, C.byref(p),
                  nv.stream_ptr())
    nv.check(code, "fbam_conv")
    flops.add(2.0 * b * grid_hw[0] * grid_hw[1] * n_out * len(taps) * c)
    debug.after_launch("conv_pass", x, wmat, out)


def conv2d_fprop(x, w_ohwi, stride, padding, dilation, act: str = "none", preact_out=None):
    b, ih, iw, c = x.shape
    o = w_ohwi.shape[0]
    oh = (ih + 2 * padding - 2 * dilation - 1) // stride + 1
    ow = (iw + 2 * padding - 2 * dilation - 1) // stride + 1
    out = debug.fresh((b, oh, ow, o), x.dtype, x.device)
    taps = [(r * dilation - padding, s * dilation - padding) for r in range(3) for s in range(3)]
    conv_pass(x, w_ohwi.reshape(o, 9 * c), o, out, grid_hw=(oh, ow), in_mul=stride, taps=taps, act=act,
              preact_out=preact_out)
    return out


def conv_out_hw(ih, iw, stride, padding, dilation):
    return ((ih + 2 * padding - 2 * dilation - 1) // stride + 1, (iw + 2 * padding - 2 * dilation - 1) // stride + 1)


def conv2d_dgrad(dy, w_ohwi, in_hw, stride, padding, dilation, gelu_grad_in=None):
    """dX[n, h, w, :] = Σ_taps dY[n, (h + pad − r·dil)/stride, (w + pad − s·dil)/stride, :] · W[:, r, s, :]
    over the taps for which the division is exact.  Output pixels are split into stride x stride
    parity classes; each class is one stride-1 gather over its own tap subset."""
    b, oh, ow, o = dy.shape
    c = w_ohwi.shape[3]
    ih, iw = in_hw
    dx = debug.fresh((b, ih, iw, c), dy.dtype, dy.device)
    parts = []                                  # (taps, filter matrix (C, taps·O), grid, output offset) per class
    for ph in range(stride):
        for pw in range(stride):
            taps, mats = [], []
            for r in range(3):
                if (ph + padding - r * dilation) % stride != 0:
                    continue
                for s in range(3):
                    if (pw + padding - s * dilation) % stride != 0:
                        continue
                    taps.append(((ph + padding - r * dilation) // stride, (pw + padding - s * dilation) // stride))
                    mats.append(w_ohwi[:, r, s, :])                       # (O, C)
            gh, gw = (ih - ph + stride - 1) // stride, (iw - pw + stride - 1) // stride
            if gh <= 0 or gw <= 0:
                continue
            if not taps:
                dx[:, ph::stride, pw::stride, :].zero_()
                continue
            # (gelu_grad_in multiplies every written element, so zero-tap classes stay zero)
            # filter matrix for this class: (C, taps·O), K ordered tap-major then output channel
            wmat = torch.stack(mats, 0).permute(2, 0, 1).reshape(c, len(taps) * o)
            parts.append((taps, wmat, (gh, gw), (ph, pw)))
    if _fuse_dgrad_classes(parts, b, c, stride):
        # all parity classes in one launch: a CTA pair runs the classes of a tile back to back, so the gradient tile
        # is streamed from DRAM once instead of once per class (heaviest class first: it touches every shifted tile)
        parts.sort(key=lambda part: -len(part[0]))
        wall = torch.cat([part[1] for part in parts], 1).contiguous()
        conv_pass(dy, wall, c, dx, grid_hw=parts[0][2], in_mul=1, taps=[t for part in parts for t in part[0]],
                  out_mul=stride, gelu_grad_in=gelu_grad_in, classes=[(part[0], part[3]) for part in parts])
        return dx
    for taps, wmat, grid, off in parts:
        conv_pass(dy, wmat.contiguous(), c, dx, grid_hw=grid, in_mul=1, taps=taps, out_mul=stride, out_off=off,
                  gelu_grad_in=gelu_grad_in)
    return dx


FUSE_DGRAD_CLASSES = True


def _fuse_dgrad_classes(parts, batch: int, n_out: int, stride: int) -> bool:
    """The fused form needs every class on the same grid with one to four taps, nine taps in all at most, and a
    problem that the CTA-pair kernel would be chosen for anyway."""
    if not FUSE_DGRAD_CLASSES or TWO_CTA is False or len(parts) < 2 or len(parts) > 4 or n_out < 256 or n_out % 16:
        return False
    if any(part[2] != parts[0][2] or not 1 <= len(part[0]) <= 4 for part in parts):
        return False
    if sum(len(part[0]) for part in parts) > 9:
        return False
    gh, gw = parts[0][2]
    tn, th, tw = _brick(batch, gh, gw, 256)
    return math.ceil(batch / tn) * math.ceil(gh / th) * math.ceil(gw / tw) >= 148


class _ConvGeluStackPool(torch.autograd.Function):
    """``[conv3x3 → GELU] x n → mean over positions`` with a hand-written backward in which every
    activation gradient rides in the epilogue of the kernel that produces its input gradient: GELU is the
    epilogue of each forward convolution (the pre-activation is stored alongside), the pool's backward
    multiplies by gelu'(z_last), and the data-gradient convolution of block i multiplies by gelu'(z_{i-1})."""

    @staticmethod
    def forward(ctx, x, stride, paddings, dilations, *weights):
        ys, zs = [x], []
        for w, pad, dil in zip(weights, paddings, dilations):
            oh, ow = conv_out_hw(ys[-1].shape[1], ys[-1].shape[2], stride, pad, dil)
            z = debug.fresh((x.shape[0], oh, ow, w.shape[0]), x.dtype, x.device)
            ys.append(conv2d_fprop(ys[-1], w, stride, pad, dil, act="gelu", preact_out=z))
            zs.append(z)
        last = ys[-1]
        n, h, wd, c = last.shape
        vec = torch.empty(n, c, dtype=last.dtype, device=x.device)
        nv.check(nv.lib(last).fbam_global_avgpool(nv.ptr(last), nv.ptr(vec), C.c_longlong(n), h * wd, c, 0, None,
                                              nv.stream_ptr()), "fbam_global_avgpool")
        ctx.save_for_backward(*ys[:-1], *zs, *weights)
        ctx.cfg = (stride, tuple(paddings), tuple(dilations), len(weights))
        return vec

    @staticmethod
    def backward(ctx, dvec):
        stride, paddings, dilations, nb = ctx.cfg
        saved = ctx.saved_tensors
        ys, zs, weights = saved[:nb], saved[nb:2 * nb], saved[2 * nb:]
        from .conv_wgrad import conv2d_wgrad
        z_last = zs[-1]
        n, h, wd, c = z_last.shape
        dz = torch.empty_like(z_last)
        nv.check(nv.lib(dvec).fbam_global_avgpool(nv.ptr(dvec.contiguous()), nv.ptr(dz), C.c_longlong(n), h * wd, c, 1,
                                              nv.ptr(z_last), nv.stream_ptr()), "fbam_global_avgpool")
        dws = [None] * nb
        for i in range(nb - 1, -1, -1):
            x_in, w = ys[i], weights[i]
            if ctx.needs_input_grad[4 + i]:
                dws[i] = conv2d_wgrad(x_in, dz, w.shape, stride, paddings[i], dilations[i])
            if i > 0 or ctx.needs_input_grad[0]:
                dz = conv2d_dgrad(dz, w, (x_in.shape[1], x_in.shape[2]), stride, paddings[i], dilations[i],
                                  gelu_grad_in=zs[i - 1] if i > 0 else None)
        dx = dz if ctx.needs_input_grad[0] else None
        return (dx, None, None, None, *dws)


class _CellConvGeluStackPool(torch.autograd.Function):
    """``cells → cell embedding → [conv3x3 → GELU] x n → mean over positions`` where the embedding and the first
    convolution are one table look-up (``ops/embconv.py``): the embedding tensor, the first layer's data gradient and
    the scatter of that gradient into the tables never exist.  Layers 2..n run as in :class:`_ConvGeluStackPool`; the
    data-gradient convolution of layer 2 delivers ``dZ₁`` (its epilogue multiplies by gelu'(z₁)), which three
    reductions turn into the gradients of the tables and of the first filter."""

    @staticmethod
    def forward(ctx, cells, cp_embed, pos_embed, colour, rows, cols, stride, paddings, dilations, *weights):
        from . import embconv
        cells = cells.contiguous()
        y1, z1, feat = embconv.first_layer_forward_native(cells, cp_embed, pos_embed, colour, weights[0], rows, cols,
                                                          stride, paddings[0], dilations[0])
        ys, zs = [y1], [z1]
        for w, pad, dil in zip(weights[1:], paddings[1:], dilations[1:]):
            oh, ow = conv_out_hw(ys[-1].shape[1], ys[-1].shape[2], stride, pad, dil)
            z = debug.fresh((cells.shape[0], oh, ow, w.shape[0]), y1.dtype, cells.device)
            ys.append(conv2d_fprop(ys[-1], w, stride, pad, dil, act="gelu", preact_out=z))
            zs.append(z)
        last = ys[-1]
        n, h, wd, c = last.shape
        vec = torch.empty(n, c, dtype=last.dtype, device=cells.device)
        nv.check(nv.lib(last).fbam_global_avgpool(nv.ptr(last), nv.ptr(vec), C.c_longlong(n), h * wd, c, 0, None,
                                              nv.stream_ptr()), "fbam_global_avgpool")
        ctx.save_for_backward(cells, feat, cp_embed, pos_embed, colour, *ys[:-1], *zs, *weights)
        ctx.cfg = (rows, cols, stride, tuple(paddings), tuple(dilations), len(weights))
        return vec

    @staticmethod
    def backward(ctx, dvec):
        from . import embconv
        from .conv_wgrad import conv2d_wgrad
        rows, cols, stride, paddings, dilations, nb = ctx.cfg
        saved = ctx.saved_tensors
        cells, feat, cp_embed, pos_embed, colour = saved[:5]
        rest = saved[5:]
        ys, zs, weights = rest[:nb - 1], rest[nb - 1:2 * nb - 1], rest[2 * nb - 1:]     # ys[i] = input of layer i + 1
        z_last = zs[-1]
        n, h, wd, c = z_last.shape
        dz = torch.empty_like(z_last)
        nv.check(nv.lib(dvec).fbam_global_avgpool(nv.ptr(dvec.contiguous()), nv.ptr(dz), C.c_longlong(n), h * wd, c, 1,
                                              nv.ptr(z_last), nv.stream_ptr()), "fbam_global_avgpool")
        dws = [None] * nb
        for i in range(nb - 1, 0, -1):
            x_in, w = ys[i - 1], weights[i]
            if ctx.needs_input_grad[9 + i]:
                dws[i] = conv2d_wgrad(x_in, dz, w.shape, stride, paddings[i], dilations[i])
            dz = conv2d_dgrad(dz, w, (x_in.shape[1], x_in.shape[2]), stride, paddings[i], dilations[i],
                              gelu_grad_in=zs[i - 1])
        d_cp, d_pos, d_col, dws[0] = embconv.first_layer_backward_native(
            cells, feat, dz, cp_embed, pos_embed, colour, weights[0], rows, cols, stride, paddings[0], dilations[0])
        return (None, d_cp.to(cp_embed.dtype), d_pos.to(pos_embed.dtype), d_col.to(colour.dtype), None, None, None, None,
                None, *dws)


def cell_conv_gelu_stack_pool(cells, cp_embed, pos_embed, colour, rows, cols, weights, stride, paddings, dilations):
    _need_elem(*weights)
    return _CellConvGeluStackPool.apply(cells, cp_embed, pos_embed, colour, rows, cols, stride, tuple(paddings),
                                        tuple(dilations), *weights)


def conv_gelu_stack_pool(x, weights, stride, paddings, dilations):
    _need_elem(x, *weights)
    return _ConvGeluStackPool.apply(x.contiguous(), stride, tuple(paddings), tuple(dilations), *weights)


class _Conv2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, stride, padding, dilation):
        ctx.save_for_backward(x, w)
        ctx.cfg = (stride, padding, dilation)
        return conv2d_fprop(x, w, stride, padding, dilation)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        stride, padding, dilation = ctx.cfg
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            if dy.shape[3] % 64 == 0:
                dx = conv2d_dgrad(dy, w, (x.shape[1], x.shape[2]), stride, padding, dilation)
            else:
                dx = torch.nn.grad.conv2d_input(x.permute(0, 3, 1, 2).shape, w.permute(0, 3, 1, 2),
                                                dy.permute(0, 3, 1, 2), stride, padding, dilation).permute(0, 2, 3, 1).contiguous()
        if ctx.needs_input_grad[1]:
            from .conv_wgrad import conv2d_wgrad
            dw = conv2d_wgrad(x, dy, w.shape, stride, padding, dilation)
        return dx, dw, None, None, None


def conv2d_nhwc(x, w_ohwi, stride, padding, dilation):
    _need_elem(x, w_ohwi)
    if x.shape[3] % 64 != 0:
        raise ValueError("native convolution needs input channels in multiples of 64")
    return _Conv2d.apply(x.contiguous(), w_ohwi, stride, padding, dilation)


# =================================================================================================
# normalisation / activations / pooling
# =================================================================================================
class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        nv.check(nv.lib(x2).fbam_rmsnorm_fwd(nv.ptr(x2), nv.ptr(weight), nv.ptr(y), nv.ptr(rstd),
                                           C.c_longlong(x2.shape[0]), x2.shape[1], C.c_float(eps), nv.stream_ptr()),
                 "fbam_rmsnorm_fwd")
        ctx.save_for_backward(x2, weight, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, rstd = ctx.saved_tensors
        dy2 = dy.reshape(x2.shape).contiguous()
        dx = torch.empty_like(x2)
        dg = torch.zeros(x2.shape[1], dtype=torch.float32, device=x2.device)
        nv.check(nv.lib(dy2).fbam_rmsnorm_bwd(nv.ptr(dy2), nv.ptr(x2), nv.ptr(weight), nv.ptr(rstd), nv.ptr(dx), nv.ptr(dg),
                                           C.c_longlong(x2.shape[0]), x2.shape[1], nv.stream_ptr()), "fbam_rmsnorm_bwd")
        return dx.view(dy.shape), dg.to(weight.dtype), None


def rms_norm(x, weight, eps):
    _need_elem(x, weight)
    return _RmsNorm.apply(x, weight, eps)


class _LayerNorm(torch.autograd.Function):
    """LayerNorm with a native backward (the reference ships the forward only: ``tensorlib/include/layer_norm.h:12-78``)."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        rows, dim = x2.shape
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        nv.check(nv.lib(x2).fbam_layernorm_fwd_stats(nv.ptr(x2), nv.ptr(weight), nv.ptr(bias), nv.ptr(y), nv.ptr(mean),
                                                   nv.ptr(rstd), C.c_longlong(rows), dim, C.c_float(eps),
                                                   nv.stream_ptr()), "fbam_layernorm_fwd_stats")
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.has_bias = bias is not None
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, dim = x2.shape
        dy2 = dy.reshape(rows, dim).contiguous()
        dx = torch.empty_like(x2)
        dw = torch.zeros(dim, dtype=torch.float32, device=x2.device)
        db = torch.zeros(dim, dtype=torch.float32, device=x2.device) if ctx.has_bias else None
        nv.check(nv.lib(dy2).fbam_layernorm_bwd(nv.ptr(dy2), nv.ptr(x2), nv.ptr(weight), nv.ptr(mean), nv.ptr(rstd),
                                             nv.ptr(dx), nv.ptr(dw), nv.ptr(db), C.c_longlong(rows), dim,
                                             nv.stream_ptr()), "fbam_layernorm_bwd")
        return dx.view(dy.shape), dw.to(weight.dtype), (db.to(weight.dtype) if db is not None else None), None


def layer_norm(x, weight, bias, eps):
    _need_elem(x, weight, bias)
    if x.shape[-1] > 8192:
        raise ValueError("native LayerNorm handles rows of up to 8192 elements")
    return _LayerNorm.apply(x, weight, bias, eps)


class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        y = torch.empty_like(x)
        nv.check(nv.lib(x).fbam_gelu(nv.ptr(x), None, nv.ptr(y), C.c_longlong(x.numel()), 0, nv.stream_ptr()), "fbam_gelu")
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return _gelu_bwd(x, dy.contiguous())


def gelu(x):
    _need_elem(x)
    return _Gelu.apply(x)


class _Geglu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        c = x.shape[-1] // 2
        rows = x.numel() // (2 * c)
        y = torch.empty(*x.shape[:-1], c, dtype=x.dtype, device=x.device)
        nv.check(nv.lib(x).fbam_geglu(nv.ptr(x), None, nv.ptr(y), C.c_longlong(rows), c, 0, nv.stream_ptr()), "fbam_geglu")
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        c = x.shape[-1] // 2
        dx = torch.empty_like(x)
        nv.check(nv.lib(x).fbam_geglu(nv.ptr(x), nv.ptr(dy.contiguous()), nv.ptr(dx), C.c_longlong(x.numel() // (2 * c)),
                                     c, 1, nv.stream_ptr()), "fbam_geglu")
        return dx


def geglu(x):
    _need_elem(x)
    return _Geglu.apply(x)


class _AvgPool2x2(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        n, h, w, c = x.shape
        y = torch.empty(n, h // 2, w // 2, c, dtype=x.dtype, device=x.device)
        nv.check(nv.lib(x).fbam_avgpool2x2(nv.ptr(x.contiguous()), nv.ptr(y), C.c_longlong(n), h // 2, w // 2, c, 0,
                                          nv.stream_ptr()), "fbam_avgpool2x2")
        ctx.shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        n, h, w, c = ctx.shape
        dx = torch.zeros(ctx.shape, dtype=dy.dtype, device=dy.device) if (h % 2 or w % 2) else \
            torch.empty(ctx.shape, dtype=dy.dtype, device=dy.device)
        nv.check(nv.lib(dy).fbam_avgpool2x2(nv.ptr(dy.contiguous()), nv.ptr(dx), C.c_longlong(n), h // 2, w // 2, c, 1,
                                          nv.stream_ptr()), "fbam_avgpool2x2")
        return dx


def avg_pool2x2_nhwc(x):
    _need_elem(x)
    if x.shape[1] % 2 or x.shape[2] % 2:
        raise ValueError("2x2 pooling needs even height and width")
    return _AvgPool2x2.apply(x)


class _GlobalAvgPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        n, h, w, c = x.shape
        y = torch.empty(n, c, dtype=x.dtype, device=x.device)
        nv.check(nv.lib(x).fbam_global_avgpool(nv.ptr(x.contiguous()), nv.ptr(y), C.c_longlong(n), h * w, c, 0, None,
                                              nv.stream_ptr()), "fbam_global_avgpool")
        ctx.shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        n, h, w, c = ctx.shape
        dx = torch.empty(ctx.shape, dtype=dy.dtype, device=dy.device)
        nv.check(nv.lib(dy).fbam_global_avgpool(nv.ptr(dy.contiguous()), nv.ptr(dx), C.c_longlong(n), h * w, c, 1, None,
                                              nv.stream_ptr()), "fbam_global_avgpool")
        return dx


def global_avg_pool_nhwc(x):
    _need_elem(x)
    return _GlobalAvgPool.apply(x)


# =================================================================================================
# cell embedding
# =================================================================================================
class _CellEmbed(torch.autograd.Function):
    @staticmethod
    def forward(ctx, cells, cp_embed, pos_embed, colour, out_dtype):
        n, p, _ = cells.shape
        e = cp_embed.shape[1]
        cells = cells.contiguous()
        out = debug.fresh((n, p, e), out_dtype, cells.device)
        nv.check(nv.lib(out_dtype).fbam_cell_embed_fwd(nv.ptr(cells), nv.ptr(cp_embed), nv.ptr(pos_embed), nv.ptr(colour),
                                              nv.ptr(out), C.c_longlong(n), p, e, cp_embed.shape[0],
                                              nv.stream_ptr()), "fbam_cell_embed_fwd")
        ctx.save_for_backward(cells)
        ctx.dims = (n, p, e, cp_embed.shape[0])
        return out

    @staticmethod
    def backward(ctx, dout):
        (cells,) = ctx.saved_tensors
        n, p, e, vocab = ctx.dims
        d_cp = torch.zeros(vocab, e, dtype=torch.float32, device=dout.device)
        d_pos = torch.zeros(p, e, dtype=torch.float32, device=dout.device)
        d_col = torch.zeros(6, e, dtype=torch.float32, device=dout.device)
        nv.check(nv.lib(dout).fbam_cell_embed_bwd(nv.ptr(cells), nv.ptr(dout.contiguous()), nv.ptr(d_cp), nv.ptr(d_pos),
                                              nv.ptr(d_col), C.c_longlong(n), p, e, vocab, nv.stream_ptr()),
                 "fbam_cell_embed_bwd")
        return None, d_cp, d_pos, d_col, None


def cell_embed(cells, cp_embed, pos_embed, colour, out_dtype):
    if out_dtype not in nv.ELEM_DTYPES:
        raise TypeError("native cell embedding writes bf16 or fp16")
    if pos_embed.shape[0] != cells.shape[1]:
        raise ValueError("position table must have one row per cell")
    return _CellEmbed.apply(cells, cp_embed.float(), pos_embed.float(), colour.float(), out_dtype)


# =================================================================================================
# LM head + cross-entropy: chunked over rows, logits reduced inside the GEMM epilogue (reference materialises them:
# src/main_action_model.cpp:156-175)
# =================================================================================================
LM_HEAD_CHUNK_ROWS = 4096
# True: cross-entropy statistics and gradient come out of the head GEMM's epilogue (no fp32 logits in HBM);
# False: the GEMM writes a chunk of fp32 logits and a row-wise kernel reads them back.
FUSED_LM_HEAD_CE = True


class _LmHeadCe(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_head, targets, vocab, scale):
        rows, h = x.shape
        vpad = w_head.shape[0]
        loss = torch.zeros(1, dtype=torch.float32, device=x.device)
        need_grad = x.requires_grad or w_head.requires_grad
        dx = torch.empty_like(x) if need_grad else None
        dw = torch.zeros(vpad, h, dtype=torch.float32, device=x.device) if need_grad else None
        targets = targets.contiguous()
        for lo in range(0, rows, LM_HEAD_CHUNK_ROWS):
            hi = min(rows, lo + LM_HEAD_CHUNK_ROWS)
            xc = x[lo:hi]
            n = hi - lo
            tg = targets[lo:hi]
            if FUSED_LM_HEAD_CE:
                # The logits never reach HBM: the head GEMM's epilogue reduces each 128 x 128 tile half, still in
                # tensor memory, to per-row (maximum, sum of exp) pairs and picks out the target logit; a small
                # kernel merges the pairs into the rows' log-sum-exp and the loss; for the backward the same GEMM
                # runs again and its epilogue turns the accumulators straight into 16-bit scale·(softmax − onehot).
                slots = 2 * ((vpad + 255) // 256)
                partial = torch.empty(n, slots, 2, dtype=torch.float32, device=x.device)
                tgt_logit = torch.zeros(n, dtype=torch.float32, device=x.device)      # targets outside the table: 0
                lse = torch.empty(n, dtype=torch.float32, device=x.device)
                gemm(xc, w_head, ce_stats=(partial, tgt_logit, tg, vocab))
                nv.check(nv.lib(partial).fbam_ce_combine(nv.ptr(partial), nv.ptr(tgt_logit), nv.ptr(lse), nv.ptr(loss),
                                                  C.c_longlong(n), slots, C.c_float(scale), nv.stream_ptr()),
                         "fbam_ce_combine")
                dlogits = None
                if need_grad:
                    dlogits = torch.empty(n, vpad, dtype=x.dtype, device=x.device)
                    with flops.not_useful():                             # the logits are computed a second time
                        gemm(xc, w_head, out=dlogits, ce_grad=(lse, tg, vocab, scale))
            else:
                logits = gemm(xc, w_head, out_dtype=torch.float32)       # (chunk, vpad) fp32 accumulators
                dlogits = torch.empty(n, vpad, dtype=x.dtype, device=x.device) if need_grad else None
                nv.check(nv.lib(x).fbam_ce_fwd_bwd_f32(nv.ptr(logits), nv.ptr(dlogits), nv.ptr(tg), nv.ptr(loss),
                                                      C.c_longlong(n), vocab, vpad, C.c_float(scale),
                                                      nv.stream_ptr()), "fbam_ce_fwd_bwd_f32")
            if need_grad:                                                # dlogits = scale·(softmax − onehot)
                gemm_nn(dlogits, w_head, out=dx[lo:hi])
                gemm_tn(dlogits, xc, out=dw, accumulate=nv.GEMM_ACC_RMW)
        ctx.save_for_backward(dx, dw)
        return loss.reshape(())

    @staticmethod
    def backward(ctx, dloss):
        dx, dw = ctx.saved_tensors
        return (dx * dloss.to(dx.dtype)), (dw * dloss).to(dx.dtype), None, None, None


def lm_head_ce(x, w_head, targets, vocab, scale):
    _need_elem(x, w_head)
    return _LmHeadCe.apply(x.contiguous(), w_head, targets, vocab, scale)


# =================================================================================================
# fused AdamW on a flat range
# =================================================================================================
def adamw_flat(param, grad, m, v, master, lo, hi, lr, b1, b2, eps, wd, bc1, bc2, grad_scale=1.0):
    n = hi - lo
    if n <= 0:
        return
    is_elem = param.dtype in nv.ELEM_DTYPES
    if not is_elem and param.dtype != torch.float32:
        raise TypeError("fused AdamW handles bf16, fp16 and fp32 parameters")
    if grad.dtype != param.dtype:
        raise TypeError("fused AdamW needs gradients of the parameters' type")
    nv.check(nv.lib(param).fbam_adamw(nv.ptr(param[lo:hi]), nv.ptr(grad[lo:hi]), nv.ptr(m[lo:hi]), nv.ptr(v[lo:hi]),
                                 nv.ptr(None if master is None else master[lo:hi]), C.c_longlong(n), int(is_elem),
                                 C.c_float(lr), C.c_float(b1), C.c_float(b2), C.c_float(eps), C.c_float(wd),
                                 C.c_float(bc1), C.c_float(bc2), C.c_float(grad_scale), nv.stream_ptr()), "fbam_adamw")


# =================================================================================================
# Newton–Schulz orthogonalisation on the tensor-core GEMM (Muon)
# =================================================================================================
NS_A, NS_B, NS_C = 3.4445, -4.7750, 2.0315


def newton_schulz(g: torch.Tensor, steps: int = 5, dtype: torch.dtype = BF16, norm: Optional[torch.Tensor] = None
                  ) -> torch.Tensor:
    """Five (by default) iterations of ``A = X Xᵀ; B = b·A + c·A A; X = a·X + B X`` in bf16, every product on the
    tcgen05 GEMM with the affine terms folded into its epilogue (``alpha`` and the residual input).  ``norm`` may
    carry a precomputed Frobenius norm (the fused gradient pull produces Σx² on the way)."""
    x = g.to(BF16)
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t().contiguous()
    if x.shape[1] % 8 != 0 or x.shape[0] % 8 != 0:
        from ..optim.muon import newton_schulz as ns_ref
        return ns_ref(g, steps, dtype)
    nrm = x.float().norm() if norm is None else norm
    x = (x.float() / (nrm + 1e-7)).to(BF16).contiguous()
    for _ in range(steps):
        a = gemm(x, x)                                            # X Xᵀ           (r x r)
        b = gemm(a, a, alpha=NS_C, residual=(a * NS_B))           # c·A A + b·A   (A is symmetric: A Aᵀ = A A)
        x = gemm(b, x, b_mn=True, residual=(x * NS_A))            # B X + a·X
    return (x.t() if transposed else x).to(dtype)


# =================================================================================================
# attention and LSTM sequence
# =================================================================================================
def attention(q, k, v, causal):
    from .mha import flash_attention
    return flash_attention(q, k, v, causal)


def lstm_sequence(x, w_ih, w_hh, b_ih, b_hh, h0, c0, compute_dtype):
    from .lstm import lstm_sequence as f
    return f(x, w_ih, w_hh, b_ih, b_hh, h0, c0, compute_dtype)
