"""Cell embedding fused with the first convolution of the frame head (no embedding tensor in memory).

The cell embedding is linear in its tables and a convolution without a normalisation in front of it is linear in
its input, so with ``W`` the ``(O, 3, 3, C)`` filter the pre-activation of the first convolution is

    Z[n, p] = Σ_tap T[cp(n, cell(p, tap)), tap] + POS[p] + F[n, p] · CC

with ``T[v, tap] = cp_embed[v] · W[:, tap]ᵀ`` (``(V, 9, O)``), ``POS`` the convolution of the position table
(one frame), ``F[n, p, tap·6 + c] = rgb_c(cell(p, tap)) / 255`` the colour features of the nine cells under the
filter and ``CC[tap·6 + c] = colour[c] · W[:, tap]ᵀ``.  The backward needs three reductions of ``dZ`` only:

    S[v, tap] = Σ dZ[n, p] over the (n, p) whose tap shows code point v          → d cp_embed, and dW through cp_embed
    D[p]      = Σ_n dZ[n, p]                                                     → d pos_embed, and dW through it
    Q         = Fᵀ · dZ                                                          → d colour, and dW through colour

and a few table-sized products.  The ``(frames × cells × C)`` embedding, the data-gradient convolution into it
and its scatter into the tables (reference: ``kernel_gen/kernel_gen/kernels/build_cell_embeds.py:74-134``,
``build_cell_embeds_bwd.py:6-322``, ``conv2d.py``, ``conv2d_bwd.py``; model structure
``src/framehead_model.cpp:601-731``) are never computed.  The six colour vectors are handled as six extra rows of
the code-point table whose "one-hot" weights are the colour features, so one product per direction covers both.

``first_layer_forward`` / ``first_layer_backward`` have a native form (kernels of ``csrc/embconv.cu`` plus the
tcgen05 GEMM / convolution entry points) and a plain-PyTorch form with the same decomposition, which is the CPU
path and what the tests compare the kernels with.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

FEATURES = 64          # colour features per output pixel: 9 taps x 6 channels, padded to one 128-byte bf16 row
SEGMENT_FRAMES = 128   # consecutive frames one warp walks (run-length state is rebuilt at every segment start)
MAX_TABLE_BYTES = 256 * 1024 * 1024

_tap_cache: Dict[Tuple, torch.Tensor] = {}


def out_hw(rows: int, cols: int, stride: int, pad: int, dil: int) -> Tuple[int, int]:
    return (rows + 2 * pad - 2 * dil - 1) // stride + 1, (cols + 2 * pad - 2 * dil - 1) // stride + 1


def tap_cells(rows: int, cols: int, stride: int, pad: int, dil: int, device) -> torch.Tensor:
    """``(P_out, 9)`` int64: the cell (row-major index within the frame) that output pixel ``p`` reads through filter
    tap ``r·3 + s``, or −1 where the tap falls into the padding."""
    key = (rows, cols, stride, pad, dil, str(device))
    if key not in _tap_cache:
        oh, ow = out_hw(rows, cols, stride, pad, dil)
        oy = torch.arange(oh).view(oh, 1, 1, 1)
        ox = torch.arange(ow).view(1, ow, 1, 1)
        r = torch.arange(3).view(1, 1, 3, 1)
        s = torch.arange(3).view(1, 1, 1, 3)
        iy = oy * stride + r * dil - pad
        ix = ox * stride + s * dil - pad
        ok = (iy >= 0) & (iy < rows) & (ix >= 0) & (ix < cols)
        idx = torch.where(ok, iy * cols + ix, torch.full_like(iy * cols + ix, -1))
        _tap_cache[key] = idx.reshape(oh * ow, 9).to(device)
    return _tap_cache[key]


def supported(cells: torch.Tensor, cp_embed: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the native kernels take this first layer: input channels in whole 64-wide K blocks, output channels in
    whole 64-wide GEMM panels, and a code-point table small enough for the (V, 9, O) product table."""
    o, kh, kw, c = w.shape
    return (kh == 3 and kw == 3 and c % 64 == 0 and o % 64 == 0 and cells.dtype == torch.int32 and
            (cp_embed.shape[0] + 8) * 9 * o * 4 <= MAX_TABLE_BYTES)


# =================================================================================================
# plain-PyTorch forms of the three kernels
# =================================================================================================
def _tap_codepoints(cells: torch.Tensor, taps: torch.Tensor, vocab: int):
    """Code point under every (pixel, tap): ``(N, P_out, 9)`` int64 and its validity (inside the frame and the table)."""
    cp = cells[..., 0].long()
    idx = taps.clamp(min=0)
    cpt = cp[:, idx]                                           # (N, P_out, 9)
    ok = (taps >= 0).unsqueeze(0) & (cpt >= 0) & (cpt < vocab)
    return cpt.clamp(0, vocab - 1), ok


def features_torch(cells: torch.Tensor, taps: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    n = cells.shape[0]
    fg, bg = cells[..., 1].long(), cells[..., 2].long()
    chans = torch.stack([(fg >> 16) & 255, (fg >> 8) & 255, fg & 255,
                         (bg >> 16) & 255, (bg >> 8) & 255, bg & 255], dim=-1).float() / 255.0     # (N, P, 6)
    f = chans[:, taps.clamp(min=0)] * (taps >= 0).view(1, -1, 9, 1)                                # (N, P_out, 9, 6)
    out = torch.zeros(n, taps.shape[0], FEATURES, dtype=dtype, device=cells.device)
    out[..., :54] = f.reshape(n, taps.shape[0], 54).to(dtype)
    return out


def gather_torch(cells: torch.Tensor, taps: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """``Σ_tap table[cp, tap]`` per (frame, pixel): ``(N, P_out, O)`` fp32."""
    vocab = table.shape[0]
    cpt, ok = _tap_codepoints(cells, taps, vocab)
    out = torch.zeros(cells.shape[0], taps.shape[0], table.shape[2], dtype=torch.float32, device=cells.device)
    for t in range(9):
        out += table[cpt[..., t], t].float() * ok[..., t].unsqueeze(-1)
    return out


def reduce_torch(cells: torch.Tensor, taps: torch.Tensor, dz: torch.Tensor, vocab: int):
    """``S (V, 9, O)`` and ``D (P_out, O)`` in fp32 from ``dz (N, P_out, O)``."""
    n, p_out, o = dz.shape
    dzf = dz.float()
    cpt, ok = _tap_codepoints(cells, taps, vocab)
    s = torch.zeros(vocab, 9, o, dtype=torch.float32, device=dz.device)
    for t in range(9):
        s[:, t].index_add_(0, cpt[..., t].reshape(-1), (dzf * ok[..., t].unsqueeze(-1)).reshape(-1, o))
    return s, dzf.sum(0)


# =================================================================================================
# native launchers
# =================================================================================================
def _geom_args(rows, cols, stride, pad, dil):
    oh, ow = out_hw(rows, cols, stride, pad, dil)
    return rows, cols, oh, ow, stride, pad, dil


def features_native(cells: torch.Tensor, rows: int, cols: int, stride: int, pad: int, dil: int,
                    dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    from . import native as nv
    oh, ow = out_hw(rows, cols, stride, pad, dil)
    n = cells.shape[0]
    out = torch.empty(n, oh * ow, FEATURES, dtype=dtype, device=cells.device)
    nv.check(nv.lib(dtype).fbam_embconv_features(nv.ptr(cells), nv.ptr(out), C.c_longlong(n),
                                            *_geom_args(rows, cols, stride, pad, dil), nv.stream_ptr()),
             "fbam_embconv_features")
    return out


def forward_native(cells, table, pos, z, y, rows, cols, stride, pad, dil, z_has_input=True, apply_gelu=True,
                   seg_len: int = SEGMENT_FRAMES) -> None:
    """``z (N, P_out, O)`` bf16 holds the colour term on entry (when ``z_has_input``) and the pre-activation on
    return; ``y`` receives ``GELU(z)``."""
    from . import native as nv
    vocab, _, o = table.shape
    nv.check(nv.lib(table).fbam_embconv_fwd(nv.ptr(cells), nv.ptr(table), nv.ptr(pos), nv.ptr(z), nv.ptr(y),
                                       C.c_longlong(cells.shape[0]), vocab, o, *_geom_args(rows, cols, stride, pad, dil),
                                       seg_len, int(z_has_input), int(apply_gelu), nv.stream_ptr()),
             "fbam_embconv_fwd")


def reduce_native(cells, dz, s, d, rows, cols, stride, pad, dil, seg_len: int = SEGMENT_FRAMES) -> None:
    """Adds into ``s`` (fp32, at least ``(V, 9, O)``; rows past ``vocab`` are left alone) and ``d`` (fp32 ``(P_out, O)``)."""
    from . import native as nv
    o = dz.shape[-1]
    nv.check(nv.lib(dz).fbam_embconv_bwd_reduce(nv.ptr(cells), nv.ptr(dz), nv.ptr(s), nv.ptr(d),
                                              C.c_longlong(cells.shape[0]), s.shape[0], o,
                                              *_geom_args(rows, cols, stride, pad, dil), seg_len, nv.stream_ptr()),
             "fbam_embconv_bwd_reduce")


# =================================================================================================
# tables
# =================================================================================================
_table_cache: Dict[int, Tuple] = {}
_cache_token: Optional[int] = None


def set_cache_token(token: Optional[int]) -> None:
    """The product tables depend on parameters only.  A trainer sets a token that changes whenever parameters may
    have changed (once per optimizer step); calls with the same token reuse the tables.  ``None`` (the default)
    rebuilds them on every call."""
    global _cache_token
    if token != _cache_token:
        _table_cache.clear()
    _cache_token = token


def _tables_native(cp_embed, pos_embed, colour, w, rows, cols, stride, pad, dil):
    """→ ``ext`` bf16 ``(V + 6, C)`` (code-point rows then the six colour vectors), ``w_p`` bf16 ``(9·O, C)`` (filter
    rows ordered tap-major), ``table`` bf16 ``(V, 9, O)``, ``cc_t`` bf16 ``(O, 64)``, ``pos_out`` fp32 ``(P_out, O)``,
    ``pos_img`` bf16 ``(1, rows, cols, C)``."""
    from . import native_ops as no
    key = (cp_embed.data_ptr(), pos_embed.data_ptr(), colour.data_ptr(), w.data_ptr(), rows, cols, stride, pad, dil)
    if _cache_token is not None and key in _table_cache:
        return _table_cache[key]
    o, _, _, c = w.shape
    v = cp_embed.shape[0]
    bf = w.dtype                                                      # the 16-bit type of the filter: bf16 or fp16
    ext = torch.cat([cp_embed, colour], 0).to(bf)
    w_p = w.permute(1, 2, 0, 3).reshape(9 * o, c).contiguous()
    prod = no.gemm(ext, w_p)                                          # (V + 6, 9·O)
    table = prod[:v].view(v, 9, o)
    cc_t = torch.zeros(o, FEATURES, dtype=bf, device=w.device)
    cc_t[:, :54] = prod[v:v + 6].view(6, 9, o).permute(2, 1, 0).reshape(o, 54)
    pos_img = pos_embed.to(bf).view(1, rows, cols, c)
    oh, ow = out_hw(rows, cols, stride, pad, dil)
    pos_out = torch.empty(1, oh, ow, o, dtype=torch.float32, device=w.device)
    taps = [(r * dil - pad, s * dil - pad) for r in range(3) for s in range(3)]
    no.conv_pass(pos_img, w.reshape(o, 9 * c), o, pos_out, grid_hw=(oh, ow), in_mul=stride, taps=taps)
    result = (ext, w_p, table, cc_t, pos_out.view(oh * ow, o), pos_img)
    if _cache_token is not None:
        _table_cache[key] = result
    return result


# =================================================================================================
# first layer, forward and backward
# =================================================================================================
def first_layer_forward_native(cells, cp_embed, pos_embed, colour, w, rows, cols, stride, pad, dil):
    """→ ``y = GELU(z)``, ``z`` (both bf16 ``(N, OH, OW, O)``) and the colour features kept for the backward."""
    from . import native_ops as no
    o = w.shape[0]
    n = cells.shape[0]
    oh, ow = out_hw(rows, cols, stride, pad, dil)
    _ext, _w_p, table, cc_t, pos_out, _pos_img = _tables_native(cp_embed, pos_embed, colour, w, rows, cols, stride, pad, dil)
    feat = features_native(cells, rows, cols, stride, pad, dil, w.dtype)
    # colour term: K = 64 makes this GEMM all epilogue; the CTA-pair kernel writes its tiles with TMA stores
    z = no.gemm(feat.view(n * oh * ow, FEATURES), cc_t, two_cta=True)
    y = torch.empty_like(z)
    forward_native(cells, table, pos_out, z, y, rows, cols, stride, pad, dil)
    return y.view(n, oh, ow, o), z.view(n, oh, ow, o), feat


def first_layer_backward_native(cells, feat, dz, cp_embed, pos_embed, colour, w, rows, cols, stride, pad, dil):
    """``dz`` bf16 ``(N, OH, OW, O)`` → gradients of the code-point table, the position table, the colour vectors
    (fp32) and the filter (bf16)."""
    from . import native_ops as no
    from .conv_wgrad import conv2d_wgrad, wgrad_pass
    o, _, _, c = w.shape
    v = cp_embed.shape[0]
    n = cells.shape[0]
    oh, ow = out_hw(rows, cols, stride, pad, dil)
    bf = w.dtype
    ext, w_p, _table, _cc_t, _pos_out, pos_img = _tables_native(cp_embed, pos_embed, colour, w, rows, cols, stride, pad, dil)
    dz = dz.contiguous()
    s = torch.zeros(v + 6, 9, o, dtype=torch.float32, device=dz.device)
    d = torch.zeros(oh * ow, o, dtype=torch.float32, device=dz.device)
    reduce_native(cells, dz.view(n, oh * ow, o), s[:v], d, rows, cols, stride, pad, dil)
    # colour-weighted sums on the tensor cores: a 1x1 "weight gradient" with the features as the input image
    q = wgrad_pass(feat.view(n, oh, ow, FEATURES), dz, o, FEATURES, [(0, 0)], 1, out_dtype=torch.float32)   # (O, 64)
    s[v:] = q[:, :54].view(o, 9, 6).permute(2, 1, 0)
    s_b = s.to(bf).view(v + 6, 9 * o)
    d_ext = no.gemm(s_b, w_p, b_mn=True, out_dtype=torch.float32)                      # (V + 6, C)
    dw_tab = no.gemm(s_b, ext, a_mn=True, b_mn=True, out_dtype=torch.float32)          # (9·O, C)
    d_img = d.to(bf).view(1, oh, ow, o)
    dw_pos = conv2d_wgrad(pos_img, d_img, w.shape, stride, pad, dil, out_dtype=torch.float32)
    d_pos = no.conv2d_dgrad(d_img, w, (rows, cols), stride, pad, dil)
    dw = (dw_tab.view(9, o, c).permute(1, 0, 2) + dw_pos.view(o, 9, c)).to(w.dtype).view(o, 3, 3, c)
    return d_ext[:v], d_pos.view(rows * cols, c).float(), d_ext[v:v + 6], dw


def first_layer_forward_torch(cells, cp_embed, pos_embed, colour, w, rows, cols, stride, pad, dil):
    """Same decomposition in fp32 PyTorch: returns the pre-activation ``z (N, OH, OW, O)`` and the features."""
    o, _, _, c = w.shape
    n = cells.shape[0]
    oh, ow = out_hw(rows, cols, stride, pad, dil)
    taps = tap_cells(rows, cols, stride, pad, dil, cells.device)
    wf = w.float()
    w_p = wf.permute(1, 2, 0, 3).reshape(9 * o, c)
    ext = torch.cat([cp_embed, colour], 0).float()
    prod = ext @ w_p.t()
    v = cp_embed.shape[0]
    table = prod[:v].view(v, 9, o)
    cc = torch.zeros(FEATURES, o, dtype=torch.float32, device=w.device)
    cc[:54] = prod[v:].view(6, 9, o).permute(1, 0, 2).reshape(54, o)
    pos_out = F.conv2d(pos_embed.float().view(1, rows, cols, c).permute(0, 3, 1, 2), wf.permute(0, 3, 1, 2), None,
                       stride, pad, dil).permute(0, 2, 3, 1).reshape(oh * ow, o)
    feat = features_torch(cells, taps, torch.float32)
    z = gather_torch(cells, taps, table) + pos_out.unsqueeze(0) + feat @ cc
    return z.view(n, oh, ow, o), feat


def first_layer_backward_torch(cells, feat, dz, cp_embed, pos_embed, colour, w, rows, cols, stride, pad, dil):
    o, _, _, c = w.shape
    v = cp_embed.shape[0]
    n = cells.shape[0]
    oh, ow = out_hw(rows, cols, stride, pad, dil)
    taps = tap_cells(rows, cols, stride, pad, dil, cells.device)
    wf = w.float()
    w_p = wf.permute(1, 2, 0, 3).reshape(9 * o, c)
    ext = torch.cat([cp_embed, colour], 0).float()
    dzf = dz.float().reshape(n, oh * ow, o)
    s_cp, d = reduce_torch(cells, taps, dzf, v)
    q = torch.einsum("npk,npo->ok", feat.float(), dzf)                                  # (O, 64)
    s = torch.cat([s_cp, q[:, :54].view(o, 9, 6).permute(2, 1, 0)], 0).reshape(v + 6, 9 * o)
    d_ext = s @ w_p
    dw_tab = s.t() @ ext
    d_img = d.view(1, oh, ow, o).permute(0, 3, 1, 2)
    pos_img = pos_embed.float().view(1, rows, cols, c).permute(0, 3, 1, 2)
    dw_pos = torch.nn.grad.conv2d_weight(pos_img, (o, c, 3, 3), d_img, stride, pad, dil).permute(0, 2, 3, 1)
    d_pos = torch.nn.grad.conv2d_input((1, c, rows, cols), wf.permute(0, 3, 1, 2), d_img, stride, pad, dil)
    dw = dw_tab.view(9, o, c).permute(1, 0, 2).reshape(o, 3, 3, c) + dw_pos
    return d_ext[:v], d_pos.permute(0, 2, 3, 1).reshape(rows * cols, c), d_ext[v:], dw.to(w.dtype)


class CellConvGelu(torch.autograd.Function):
    """``GELU(conv3x3(cell_embed(cells)))`` through the table decomposition.  CUDA bf16 / fp16 parameters take the native
    kernels; anything else the PyTorch form (which is how the decomposition is tested on the CPU)."""

    @staticmethod
    def forward(ctx, cells, cp_embed, pos_embed, colour, w, rows, cols, stride, pad, dil):
        cells = cells.contiguous()
        native = cells.is_cuda and w.dtype in (torch.bfloat16, torch.float16) and supported(cells, cp_embed, w)
        geom = (rows, cols, stride, pad, dil)
        if native:
            y, z, feat = first_layer_forward_native(cells, cp_embed, pos_embed, colour, w, *geom)
        else:
            z, feat = first_layer_forward_torch(cells, cp_embed, pos_embed, colour, w, *geom)
            y = F.gelu(z).to(w.dtype)
            z = z.to(w.dtype)
        ctx.save_for_backward(cells, feat, z, cp_embed, pos_embed, colour, w)
        ctx.geom, ctx.native = geom, native
        return y

    @staticmethod
    def backward(ctx, dy):
        cells, feat, z, cp_embed, pos_embed, colour, w = ctx.saved_tensors
        if ctx.native:
            from .native_ops import _gelu_bwd
            dz = _gelu_bwd(z, dy.contiguous())
            d_cp, d_pos, d_col, dw = first_layer_backward_native(cells, feat, dz, cp_embed, pos_embed, colour, w, *ctx.geom)
        else:
            from .reference import gelu_grad
            dz = dy.float() * gelu_grad(z)
            d_cp, d_pos, d_col, dw = first_layer_backward_torch(cells, feat, dz, cp_embed, pos_embed, colour, w, *ctx.geom)
        return (None, d_cp.to(cp_embed.dtype), d_pos.to(pos_embed.dtype), d_col.to(colour.dtype), dw,
                None, None, None, None, None)


def cell_conv_gelu(cells, cp_embed, pos_embed, colour, w, rows, cols, stride, pad, dil):
    """``cells`` int32 ``(N, rows·cols, 3)`` → ``(N, OH, OW, O)``."""
    return CellConvGelu.apply(cells, cp_embed, pos_embed, colour, w, rows, cols, stride, pad, dil)
