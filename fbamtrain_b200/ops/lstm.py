"""LSTM over a whole sequence on the GPU.

Forward: one tensor-core GEMM computes the input projection of all time steps
(``X·W_ihᵀ + b_ih + b_hh``, fp32 out), then one persistent cooperative kernel runs the recurrence
with ``W_hh`` resident in registers (``csrc/lstm.cu``).  Backward: one persistent kernel does BPTT and
emits ``dGates`` for every step; the weight and input gradients are then three large GEMMs over all
``T·B`` rows (``dX = dGates·W_ih``, ``dW_ih = dGatesᵀ·X``, ``dW_hh = dGatesᵀ·H_prev``) and a column sum.
The reference performs the same mathematics one step at a time with a GEMM per step and recomputes
the gates in the backward pass (reference: ``tensorlib/src/streaming_lstm_fwd.cpp:430-465``,
``streaming_lstm_bwd.cpp:1218-1307``); here the activated gates are kept (in the buffer that held the
pre-activations), so nothing is recomputed.

Shapes beyond the persistent kernels' limits (hidden > 2048 or batch > 8) run step by step: a GEMM
per step against ``W_hh`` followed by the same gate arithmetic.
"""
from __future__ import annotations


import torch

from ..utils import flops

from . import native as nv
from . import reference as ref
from .native_ops import gemm, gemm_nn, gemm_tn

_scratch = {}


def _counter(device) -> torch.Tensor:
    key = ("ctr", device.index)
    if key not in _scratch:
        _scratch[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _scratch[key]


def persistent_ok(batch: int, hidden: int) -> bool:
    return batch <= 8 and hidden % 16 == 0 and hidden <= nv.lib().fbam_lstm_persistent_max_hidden()


class _LstmSequence(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_ih, w_hh, b_ih, b_hh, h0, c0):
        t_len, b, i_dim = x.shape
        h = w_hh.shape[1]
        dev = x.device
        x2 = x.reshape(t_len * b, i_dim).contiguous()
        wi, wh = w_ih.to(x.dtype), w_hh.to(x.dtype)
        bias = (b_ih.float() + b_hh.float()).contiguous()
        gates = gemm(x2, wi, bias=bias, out_dtype=torch.float32).view(t_len, b, 4 * h)
        y = torch.empty(t_len, b, h, dtype=x.dtype, device=dev)
        c_all = torch.empty(t_len, b, h, dtype=torch.float32, device=dev)
        hbuf = torch.empty(2 * 8 * h, dtype=x.dtype, device=dev)
        h0f, c0f = h0.float().contiguous(), c0.float().contiguous()
        per_sample = int(h0.dim() == 2)
        nv.check(nv.lib(wh).fbam_lstm_fwd_ex(nv.ptr(gates), nv.ptr(wh), nv.ptr(h0f), nv.ptr(c0f), nv.ptr(y),
                                           nv.ptr(c_all), nv.ptr(hbuf), nv.ptr(_counter(dev)),
                                           nv.ptr(nv.status_word(dev)), t_len, b, h, per_sample, nv.stream_ptr()),
                 "fbam_lstm_fwd")
        flops.add(2.0 * t_len * b * h * 4 * h)          # the recurrent product; the input projection is a counted GEMM
        ctx.save_for_backward(x2, wi, wh, gates, y, c_all, h0f, c0f)
        ctx.dims = (t_len, b, i_dim, h)
        ctx.per_sample = per_sample
        return y, y[-1].clone(), c_all[-1].clone()

    @staticmethod
    def backward(ctx, dy, dh_last, dc_last):
        x2, wi, wh, gates, y, c_all, h0f, c0f = ctx.saved_tensors
        t_len, b, i_dim, h = ctx.dims
        dev = dy.device
        dy = dy.contiguous()
        wh_t = wh.t().contiguous()
        dgates = torch.empty(t_len, b, 4 * h, dtype=wh.dtype, device=dev)
        dh0 = torch.empty(b, h, dtype=torch.float32, device=dev)
        dc0 = torch.empty(b, h, dtype=torch.float32, device=dev)
        dhl = None if dh_last is None else dh_last.float().contiguous()
        dcl = None if dc_last is None else dc_last.float().contiguous()
        nv.check(nv.lib(wh).fbam_lstm_bwd_ex(nv.ptr(gates), nv.ptr(c_all), nv.ptr(c0f), nv.ptr(dy), nv.ptr(wh_t),
                                           nv.ptr(dgates), nv.ptr(dh0), nv.ptr(dc0), nv.ptr(dhl), nv.ptr(dcl),
                                           nv.ptr(_counter(dev)), nv.ptr(nv.status_word(dev)), t_len, b, h,
                                           ctx.per_sample, nv.stream_ptr()), "fbam_lstm_bwd")
        flops.add(2.0 * t_len * b * h * 4 * h)
        dg2 = dgates.view(t_len * b, 4 * h)
        dx = gemm_nn(dg2, wi).view(t_len, b, i_dim) if ctx.needs_input_grad[0] else None
        dw_ih = gemm_tn(dg2, x2, out_dtype=torch.float32)
        h_first = h0f.to(y.dtype).view(1, b, h) if ctx.per_sample else h0f.to(y.dtype).expand(1, b, h)
        h_prev = torch.cat([h_first, y[:-1]], 0).reshape(t_len * b, h)
        dw_hh = gemm_tn(dg2, h_prev, out_dtype=torch.float32)
        from .native_ops import _colsum
        db = _colsum(dg2)
        if ctx.per_sample:
            return dx, dw_ih, dw_hh, db, db.clone(), dh0, dc0
        return dx, dw_ih, dw_hh, db, db.clone(), dh0.sum(0), dc0.sum(0)


def _stepwise(x, w_ih, w_hh, b_ih, b_hh, h0, c0):
    """Fallback for shapes the persistent kernels do not cover: tensor-core GEMM per step, autograd."""
    from .native_ops import linear
    t_len, b, _ = x.shape
    hdim = w_hh.shape[1]
    wi, wh = w_ih.to(x.dtype), w_hh.to(x.dtype)
    bias = b_ih.float() + b_hh.float()
    xg = linear(x.reshape(t_len * b, -1), wi).float().view(t_len, b, 4 * hdim)
    h = h0.to(x.dtype).unsqueeze(0).expand(b, hdim).contiguous()
    c = c0.float().unsqueeze(0).expand(b, hdim)
    ys = []
    for t in range(t_len):
        hf, c = ref.lstm_cell(xg[t] + linear(h, wh).float() + bias, c)
        h = hf.to(x.dtype)
        ys.append(h)
    return torch.stack(ys, 0), h, c


def lstm_sequence(x, w_ih, w_hh, b_ih, b_hh, h0, c0, compute_dtype):
    if compute_dtype not in nv.ELEM_DTYPES:
        raise TypeError("native LSTM computes in bf16 or fp16")
    x = x.to(compute_dtype)
    if not persistent_ok(x.shape[1], w_hh.shape[1]) or x.shape[2] % 8 != 0:
        return _stepwise(x, w_ih, w_hh, b_ih, b_hh, h0, c0)
    return _LstmSequence.apply(x, w_ih, w_hh, b_ih, b_hh, h0, c0)
