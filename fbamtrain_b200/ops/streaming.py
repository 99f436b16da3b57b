"""Streaming LSTM + LM head + cross-entropy over sequences that are never resident on the device as a whole.

This is the reference's long-sequence mechanism (reference: ``tensorlib/src/streaming_lstm_fwd.cpp:22-583``,
``streaming_lstm_bwd.cpp:676-1390``, hook / supplier in ``src/main.cpp:1377-1463`` and
``src/main_action_model.cpp:117-203``) on the persistent kernels:

* the input ``x`` ``(T, B, I)`` may live in pinned host memory; it is uploaded chunk by chunk
  (``streaming_chunk_size`` steps, next chunk prefetched on a copy stream);
* per chunk the forward runs input-projection GEMM → persistent recurrent kernel with the state carried from the
  previous chunk, and — the *per-chunk hook* — immediately computes the LM head and the cross-entropy for that
  chunk, including ``dY = dLogits·W_headᵀ`` and ``dW_head += yᵀ·dLogits``, so neither the logits nor y outlive the
  chunk; only the (h, c) state at each chunk boundary and the bf16 ``dY`` chunks are kept (``dY`` optionally in
  pinned host memory);
* the backward walks the chunks in reverse, re-uploads x, *recomputes* the chunk's gates and cell states from the
  boundary state (the recompute FLOPs are not counted as useful), runs the BPTT kernel with the stored ``dY``
  (the *dY supplier*), and accumulates ``dW_ih``, ``dW_hh``, the biases and ``dX``.
"""
from __future__ import annotations

import ctypes as C
from typing import List

import torch

from ..utils import flops

from ..utils.stream_io import TensorStreamIterator, TensorStreamPopulator
from . import native as nv
from .native_ops import _colsum, gemm, gemm_nn, gemm_tn


def _fwd_chunk(x2, wi, wh, bias, h_state, c_state, t_len, b, h, dev, counter):
    gates = gemm(x2, wi, bias=bias, out_dtype=torch.float32).view(t_len, b, 4 * h)
    y = torch.empty(t_len, b, h, dtype=wh.dtype, device=dev)
    c_all = torch.empty(t_len, b, h, dtype=torch.float32, device=dev)
    hbuf = torch.empty(2 * 8 * h, dtype=wh.dtype, device=dev)
    nv.check(nv.lib(wh).fbam_lstm_fwd_ex(nv.ptr(gates), nv.ptr(wh), nv.ptr(h_state), nv.ptr(c_state), nv.ptr(y),
                                       nv.ptr(c_all), nv.ptr(hbuf), nv.ptr(counter), nv.ptr(nv.status_word(dev)),
                                       t_len, b, h, 1, nv.stream_ptr()), "fbam_lstm_fwd")
    return gates, y, c_all


class _StreamingLstmHeadCe(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_ih, w_hh, b_ih, b_hh, h0, c0, w_head, targets, vocab, scale, chunk, offload):
        t_total, b, i_dim = x.shape
        h = w_hh.shape[1]
        dev = w_ih.device
        elem = w_head.dtype                       # the model's 16-bit compute type
        wi, wh = w_ih.to(elem), w_hh.to(elem)
        bias = (b_ih.float() + b_hh.float()).contiguous()
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        h_state = h0.float().unsqueeze(0).expand(b, h).contiguous()
        c_state = c0.float().unsqueeze(0).expand(b, h).contiguous()
        loss = torch.zeros(1, dtype=torch.float32, device=dev)
        dw_head = torch.zeros(w_head.shape, dtype=torch.float32, device=dev)
        vpad = w_head.shape[0]
        dy_store = torch.empty((t_total, b, h), dtype=elem, device="cpu" if offload else dev,
                               pin_memory=offload and dev.type == "cuda")
        populator = TensorStreamPopulator(dy_store) if offload else None
        boundary: List[tuple] = []
        targets = targets.to(dev)
        ce_stream = torch.cuda.Stream(device=dev)
        for lo, hi, x_c in TensorStreamIterator(x, chunk, dev):
            n = hi - lo
            boundary.append((h_state, c_state))
            x2 = x_c.to(elem).reshape(n * b, i_dim)
            _, y, c_all = _fwd_chunk(x2, wi, wh, bias, h_state, c_state, n, b, h, dev, counter)
            h_state, c_state = y[-1].float(), c_all[-1].clone()
            # per-chunk hook on its own stream: LM head + CE forward/backward for this chunk
            ce_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(ce_stream):
                y2 = y.view(n * b, h)
                logits = gemm(y2, w_head)
                nv.check(nv.lib(logits).fbam_ce_fwd_bwd(nv.ptr(logits), nv.ptr(targets[lo:hi].reshape(-1).contiguous()),
                                                  nv.ptr(loss), C.c_longlong(n * b), vocab, vpad, C.c_float(scale), 1,
                                                  nv.stream_ptr()), "fbam_ce_fwd_bwd")
                dy_c = gemm_nn(logits, w_head).view(n, b, h)
                gemm_tn(logits, y2, out=dw_head, accumulate=nv.GEMM_ACC_RMW)
                if offload:
                    populator.write(lo, dy_c)
                else:
                    dy_store[lo:hi].copy_(dy_c)
            y.record_stream(ce_stream)
        torch.cuda.current_stream().wait_stream(ce_stream)
        if populator is not None:
            populator.synchronize()
        ctx.save_for_backward(w_ih, wi, wh, bias, dw_head, w_head)
        ctx.x, ctx.dy_store, ctx.boundary = x, dy_store, boundary
        ctx.meta = (t_total, b, i_dim, h, chunk, offload)
        ctx.final_state = (h_state, c_state)
        return loss.reshape(())

    @staticmethod
    def backward(ctx, dloss):
        w_ih, wi, wh, bias, dw_head, w_head = ctx.saved_tensors
        t_total, b, i_dim, h, chunk, offload = ctx.meta
        dev = wi.device
        x, dy_store = ctx.x, ctx.dy_store
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        wh_t = wh.t().contiguous()
        dw_ih = torch.zeros(4 * h, i_dim, dtype=torch.float32, device=dev)
        dw_hh = torch.zeros(4 * h, h, dtype=torch.float32, device=dev)
        db = torch.zeros(4 * h, dtype=torch.float32, device=dev)
        dx = torch.empty((t_total, b, i_dim), dtype=wi.dtype, device="cpu" if x.device.type == "cpu" and offload else dev,
                         pin_memory=offload and x.device.type == "cpu" and dev.type == "cuda")
        dx_pop = TensorStreamPopulator(dx) if not dx.is_cuda else None
        dh_carry = dc_carry = None
        bounds = [(lo, min(t_total, lo + chunk)) for lo in range(0, t_total, chunk)]
        dy_iter = iter(TensorStreamIterator(dy_store, chunk, dev, reverse=True))
        for k, (lo, hi, x_c) in zip(range(len(bounds) - 1, -1, -1), TensorStreamIterator(x, chunk, dev, reverse=True)):
            _, _, dy_c = next(dy_iter)
            n = hi - lo
            h_start, c_start = ctx.boundary[k]
            x2 = x_c.to(wi.dtype).reshape(n * b, i_dim)
            with flops.not_useful():                  # recomputation of what a resident run would have kept
                gates, y, c_all = _fwd_chunk(x2, wi, wh, bias, h_start, c_start, n, b, h, dev, counter)
            dgates = torch.empty(n, b, 4 * h, dtype=wi.dtype, device=dev)
            dh0 = torch.empty(b, h, dtype=torch.float32, device=dev)
            dc0 = torch.empty(b, h, dtype=torch.float32, device=dev)
            nv.check(nv.lib(wh_t).fbam_lstm_bwd_ex(nv.ptr(gates), nv.ptr(c_all), nv.ptr(c_start), nv.ptr(dy_c.contiguous()),
                                               nv.ptr(wh_t), nv.ptr(dgates), nv.ptr(dh0), nv.ptr(dc0),
                                               nv.ptr(dh_carry), nv.ptr(dc_carry), nv.ptr(counter),
                                               nv.ptr(nv.status_word(dev)), n, b, h, 1, nv.stream_ptr()),
                     "fbam_lstm_bwd")
            dh_carry, dc_carry = dh0, dc0
            dg2 = dgates.view(n * b, 4 * h)
            dx_c = gemm_nn(dg2, wi).view(n, b, i_dim)
            if dx_pop is not None:
                dx_pop.write(lo, dx_c)
            else:
                dx[lo:hi].copy_(dx_c)
            gemm_tn(dg2, x2, out=dw_ih, accumulate=nv.GEMM_ACC_RMW)
            h_prev = torch.cat([h_start.to(y.dtype).view(1, b, h), y[:-1]], 0).reshape(n * b, h)
            gemm_tn(dg2, h_prev, out=dw_hh, accumulate=nv.GEMM_ACC_RMW)
            db += _colsum(dg2)
        if dx_pop is not None:
            dx_pop.synchronize()
        s = dloss.float()
        dxo = dx if not ctx.needs_input_grad[0] else (dx * s.to(dx.device).to(dx.dtype) if float(s) != 1.0 else dx)
        return (dxo if ctx.needs_input_grad[0] else None, dw_ih * s, dw_hh * s, db * s, db * s,
                dh_carry.sum(0) * s, dc_carry.sum(0) * s, (dw_head * s).to(w_head.dtype), None, None, None, None, None)


def streaming_lstm_head_ce(x, w_ih, w_hh, b_ih, b_hh, h0, c0, w_head, targets, vocab: int, scale: float,
                           chunk: int, offload: bool = False):
    """Loss of ``LM-head(LSTM(x))`` against ``targets`` (time-major ``(T, B)``), streamed in chunks of ``chunk`` steps.
    ``x`` may be a pinned host tensor; with ``offload`` the stored ``dY`` (and ``dX`` for a host ``x``) also stay in
    pinned host memory."""
    return _StreamingLstmHeadCe.apply(x, w_ih, w_hh, b_ih, b_hh, h0, c0, w_head, targets, vocab, scale, chunk, offload)
