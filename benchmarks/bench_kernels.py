#!/usr/bin/env python
"""Per-kernel benchmarks (device-timed with CUDA events, L2 flushed between iterations).

    python benchmarks/bench_kernels.py gemm  [--m 4096 --n 4096 --k 4096] [--library]
    python benchmarks/bench_kernels.py conv  [--batch 512 --h 48 --w 160 --cin 128 --cout 256 --stride 2]
    python benchmarks/bench_kernels.py lstm  [--t 1024 --b 8 --hidden 1024]
    python benchmarks/bench_kernels.py lstm-stream [--t 1024 --b 8 --hidden 1024 --vocab 4096 --chunk 64] [--offload]
    python benchmarks/bench_kernels.py mha   [--b 8 --heads 8 --t 1024 --d 128] [--causal]
    python benchmarks/bench_kernels.py simt  [--rows 16384 --dim 1024 --vocab 4096 --numel 67108864]
    python benchmarks/bench_kernels.py embconv [--frames 1024 --rows 48 --cols 160 --vocab 512 --cin 128 --cout 256
                                                --change 0.05]

Shapes default to the ones the reference's own benchmark programs use (GEMM 4096³ / 8192³, conv
(32, 48, 160, 1024→1024), MHA (8, 8, 1024, 128), streaming LSTM; reference: ``benchmarks/`` and
``benchmarks/common/benchmark_utils.h:59-71``) — ``BENCH_WARMUP`` / ``BENCH_ITERS`` are honoured as there.
``--library`` times the cuBLAS / cuDNN / SDPA call for the same problem next to the native kernel.
Each run prints one JSON line with milliseconds, TFLOP/s and the fraction of the measured peaks.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

WARMUP = int(os.environ.get("BENCH_WARMUP", "5"))
ITERS = int(os.environ.get("BENCH_ITERS", "20"))


def timeit(fn, iters=ITERS, warmup=WARMUP):
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")   # larger than the 126 MB L2
    times = []
    for _ in range(iters):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    times.sort()
    return times[len(times) // 2]


def report(name, ms, flops=None, bytes_moved=None, extra=None):
    from fbamtrain_b200.utils.mfu import measured_peaks
    peaks = measured_peaks()
    out = {"bench": name, "ms": ms, "peaks": peaks["source"]}
    if flops:
        out["tflops"] = flops / ms / 1e9
        out["frac_of_cublas_burst"] = out["tflops"] / peaks["bf16_tflops"]
    if bytes_moved:
        out["gbs"] = bytes_moved / ms / 1e6
        out["frac_of_copy_bw"] = out["gbs"] / peaks["hbm_gbs"]
    if extra:
        out.update(extra)
    print(json.dumps(out), flush=True)


def bench_gemm(a):
    from fbamtrain_b200.ops import native_ops as no
    x = torch.randn(a.m, a.k, device="cuda").bfloat16()
    w = torch.randn(a.n, a.k, device="cuda").bfloat16()
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    flops = 2.0 * a.m * a.n * a.k
    bias = torch.randn(a.n, device="cuda").bfloat16() if a.bias or a.gelu else None
    pre = torch.empty_like(out) if a.gelu else None
    tag = f"{a.m}x{a.n}x{a.k}" + (" +bias" if bias is not None else "") + (" +gelu +preact" if a.gelu else "")
    report("gemm_tcgen05 " + tag, timeit(lambda: no.gemm(x, w, out=out, bias=bias, act="gelu" if a.gelu else "none",
                                                         preact_out=pre)), flops)
    if a.library:
        if a.gelu:
            lib = lambda: torch.nn.functional.gelu(torch.addmm(bias, x, w.t()))
        elif bias is not None:
            lib = lambda: torch.addmm(bias, x, w.t(), out=out)
        else:
            lib = lambda: torch.matmul(x, w.t(), out=out)
        report("gemm_cublas " + tag, timeit(lib), flops)


def bench_conv(a):
    from fbamtrain_b200.ops import native_ops as no
    from fbamtrain_b200.ops.conv_wgrad import conv2d_wgrad
    x = torch.randn(a.batch, a.h, a.w, a.cin, device="cuda").bfloat16()
    w = (torch.randn(a.cout, 3, 3, a.cin, device="cuda") / math.sqrt(9 * a.cin)).bfloat16()
    pad = a.dilation
    oh, ow = no.conv_out_hw(a.h, a.w, a.stride, pad, a.dilation)
    flops = 2.0 * a.batch * oh * ow * a.cout * a.cin * 9
    tag = f"n{a.batch} {a.h}x{a.w} {a.cin}->{a.cout} s{a.stride} d{a.dilation}"
    report("conv_fprop " + tag, timeit(lambda: no.conv2d_fprop(x, w, a.stride, pad, a.dilation)), flops)
    dy = torch.randn(a.batch, oh, ow, a.cout, device="cuda").bfloat16()
    report("conv_dgrad " + tag, timeit(lambda: no.conv2d_dgrad(dy, w, (a.h, a.w), a.stride, pad, a.dilation)), flops)
    report("conv_wgrad " + tag, timeit(lambda: conv2d_wgrad(x, dy, w.shape, a.stride, pad, a.dilation)), flops)
    if a.library:
        xc = x.permute(0, 3, 1, 2)
        wc = w.permute(0, 3, 1, 2)
        report("conv_fprop_cudnn " + tag,
               timeit(lambda: torch.nn.functional.conv2d(xc, wc, None, a.stride, pad, a.dilation)), flops)


def bench_lstm(a):
    from fbamtrain_b200.ops import lstm as L
    h = a.hidden
    k = 1.0 / math.sqrt(h)
    x = torch.randn(a.t, a.b, h, device="cuda").bfloat16().requires_grad_(True)
    ps = [((torch.rand(4 * h, h, device="cuda") * 2 - 1) * k).requires_grad_(True) for _ in range(2)]
    bs = [((torch.rand(4 * h, device="cuda") * 2 - 1) * k).requires_grad_(True) for _ in range(2)]
    h0 = torch.zeros(h, device="cuda", requires_grad=True)
    c0 = torch.zeros(h, device="cuda", requires_grad=True)
    useful = 2.0 * a.t * a.b * 2 * h * 4 * h

    def fwd():
        return L.lstm_sequence(x, ps[0], ps[1], bs[0], bs[1], h0, c0, torch.bfloat16)

    report(f"lstm_fwd T{a.t} B{a.b} H{h}", timeit(fwd, iters=10), useful,
           extra={"us_per_step": None})
    y, _, _ = fwd()
    g = torch.randn_like(y)

    def fwd_bwd():
        yy, _, _ = fwd()
        torch.autograd.grad(yy, [x] + ps + bs, g)

    report(f"lstm_fwd_bwd T{a.t} B{a.b} H{h}", timeit(fwd_bwd, iters=10), 3 * useful)


def bench_lstm_stream(a):
    """Streaming LSTM with the per-chunk LM-head + cross-entropy hook and the recomputing backward whose dY comes
    from the head (the reference's "backward with supplier" benchmark: ``benchmarks/bench_streaming_lstm*``)."""
    from fbamtrain_b200.ops.streaming import streaming_lstm_head_ce
    h, vocab = a.hidden, a.vocab
    k = 1.0 / math.sqrt(h)
    x = torch.randn(a.t, a.b, h).bfloat16()
    x = x.pin_memory() if a.offload else x.cuda().requires_grad_(True)
    ps = [((torch.rand(4 * h, h, device="cuda") * 2 - 1) * k).requires_grad_(True) for _ in range(2)]
    bs = [((torch.rand(4 * h, device="cuda") * 2 - 1) * k).requires_grad_(True) for _ in range(2)]
    h0 = torch.zeros(h, device="cuda", requires_grad=True)
    c0 = torch.zeros(h, device="cuda", requires_grad=True)
    w_head = (torch.randn((vocab + 7) // 8 * 8, h, device="cuda") * k).bfloat16().requires_grad_(True)
    tg = torch.randint(0, vocab, (a.t, a.b), device="cuda")
    scale = 1.0 / (a.t * a.b)
    useful = 2.0 * a.t * a.b * (2 * h * 4 * h + h * vocab)

    def fwd():
        with torch.no_grad():
            return streaming_lstm_head_ce(x, ps[0], ps[1], bs[0], bs[1], h0, c0, w_head, tg, vocab, scale, a.chunk,
                                          a.offload)

    def fwd_bwd():
        loss = streaming_lstm_head_ce(x, ps[0], ps[1], bs[0], bs[1], h0, c0, w_head, tg, vocab, scale, a.chunk,
                                      a.offload)
        torch.autograd.grad(loss, ps + bs + [w_head])

    tag = f"T{a.t} B{a.b} H{h} V{vocab} chunk{a.chunk} offload={a.offload}"
    report(f"lstm_stream_fwd {tag}", timeit(fwd, iters=5), useful)
    report(f"lstm_stream_fwd_bwd_supplier {tag}", timeit(fwd_bwd, iters=5), 3 * useful,
           extra={"note": "time includes the recomputation of every chunk's gates (not counted as useful FLOPs)"})


def bench_mha(a):
    from fbamtrain_b200 import ops
    q, k, v = (torch.randn(a.b, a.t, a.heads, a.d, device="cuda").bfloat16().requires_grad_(True) for _ in range(3))
    flops = 4.0 * a.b * a.heads * a.t * a.t * a.d * (0.5 if a.causal else 1.0)
    report(f"mha_fwd B{a.b} H{a.heads} T{a.t} D{a.d} causal={a.causal}",
           timeit(lambda: ops.attention(q, k, v, a.causal)), flops)
    o = ops.attention(q, k, v, a.causal)
    g = torch.randn_like(o)

    def fb():
        torch.autograd.grad(ops.attention(q, k, v, a.causal), (q, k, v), g)

    report(f"mha_fwd_bwd B{a.b} H{a.heads} T{a.t} D{a.d} causal={a.causal}", timeit(fb), 3.5 * flops)


def coherent_cells(frames, cells_per_frame, vocab, change, seed=0, device="cuda"):
    """Frames of (code point, fg, bg) words in which every frame copies its predecessor and redraws a fraction
    ``change`` of the cells (the benchmark configurations' frame statistics)."""
    g = torch.Generator(device=device).manual_seed(seed)

    def fresh(n):
        return torch.stack([torch.randint(0, vocab, (n, cells_per_frame), generator=g, device=device),
                            torch.randint(0, 1 << 24, (n, cells_per_frame), generator=g, device=device),
                            torch.randint(0, 1 << 24, (n, cells_per_frame), generator=g, device=device)], -1).int()
    new = fresh(frames)
    if change >= 1.0:
        return new
    keep = torch.rand(frames, cells_per_frame, generator=g, device=device) >= change
    keep[0] = False
    # index of the last redraw at or before each frame, per cell
    idx = torch.where(keep, torch.zeros_like(keep, dtype=torch.long),
                      torch.arange(frames, device=device).view(-1, 1).expand(-1, cells_per_frame))
    idx = torch.cummax(idx, 0).values
    return torch.gather(new, 0, idx.unsqueeze(-1).expand(-1, -1, 3)).contiguous()


def bench_embconv(a):
    """The kernels of the fused "cell embedding + first convolution" layer on one chunk of frames, each timed alone,
    with the bytes that have to move as the roofline."""
    from fbamtrain_b200.ops import embconv
    from fbamtrain_b200.ops import native_ops as no
    from fbamtrain_b200.ops.conv_wgrad import wgrad_pass
    rows, cols, o, c, n = a.rows, a.cols, a.cout, a.cin, a.frames
    geom = (rows, cols, 2, 1, 1)
    oh, ow = embconv.out_hw(*geom)
    cells = coherent_cells(n, rows * cols, a.vocab, a.change)
    table = torch.randn(a.vocab, 9, o, device="cuda").bfloat16()
    pos = torch.randn(oh * ow, o, device="cuda")
    cc_t = torch.randn(o, embconv.FEATURES, device="cuda").bfloat16()
    z = torch.empty(n, oh * ow, o, device="cuda", dtype=torch.bfloat16)
    y = torch.empty_like(z)
    dz = torch.randn(n, oh, ow, o, device="cuda").bfloat16()
    s = torch.zeros(a.vocab, 9, o, device="cuda")
    d = torch.zeros(oh * ow, o, device="cuda")
    tag = f"n{n} {rows}x{cols} v{a.vocab} ->{o} change{a.change}"
    feat = embconv.features_native(cells, *geom)
    pix = n * oh * ow
    report("embconv_features " + tag, timeit(lambda: embconv.features_native(cells, *geom)),
           bytes_moved=cells.numel() * 4 + pix * 128)
    report("embconv_colour_gemm " + tag, timeit(lambda: no.gemm(feat.view(pix, 64), cc_t, out=z.view(pix, o))),
           flops=2.0 * pix * 64 * o, bytes_moved=pix * 128 + pix * o * 2)
    report("embconv_fwd " + tag, timeit(lambda: embconv.forward_native(cells, table, pos, z, y, *geom)),
           bytes_moved=3 * pix * o * 2 + cells.numel() * 4 // 3)
    report("embconv_bwd_reduce " + tag, timeit(lambda: embconv.reduce_native(cells, dz.view(n, oh * ow, o), s, d, *geom)),
           bytes_moved=pix * o * 2 + cells.numel() * 4 // 3)
    report("embconv_colour_wgrad " + tag,
           timeit(lambda: wgrad_pass(feat.view(n, oh, ow, 64), dz, o, 64, [(0, 0)], 1, out_dtype=torch.float32)),
           flops=2.0 * pix * 64 * o, bytes_moved=pix * 128 + pix * o * 2)


def bench_simt(a):
    """The bandwidth-bound kernels on sizes larger than L2: RMSNorm forward / backward, LayerNorm forward / backward,
    cross-entropy forward + backward on fp32 logits, the fused AdamW step."""
    from fbamtrain_b200.ops import native as nv
    from fbamtrain_b200.ops import native_ops as no
    import ctypes as C
    rows, dim = a.rows, a.dim
    x = torch.randn(rows, dim, device="cuda").bfloat16().requires_grad_(True)
    w = torch.ones(dim, device="cuda").bfloat16().requires_grad_(True)
    b = torch.zeros(dim, device="cuda").bfloat16().requires_grad_(True)
    g = torch.randn(rows, dim, device="cuda").bfloat16()
    report(f"rmsnorm_fwd {rows}x{dim}", timeit(lambda: no.rms_norm(x.detach(), w.detach(), 1e-5)),
           bytes_moved=2 * rows * dim * 2)
    y = no.rms_norm(x, w, 1e-5)
    report(f"rmsnorm_fwd_bwd {rows}x{dim}",
           timeit(lambda: torch.autograd.grad(no.rms_norm(x, w, 1e-5), (x, w), g)), bytes_moved=5 * rows * dim * 2)
    report(f"layernorm_fwd_bwd {rows}x{dim}",
           timeit(lambda: torch.autograd.grad(no.layer_norm(x, w, b, 1e-5), (x, w, b), g)), bytes_moved=5 * rows * dim * 2)
    vrows, vocab = 4096, a.vocab
    logits = torch.randn(vrows, vocab, device="cuda")
    dlogits = torch.empty(vrows, vocab, device="cuda", dtype=torch.bfloat16)
    tg = torch.randint(0, vocab, (vrows,), device="cuda")
    loss = torch.zeros(1, device="cuda")
    report(f"ce_fwd_bwd_f32 {vrows}x{vocab}",
           timeit(lambda: nv.check(nv.lib().fbam_ce_fwd_bwd_f32(nv.ptr(logits), nv.ptr(dlogits), nv.ptr(tg), nv.ptr(loss),
                                                               C.c_longlong(vrows), vocab, vocab, C.c_float(1.0),
                                                               nv.stream_ptr()), "fbam_ce_fwd_bwd_f32")),
           bytes_moved=vrows * vocab * 6)
    n = a.numel
    p = torch.randn(n, device="cuda").bfloat16()
    gr = torch.randn(n, device="cuda").bfloat16()
    m, v, master = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), p.float()
    report(f"adamw bf16 {n}", timeit(lambda: no.adamw_flat(p, gr, m, v, master, 0, n, 1e-3, 0.9, 0.999, 1e-8, 0.1, 0.1, 0.001)),
           bytes_moved=n * (2 + 2 + 4 * 3 * 2))


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=4096)
    g.add_argument("--n", type=int, default=4096)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--library", action="store_true")
    g.add_argument("--bias", action="store_true")
    g.add_argument("--gelu", action="store_true", help="bias + GELU + pre-activation store (the MLP's first layer)")
    c = sub.add_parser("conv")
    for name, default in (("batch", 32), ("h", 48), ("w", 160), ("cin", 1024), ("cout", 1024), ("stride", 1),
                          ("dilation", 2)):
        c.add_argument("--" + name, type=int, default=default)
    c.add_argument("--library", action="store_true")
    l = sub.add_parser("lstm")
    l.add_argument("--t", type=int, default=1024)
    l.add_argument("--b", type=int, default=8)
    l.add_argument("--hidden", type=int, default=1024)
    ls = sub.add_parser("lstm-stream")
    ls.add_argument("--t", type=int, default=1024)
    ls.add_argument("--b", type=int, default=8)
    ls.add_argument("--hidden", type=int, default=1024)
    ls.add_argument("--vocab", type=int, default=4096)
    ls.add_argument("--chunk", type=int, default=64)
    ls.add_argument("--offload", action="store_true")
    m = sub.add_parser("mha")
    for name, default in (("b", 8), ("heads", 8), ("t", 1024), ("d", 128)):
        m.add_argument("--" + name, type=int, default=default)
    m.add_argument("--causal", action="store_true")
    sm = sub.add_parser("simt")
    for name, default in (("rows", 16384), ("dim", 1024), ("vocab", 4096), ("numel", 64 * 1024 * 1024)):
        sm.add_argument("--" + name, type=int, default=default)
    e = sub.add_parser("embconv")
    for name, default in (("frames", 1024), ("rows", 48), ("cols", 160), ("vocab", 512), ("cin", 128), ("cout", 256)):
        e.add_argument("--" + name, type=int, default=default)
    e.add_argument("--change", type=float, default=0.05)
    a = ap.parse_args()
    {"gemm": bench_gemm, "conv": bench_conv, "lstm": bench_lstm, "lstm-stream": bench_lstm_stream,
     "mha": bench_mha, "embconv": bench_embconv, "simt": bench_simt}[a.cmd](a)


if __name__ == "__main__":
    main()
