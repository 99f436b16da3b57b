#!/usr/bin/env python
"""Times the reference's own Triton kernels on this GPU, next to this package's kernels, at the shapes the
reference's committed autotune tables quote.

    python benchmarks/bench_reference_kernels.py [--reference-dir DIR] [--only gemm,attention,conv]

The reference ships its kernels as Triton sources that it compiles ahead of time; on an sm_100 part Triton lowers
``tl.dot`` to the tcgen05 tensor cores, so these are the reference's real Blackwell kernels
(``kernel_gen/kernel_gen/kernels/addmm_act.py:65-226`` GEMM + bias + GELU with the tile configuration of
``configs/triton_matmul_autotune_sm100.json``, ``flash_attention_fwd.py:268-320`` attention forward,
``conv2d.py:194-324`` NHWC convolution).  The sources are imported unmodified from a checkout of the reference
(``--reference-dir``, ``FBAM_REFERENCE_DIR``, ``baseline/_ref`` or a sibling directory ``reference``) through their
own Python entry points and JIT-compiled by the installed Triton; nothing of them is part of this package.  Each
kernel that cannot be imported, compiled or run is reported as unavailable with the error, and the run goes on.

Timing: CUDA events around one call, L2 flushed before every timed call, median of ``BENCH_ITERS`` after
``BENCH_WARMUP`` warm-up calls.  One JSON line per measurement, with ``impl`` = ``reference-triton`` or ``ours``.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import sys
import traceback

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from bench_kernels import timeit  # noqa: E402


def find_reference(explicit: str) -> str:
    cands = [explicit, os.environ.get("FBAM_REFERENCE_DIR", ""), os.path.join(ROOT, "baseline", "_ref"),
             os.path.join(os.path.dirname(ROOT), "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "kernel_gen", "kernel_gen", "kernels")):
            return c
    return ""


def emit(name, impl, ms=None, flops=None, error=None, **extra):
    out = {"bench": name, "impl": impl}
    if error is not None:
        out["unavailable"] = error
    else:
        out["ms"] = ms
        if flops:
            out["tflops"] = flops / ms / 1e9
    out.update(extra)
    print(json.dumps(out), flush=True)


def guarded(name, fn):
    try:
        fn()
    except Exception as ex:  # noqa: BLE001 - reported, the other kernels still run
        last = traceback.format_exc().strip().splitlines()[-1]
        emit(name, "reference-triton", error=f"{type(ex).__name__}: {last[:300]}")


def bench_gemm(kernels):
    from fbamtrain_b200.ops import native_ops as no
    mod = importlib.import_module("kernels.addmm_act")
    import triton
    m = n = k = 4096
    flops = 2.0 * m * n * k
    a = torch.randn(m, k, device="cuda").bfloat16()
    b_kn = torch.randn(k, n, device="cuda").bfloat16()
    bias = torch.randn(n, device="cuda").bfloat16()
    c = bias.unsqueeze(0).expand(m, n)                      # broadcast bias: row stride 0, as the reference passes it
    d = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    cfg = {"BLOCK_SIZE_M": 128, "BLOCK_SIZE_N": 256, "BLOCK_SIZE_K": 64, "GROUP_SIZE_M": 8}     # its sm100 table

    def ref_call(act):
        grid = (triton.cdiv(m, cfg["BLOCK_SIZE_M"]) * triton.cdiv(n, cfg["BLOCK_SIZE_N"]),)
        mod.addmm_act[grid](a, b_kn, c, d, m, n, k, *a.stride(), *b_kn.stride(), *c.stride(), *d.stride(),
                            num_warps=8, num_stages=3, ACTIVATION=act, ACCUMULATE_IN_FP16=False, HAS_BIAS=True,
                            ACCUMULATE_OUTPUT=False, **cfg)

    for act, label in ((0, "gemm+bias"), (2, "gemm+bias+gelu")):
        guarded(f"{label} 4096^3 bf16", lambda act=act, label=label: emit(
            f"{label} 4096^3 bf16", "reference-triton", timeit(lambda: ref_call(act)), flops,
            tile="128x256x64, 8 warps, 3 stages (configs/triton_matmul_autotune_sm100.json)"))
    w_nk = b_kn.t().contiguous()
    emit("gemm+bias 4096^3 bf16", "ours", timeit(lambda: no.gemm(a, w_nk, bias=bias, out=d)), flops)
    emit("gemm+bias+gelu 4096^3 bf16", "ours", timeit(lambda: no.gemm(a, w_nk, bias=bias, act="gelu", out=d)), flops)


def bench_attention(kernels):
    from fbamtrain_b200 import ops
    mod = importlib.import_module("kernels.flash_attention_fwd")
    b, h, t, d = 8, 8, 1024, 128
    flops = 4.0 * b * h * t * t * d
    q, k, v = (torch.randn(b, t, h, d, device="cuda").bfloat16() for _ in range(3))
    scale = 1.0 / math.sqrt(d)
    for ws in (True, False):
        guarded(f"attention fwd B{b} H{h} T{t} D{d} non-causal", lambda ws=ws: emit(
            f"attention fwd B{b} H{h} T{t} D{d} non-causal", "reference-triton",
            timeit(lambda: mod.flash_attn_fwd(q, k, v, causal=False, sm_scale=scale, warp_specialize=ws)), flops,
            warp_specialize=ws))
    emit(f"attention fwd B{b} H{h} T{t} D{d} non-causal", "ours", timeit(lambda: ops.attention(q, k, v, False)), flops)


def bench_conv(kernels):
    from fbamtrain_b200.ops import native_ops as no
    mod = importlib.import_module("kernels.conv2d")
    for (n, hh, ww, cin, cout, stride, dil) in ((32, 48, 160, 1024, 1024, 1, 2), (256, 48, 160, 128, 256, 2, 1)):
        pad = dil
        oh, ow = no.conv_out_hw(hh, ww, stride, pad, dil)
        flops = 2.0 * n * oh * ow * cout * cin * 9
        x_nhwc = torch.randn(n, hh, ww, cin, device="cuda").bfloat16()
        w_ohwi = (torch.randn(cout, 3, 3, cin, device="cuda") / math.sqrt(9 * cin)).bfloat16()
        x_nchw_cl = x_nhwc.permute(0, 3, 1, 2)              # NCHW view of channels-last memory: what its wrapper takes
        w_oihw = w_ohwi.permute(0, 3, 1, 2).contiguous()
        tag = f"conv fprop n{n} {hh}x{ww} {cin}->{cout} s{stride} d{dil}"
        guarded(tag, lambda: emit(tag, "reference-triton",
                                  timeit(lambda: mod._conv2d_triton(x_nchw_cl, w_oihw, None, stride, pad, dil)), flops))
        emit(tag, "ours", timeit(lambda: no.conv2d_fprop(x_nhwc, w_ohwi, stride, pad, dil)), flops)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-dir", default="")
    ap.add_argument("--only", default="gemm,attention,conv")
    a = ap.parse_args()
    ref = find_reference(a.reference_dir)
    if not ref:
        print(json.dumps({"impl": "reference-triton", "unavailable": "no checkout of the reference found (pass "
                          "--reference-dir or set FBAM_REFERENCE_DIR)"}))
        return
    sys.path.insert(0, os.path.join(ref, "kernel_gen", "kernel_gen"))
    try:
        import triton
        print(json.dumps({"reference_dir": ref, "triton": triton.__version__, "device": torch.cuda.get_device_name(0)}))
    except Exception as ex:  # noqa: BLE001
        print(json.dumps({"impl": "reference-triton", "unavailable": f"triton does not import: {ex}"}))
        return
    for name, fn in (("gemm", bench_gemm), ("attention", bench_attention), ("conv", bench_conv)):
        if name in a.only.split(","):
            try:
                fn(ref)
            except Exception as ex:  # noqa: BLE001 - an import error of the reference module, or a failure of ours
                last = traceback.format_exc().strip().splitlines()[-1]
                print(json.dumps({"bench": name, "unavailable": f"{type(ex).__name__}: {last[:300]}"}), flush=True)


if __name__ == "__main__":
    main()
