"""Micro-benchmarks of the fused compute+collective kernels against "NCCL collective + separate kernels".

Launch with one process per GPU::

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_comm.py \
        [--paths rs_adamw_ag,ag_gemm,gemm_rs,muon] [--iters 10] [--multicast]

For every path rank 0 prints one JSON line with the fused time, the library time (same arithmetic, NCCL for the
collective), and the roofline time = the slower of (FLOPs / measured cuBLAS bf16 peak) and (bytes that must cross
NVLink per GPU and direction / measured peer-copy bandwidth).  All times are CUDA-event times on the launching
stream after warm-up, maximum over ranks.  The reference has no kernel that fuses compute with a collective (its
collectives are separate NCCL stream ops: ``src/main.cpp:647-666, 3588-3644``), so the library column is the
stand-in for it.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS = 770.0   # measured peer-copy bandwidth per direction per GPU on this class of machine (900 nominal)
BF = torch.bfloat16


def _peaks():
    from fbamtrain_b200.utils.mfu import measured_peaks
    return measured_peaks()


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _report(rank, name, world, fused_ms, nccl_ms, flops, link_bytes, extra=None, hbm_bytes=0.0):
    pk = _peaks()
    t_compute = flops / (pk["bf16_tflops"] * 1e12) * 1e3
    t_link = link_bytes / (NVLINK_GBS * 1e9) * 1e3
    t_hbm = hbm_bytes / (pk["hbm_gbs"] * 1e9) * 1e3
    roof = max(t_compute, t_link, t_hbm)
    if rank == 0:
        out = {"bench": name, "n_gpus": world, "fused_ms": round(fused_ms, 4), "nccl_ms": round(nccl_ms, 4),
               "speedup_vs_nccl": round(nccl_ms / fused_ms, 3), "roofline_ms": round(roof, 4),
               "roofline_bound": {t_compute: "compute", t_link: "nvlink", t_hbm: "hbm"}[roof],
               "fused_frac_of_roofline": round(roof / fused_ms, 3), "nccl_frac_of_roofline": round(roof / nccl_ms, 3),
               "peaks": pk["source"], "nvlink_gbs_per_dir": NVLINK_GBS}
        out.update(extra or {})
        print(json.dumps(out), flush=True)


# -------------------------------------------------------------------------------------------------------
def bench_rs_adamw_ag(a, rank, world, dev):
    """Gradient reduce-scatter + AdamW on the shard + parameter all-gather for one flat bf16 bucket."""
    from fbamtrain_b200.ops import native as nv
    from fbamtrain_b200.ops import native_ops as no
    from fbamtrain_b200.parallel.peer_window import PeerGroup
    n = a.bucket_mib * (1 << 20) // 2
    n -= n % (8 * world * 8)
    peers = PeerGroup(None, dev, use_multicast=a.multicast)
    wg, wp = peers.allocate("g", n, BF), peers.allocate("p", n, BF)
    wg.local.normal_(std=1e-3)
    wp.local.normal_()
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    master = wp.local.float()
    per = n // world
    lo, hi = rank * per, (rank + 1) * per
    status = nv.status_word(dev)
    hp = dict(lr=1e-4, b1=0.9, b2=0.999, eps=1e-8, wd=0.01)

    def fused():
        code = nv.lib().fbam_rs_adamw_ag(
            wg.c_ptrs, wp.c_ptrs, peers.flags.c_ptrs, C.c_void_p(wg.multicast_ptr), C.c_void_p(wp.multicast_ptr),
            nv.ptr(m), nv.ptr(v), nv.ptr(master), C.c_longlong(lo), C.c_longlong(hi), 1, C.c_float(hp["lr"]),
            C.c_float(hp["b1"]), C.c_float(hp["b2"]), C.c_float(hp["eps"]), C.c_float(hp["wd"]), C.c_float(0.1),
            C.c_float(0.001), C.c_float(1.0), rank, world, C.c_uint(peers.next_epoch()), 1, C.c_uint(1 << 22),
            nv.ptr(status), nv.ptr(peers.arrive), 0, nv.stream_ptr())
        nv.check(code, "fbam_rs_adamw_ag")

    g2, p2 = wg.local.clone(), wp.local.clone()
    red = torch.empty(per, dtype=BF, device=dev)

    def library():
        dist.reduce_scatter_tensor(red, g2)
        no.adamw_flat(p2[lo:hi], red, m[lo:hi], v[lo:hi], master[lo:hi], 0, per, hp["lr"], hp["b1"], hp["b2"],
                      hp["eps"], hp["wd"], 0.1, 0.001)
        dist.all_gather_into_tensor(p2, p2[lo:hi])

    tf, tl = _time(fused, a.iters), _time(library, a.iters)
    nv.check_status(dev)
    link = (world - 1) / world * n * 2          # incoming gradient slices; the outgoing parameter slices are equal
    hbm = per * (2 + 24 + 2) + (world - 1) / world * n * 2   # local grads, m/v/master read+write, params; peers' writes
    _report(rank, "rs_adamw_ag" + ("_multimem" if a.multicast and wg.multicast_ptr else "_p2p"), world, tf, tl, 0.0,
            link, {"bucket_bytes": n * 2}, hbm_bytes=hbm)


def bench_ag_gemm(a, rank, world, dev):
    """all-gather(rows of X) -> GEMM with a column shard of W (tensor-parallel fc1 / qkv)."""
    from fbamtrain_b200.ops import native as nv
    from fbamtrain_b200.ops import native_ops as no
    from fbamtrain_b200.parallel.tensor_parallel import TpContext
    tp = TpContext(None, dev, "fused")
    for m_full, k, n_out in a.shapes:
        rows = m_full // world
        x = torch.randn(rows, k, device=dev).to(BF)
        w = (torch.randn(n_out // world, k, device=dev) / k ** 0.5).to(BF)

        def fused():
            tp.ag_gemm(x, w, None, "none")

        def library():
            full = tp.all_gather_rows(x)
            no.gemm(full, w)

        tf, tl = _time(fused, a.iters), _time(library, a.iters)
        nv.check_status(dev)
        flops = 2.0 * m_full * k * (n_out // world)
        link = (world - 1) * rows * k * 2       # every other rank's shard comes in (and this one goes out)
        _report(rank, f"ag_gemm M{m_full} K{k} N{n_out}/{world}", world, tf, tl, flops, link)


def bench_gemm_rs(a, rank, world, dev):
    """GEMM with a row shard of W (K split) -> reduce-scatter over rows (tensor-parallel fc2 / out-proj), in both
    forms of the fused transport: partial tiles stored to the owners from the GEMM epilogue, and one GEMM per
    owner's block with copy-engine transfers under the next GEMM."""
    from fbamtrain_b200.ops import native as nv
    from fbamtrain_b200.ops import native_ops as no
    from fbamtrain_b200.parallel.tensor_parallel import TpContext
    contexts = {}
    for mode in ("epilogue", "chunked"):
        os.environ["FBAMTRAIN_TP_RS_MODE"] = mode
        contexts[mode] = TpContext(None, dev, "fused")
    os.environ.pop("FBAMTRAIN_TP_RS_MODE", None)
    # the epilogue form with 64 contiguous bytes per row and store instruction (lane-quad exchange)
    contexts["epilogue+row_stores"] = TpContext(None, dev, "fused")
    contexts["epilogue+row_stores"].rs_row_stores = True
    for m_full, k, n_out in a.shapes:
        kk = n_out // world                     # the K of this GEMM is the sharded hidden dimension
        h = torch.randn(m_full, kk, device=dev).to(BF)
        w = (torch.randn(k, kk, device=dev) / n_out ** 0.5).to(BF)
        tp = contexts["epilogue"]

        def library():
            tp.reduce_scatter_rows(no.gemm(h, w))

        tl = _time(library, a.iters)
        flops = 2.0 * m_full * kk * k
        link = (world - 1) / world * m_full * k * 2     # bf16 partial tiles stored into the owners' slots
        for mode, ctx in contexts.items():
            tf = _time(lambda: ctx.gemm_rs(h, w), a.iters)
            nv.check_status(dev)
            _report(rank, f"gemm_rs[{mode}] M{m_full} K{n_out}/{world} N{k}", world, tf, tl, flops, link)


def bench_muon(a, rank, world, dev):
    """Muon on one matrix per rank: gradient gather to the owner + Newton-Schulz + parameter broadcast."""
    from fbamtrain_b200.ops import native as nv
    from fbamtrain_b200.ops import native_ops as no
    from fbamtrain_b200.parallel.peer_window import PeerGroup
    r_, c_ = a.muon_shape
    n = r_ * c_
    peers = PeerGroup(None, dev)
    wg, wp = peers.allocate("g", n * world, BF), peers.allocate("p", n * world, BF)
    wg.local.normal_(std=1e-3)
    wp.local.normal_()
    mom = torch.zeros(n, device=dev)
    status = nv.status_word(dev)
    off = rank * n

    def barrier(slot):
        nv.check(nv.lib().fbam_peer_barrier(peers.flags.c_ptrs, rank, world, slot, C.c_uint(peers.next_epoch()),
                                            C.c_uint(1 << 22), nv.ptr(status), nv.stream_ptr()), "fbam_peer_barrier")

    def fused():
        barrier(6)
        u = torch.empty(n, dtype=BF, device=dev)
        sumsq = torch.zeros(1, device=dev)
        nv.check(nv.lib().fbam_reduce_pull(wg.c_ptrs, nv.ptr(mom), nv.ptr(u), nv.ptr(sumsq), C.c_longlong(off),
                                           C.c_longlong(off + n), 1, C.c_float(0.95), 1, C.c_float(1.0), world,
                                           nv.stream_ptr()), "fbam_reduce_pull")
        u2 = no.newton_schulz(u.view(r_, c_), 5, norm=sumsq.sqrt())
        wp.local[off:off + n].view(r_, c_).add_(u2, alpha=-1e-3)
        nv.check(nv.lib().fbam_push_shard(wp.c_ptrs, peers.flags.c_ptrs, C.c_longlong(off * 2),
                                          C.c_longlong((off + n) * 2), rank, world, 7, C.c_uint(peers.next_epoch()),
                                          nv.ptr(peers.arrive[2:]), nv.stream_ptr()), "fbam_push_shard")
        barrier(8)

    g2, p2 = wg.local.clone(), wp.local.clone()
    red = torch.empty(n, dtype=BF, device=dev)

    def library():
        dist.reduce_scatter_tensor(red, g2)
        gf = red.float()
        mom.mul_(0.95).add_(gf)
        u = (gf + 0.95 * mom).to(BF)
        u2 = no.newton_schulz(u.view(r_, c_), 5)
        mine = p2[off:off + n].view(r_, c_).add(u2, alpha=-1e-3)
        dist.all_gather_into_tensor(p2, mine.reshape(-1))

    tf, tl = _time(fused, a.iters), _time(library, a.iters)
    nv.check_status(dev)
    rr, cc = min(r_, c_), max(r_, c_)
    flops = 5.0 * (4.0 * rr * rr * cc + 2.0 * rr ** 3)
    link = (world - 1) * n * 2
    _report(rank, f"muon_gather_ns_push {r_}x{c_} per rank", world, tf, tl, flops, link)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--paths", default="rs_adamw_ag,ag_gemm,gemm_rs,muon")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--bucket-mib", type=int, default=256)
    ap.add_argument("--multicast", action="store_true", help="sum/broadcast through NVSwitch multicast (multimem)")
    ap.add_argument("--shapes", default="4096x2048x8192,16384x2048x8192,32768x4096x16384",
                    help="MxKxN of the tensor-parallel layer (rows of the full batch, model width, full hidden)")
    ap.add_argument("--muon-shape", default="2048x8192")
    a = ap.parse_args()
    a.shapes = [tuple(int(v) for v in s.split("x")) for s in a.shapes.split(",")]
    a.muon_shape = tuple(int(v) for v in a.muon_shape.split("x"))
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("launch with torch.distributed.run on at least 2 GPUs")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    table = {"rs_adamw_ag": bench_rs_adamw_ag, "ag_gemm": bench_ag_gemm, "gemm_rs": bench_gemm_rs, "muon": bench_muon}
    for name in a.paths.split(","):
        table[name](a, rank, world, dev)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
