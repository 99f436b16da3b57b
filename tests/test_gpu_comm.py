"""Fused communication kernels: arithmetic on one GPU (several emulated ranks, no cross-rank waits) and the
real peer-memory path on two GPUs when the machine has them."""
import ctypes as C
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _nv():
    from fbamtrain_b200.ops import native
    return native


@pytest.mark.parametrize("dtype", [BF, torch.float16, torch.float32])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_rs_adamw_ag_emulated_ranks(dtype, world):
    from fbamtrain_b200.parallel.peer_window import LocalPeerGroup
    nv = _nv()
    torch.manual_seed(0)
    n = 8 * 1024 * world + 8 * world * 3
    peers = LocalPeerGroup(world, torch.device(DEV))
    grads = peers.allocate("g", n, dtype)
    params = peers.allocate("p", n, dtype)
    master0 = torch.randn(n, device=DEV)
    for w in params:
        w.local.copy_(master0.to(dtype))
    gsum = torch.zeros(n, device=DEV)
    for w in grads:
        g = torch.randn(n, device=DEV).to(dtype)
        w.local.copy_(g)
        gsum += g.float()
    m = [torch.rand(n, device=DEV) * 0.1 for _ in range(world)]
    v = [torch.rand(n, device=DEV) * 0.01 for _ in range(world)]
    m[1:] = [m[0].clone() for _ in range(world - 1)]
    v[1:] = [v[0].clone() for _ in range(world - 1)]
    masters = [master0.to(dtype).float().clone() if dtype != torch.float32 else None for _ in range(world)]
    em, ev = m[0].clone(), v[0].clone()
    ew = master0.to(dtype).float().clone()
    lr, b1, b2, eps, wd, step = 1e-2, 0.9, 0.99, 1e-8, 0.1, 2
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    per = n // world
    status = nv.status_word(torch.device(DEV))
    for r in range(world):
        code = nv.lib(dtype).fbam_rs_adamw_ag(
            grads[r].c_ptrs, params[r].c_ptrs, None, None, None, nv.ptr(m[r]), nv.ptr(v[r]), nv.ptr(masters[r]),
            C.c_longlong(r * per), C.c_longlong((r + 1) * per), int(dtype != torch.float32), C.c_float(lr), C.c_float(b1),
            C.c_float(b2), C.c_float(eps), C.c_float(wd), C.c_float(bc1), C.c_float(bc2), C.c_float(1.0), r, world,
            C.c_uint(1), 0, C.c_uint(1000), nv.ptr(status), nv.ptr(peers.arrive), 0, nv.stream_ptr())
        nv.check(code, "fbam_rs_adamw_ag")
    nv.check_status(torch.device(DEV))
    ew.mul_(1 - lr * wd)
    em.mul_(b1).add_(gsum, alpha=1 - b1)
    ev.mul_(b2).addcmul_(gsum, gsum, value=1 - b2)
    ew.addcdiv_(em / bc1, (ev / bc2).sqrt() + eps, value=-lr)
    expect = ew.to(dtype)
    for r in range(world):
        assert torch.allclose(params[r].local.float(), expect.float(), atol=1e-5 if dtype == torch.float32 else 8e-3), r
        assert torch.equal(params[r].local, params[0].local)
        sl = slice(r * per, (r + 1) * per)
        assert torch.allclose(m[r][sl], em[sl], atol=1e-6) and torch.allclose(v[r][sl], ev[sl], atol=1e-6)


def test_reduce_pull_and_push_shard_emulated():
    from fbamtrain_b200.parallel.peer_window import LocalPeerGroup, FLAG_SLOTS, MAX_RANKS
    nv = _nv()
    torch.manual_seed(1)
    world, n = 4, 4096
    peers = LocalPeerGroup(world, torch.device(DEV))
    grads = peers.allocate("g", n, BF)
    total = torch.zeros(n, device=DEV)
    for w in grads:
        g = torch.randn(n, device=DEV).to(BF)
        w.local.copy_(g)
        total += g.float()
    lo, hi = 512, 2048
    buf = torch.randn(hi - lo, device=DEV)
    expect_buf = 0.9 * buf + 0.1 * total[lo:hi]              # moving average, as the reference keeps it
    out = torch.empty(hi - lo, device=DEV, dtype=BF)
    sumsq = torch.zeros(1, device=DEV)
    nv.check(nv.lib().fbam_reduce_pull(grads[0].c_ptrs, nv.ptr(buf), nv.ptr(out), nv.ptr(sumsq), C.c_longlong(lo),
                                       C.c_longlong(hi), 1, C.c_float(0.9), 1, C.c_float(1.0), world,
                                       nv.stream_ptr()), "fbam_reduce_pull")
    u = 0.1 * total[lo:hi] + 0.9 * expect_buf
    assert torch.allclose(buf, expect_buf, atol=1e-5)
    assert torch.allclose(out.float(), u, atol=3e-2, rtol=1e-2)
    assert abs(float(sumsq) - float((u * u).sum())) / float((u * u).sum()) < 1e-3
    # push: rank 2's slice lands in every buffer and its flag is raised everywhere
    bufs = peers.allocate("b", n, BF)
    flags = peers.allocate("f", FLAG_SLOTS * MAX_RANKS, torch.int32)
    bufs[2].local.copy_(torch.randn(n, device=DEV).to(BF))
    nv.check(nv.lib().fbam_push_shard(bufs[2].c_ptrs, flags[2].c_ptrs, C.c_longlong(1024), C.c_longlong(4096), 2,
                                      world, 3, C.c_uint(7), nv.ptr(peers.arrive), nv.stream_ptr()), "fbam_push_shard")
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(bufs[r].local[512:2048], bufs[2].local[512:2048])
        assert int(flags[r].local[3 * MAX_RANKS + 2]) == 7
        if r != 2:
            assert float(bufs[r].local[:512].abs().max()) == 0.0


def test_bounded_wait_reports_timeout_and_context_survives():
    """A wait on a flag that nobody sets must end in a status code, not a hang."""
    from fbamtrain_b200.parallel.peer_window import FLAG_SLOTS, MAX_RANKS
    nv = _nv()
    dev = torch.device(DEV)
    flags = torch.zeros(FLAG_SLOTS * MAX_RANKS, dtype=torch.int32, device=DEV)
    status = nv.status_word(dev)
    status.zero_()
    nv.check(nv.lib().fbam_wait_flags(nv.ptr(flags), 0, 2, C.c_uint(5), C.c_uint(2000), nv.ptr(status),
                                      nv.stream_ptr()), "fbam_wait_flags")
    torch.cuda.synchronize()
    code = int(status.item())
    assert code % 1000 == 301 and code // 1000 == 1      # timed out waiting for rank 0
    status.zero_()
    x = torch.ones(8, device=DEV)
    assert float((x * 2).sum()) == 16.0                  # the context is still usable


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("variant", ["p2p", "multicast", "muon", "ipc"])
def test_fused_dp_matches_nccl_zero1_on_two_gpus(tmp_path, variant):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = tmp_path / "result.txt"
    worker = os.path.join(os.path.dirname(__file__), "workers", "dp_fused_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), worker, str(out)]
    if variant != "p2p":
        cmd.append(variant)
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, _tail(r)
    assert out.read_text() == "ok"


def _tail(r):
    """The part of a child's output that holds the Python traceback (torchrun appends a long banner after it)."""
    text = r.stdout + r.stderr
    i = text.find("Traceback")
    return text[i:i + 4000] if i >= 0 else text[-4000:]


@pytest.mark.parametrize("rs_mode", ["epilogue", "chunked"])
def test_fused_tensor_parallel_block_matches_nccl_on_two_gpus(tmp_path, rs_mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    if rs_mode == "chunked" and os.environ.get("FBAMTRAIN_TEST_OPT_IN_PATHS") != "1":
        pytest.skip("the chunked reduce-scatter is an opt-in path; set FBAMTRAIN_TEST_OPT_IN_PATHS=1 to test it")
    out = tmp_path / "result.txt"
    worker = os.path.join(os.path.dirname(__file__), "workers", "tp_fused_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), worker, str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, FBAMTRAIN_TP_RS_MODE=rs_mode))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert out.read_text() == "ok"


def test_flag_gated_gemm_and_reduce_scatter_epilogue_single_gpu():
    """The gated producer with flags already raised, and the reduce-scatter epilogue with every 'peer' buffer
    on this device (one rank's launch at a time, no cross-rank waits)."""
    from fbamtrain_b200.ops import native_ops as no
    nv = _nv()
    torch.manual_seed(3)
    m, n, k, world = 512, 384, 256, 4
    a = torch.randn(m, k, device=DEV).to(BF)
    b = torch.randn(n, k, device=DEV).to(BF)
    expect = a.float() @ b.float().t()
    flags = torch.full((8,), 9, dtype=torch.int32, device=DEV)
    y = no.gemm(a, b, ready_flags=flags, flag_rows=m // world, flag_epoch=9, flag_spin_limit=100, tile_m_rotate=2)
    assert float((y.float() - expect).norm() / expect.norm()) < 5e-3
    # a flag that is never raised: the producer gives up, the kernel unwinds, the status word says so
    status = nv.status_word(torch.device(DEV))
    status.zero_()
    flags.fill_(1)
    no.gemm(a, b, ready_flags=flags, flag_rows=m // world, flag_epoch=5, flag_spin_limit=50)
    torch.cuda.synchronize()
    assert int(status.item()) in (101, 102, 103)
    status.zero_()
    # the same two cases on the CTA-pair kernel (each CTA of a pair waits for the rows its own loads read)
    flags.fill_(9)
    y = no.gemm(a, b, ready_flags=flags, flag_rows=m // world, flag_epoch=9, flag_spin_limit=100, tile_m_rotate=1,
                two_cta=True)
    assert float((y.float() - expect).norm() / expect.norm()) < 5e-3
    flags.fill_(1)
    no.gemm(a, b, ready_flags=flags, flag_rows=m // world, flag_epoch=5, flag_spin_limit=50, two_cta=True)
    torch.cuda.synchronize()
    assert int(status.item()) in (101, 102, 103)
    status.zero_()
    # reduce-scatter epilogue: two "ranks" contribute partial products into four owners' buffers
    rows = m // world
    owners = [torch.zeros(rows, n, device=DEV) for _ in range(world)]
    from fbamtrain_b200.parallel.tensor_parallel import _RsShape
    for part in range(2):
        ap, bp = a[:, part * 128:(part + 1) * 128].contiguous(), b[:, part * 128:(part + 1) * 128].contiguous()
        shape = _RsShape((m, n), torch.float32, n, owners[0].data_ptr())
        no.gemm(ap, bp, out=shape, rs_out=[o.data_ptr() for o in owners], rs_rows_per_rank=rows)
    nv.check_status(torch.device(DEV))
    got = torch.cat(owners, 0)
    assert float((got - expect).norm() / expect.norm()) < 5e-3
    # slot form: each "rank" stores its bf16 partial tiles into its slot of the owners' buffers, the owners sum
    import ctypes as C
    for pair in (False, True):
        slots = [torch.zeros(2, rows, n, device=DEV, dtype=BF) for _ in range(world)]
        for part in range(2):
            ap, bp = a[:, part * 128:(part + 1) * 128].contiguous(), b[:, part * 128:(part + 1) * 128].contiguous()
            shape = _RsShape((m, n), BF, n, slots[0].data_ptr())
            no.gemm(ap, bp, out=shape, rs_out=[o.data_ptr() for o in slots], rs_rows_per_rank=rows, rs_slot=part,
                    tile_m_rotate=1, two_cta=pair, bm=256 if pair else 128)
        outs = []
        for o in slots:
            red = torch.empty(rows, n, device=DEV, dtype=BF)
            nv.check(nv.lib().fbam_reduce_slots(nv.ptr(o), nv.ptr(red), C.c_longlong(rows * n), 2, None, 0, 0,
                                                C.c_uint(0), C.c_uint(0), nv.ptr(status), nv.stream_ptr()),
                     "fbam_reduce_slots")
            outs.append(red)
        nv.check_status(torch.device(DEV))
        got = torch.cat(outs, 0).float()
        assert float((got - expect).norm() / expect.norm()) < 1e-2


@pytest.mark.parametrize("pair", [False, True])
def test_reduce_scatter_row_stores_single_gpu(pair):
    """The opt-in store pattern of the slot epilogue (lane quads exchange pieces, 64 contiguous bytes per row and
    instruction) must write exactly what the default pattern writes; every 'peer' buffer is on this device."""
    if os.environ.get("FBAMTRAIN_TEST_OPT_IN_PATHS") != "1":
        pytest.skip("opt-in path; set FBAMTRAIN_TEST_OPT_IN_PATHS=1 to test it")
    from fbamtrain_b200.ops import native_ops as no
    from fbamtrain_b200.parallel.tensor_parallel import _RsShape
    nv = _nv()
    if not nv.lib().fbam_has_rs_row_stores():
        pytest.skip("library built without the row-store epilogue (FBAMTRAIN_RS_ROW_STORES=1 python -m "
                    "fbamtrain_b200.build --force)")
    torch.manual_seed(5)
    m, n, k, world = 1024, 512, 192, 4
    rows = m // world
    a = torch.randn(m, k, device=DEV).to(BF)
    b = torch.randn(n, k, device=DEV).to(BF)
    results = []
    for row_stores in (False, True):
        slots = [torch.zeros(3, rows, n, device=DEV, dtype=BF) for _ in range(world)]
        shape = _RsShape((m, n), BF, n, slots[0].data_ptr())
        no.gemm(a, b, out=shape, rs_out=[o.data_ptr() for o in slots], rs_rows_per_rank=rows, rs_slot=1,
                tile_m_rotate=1, two_cta=pair, bm=256 if pair else 128, rs_row_stores=row_stores)
        nv.check_status(torch.device(DEV))
        results.append(torch.stack(slots, 0))
    assert torch.equal(results[0], results[1])
    expect = (a.float() @ b.float().t()).view(world, rows, n)
    got = results[1][:, 1].float()
    assert float((got - expect).norm() / expect.norm()) < 1e-2
    assert float(results[1][:, 0].abs().max()) == 0.0 and float(results[1][:, 2].abs().max()) == 0.0


def test_scoped_group_next_to_the_default_group_on_two_gpus(tmp_path):
    """The stand-alone NCCL communicator that pipelines with dynamic membership build per position
    (``parallel/ft_pipeline.py``): collectives, object exchange and the shared-state comparison on two GPUs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = tmp_path / "result.txt"
    worker = os.path.join(os.path.dirname(__file__), "workers", "scoped_group_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), worker, str(out), str(_free_port())]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, _tail(r)
    assert out.read_text() == "ok"


def test_cli_pipelines_with_dynamic_membership_on_four_gpus(tmp_path):
    """Two one-plus-one pipelines, each a job of its own on its own pair of GPUs, under the membership master
    (``frame_head_parallel`` + ``ddp_parallel.transport = "ftccl"``): same-position ranks exchange gradients over their
    stand-alone NCCL communicators, and once both pipelines are in the group they report the same committed losses."""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs four GPUs")
    import json
    from fbamtrain_b200 import presets
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = presets.tiny("bf16")
    cfg["model_config"].update({"action_heads": 2, "lstm_layers": 1, "cell_embed_dim": 64, "downsample_channels": [64],
                                "n_embed": 64})
    cfg["micro_batch_size"], cfg["total_batch_size"] = 1, 2
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    ports = [_free_port(), _free_port()]
    par = {"frame_head_parallel": {"use_frame_head_parallel": True, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": ports[0]}},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ftccl",
                            "ftccl_master": {"ip": "127.0.0.1", "port": ports[1]}}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    env = dict(os.environ, PYTHONPATH=root, FBAMTRAIN_LOG_LEVEL="INFO", FBAMTRAIN_METRICS_JSON="1",
               NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    master = subprocess.Popen([sys.executable, "-m", "fbamtrain_b200.cli", "--parallel-config", str(parallel),
                               "--ftccl-master"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    procs = []
    try:
        base = [sys.executable, "-m", "fbamtrain_b200.cli", "-c", str(run), "--parallel-config", str(parallel),
                "--synthetic", "--steps", "8", "--world-size", "2", "--ddp-world-size", "2"]
        for replica in (0, 1):
            for worker, extra in ((0, []), (1, ["--master"])):
                procs.append(subprocess.Popen(
                    base + ["--replica-id", str(replica), "--worker_id", str(worker), "--device",
                            f"cuda:{2 * replica + worker}"] + extra,
                    stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env))
        outs = []
        for p in procs:
            try:
                outs.append(p.communicate(timeout=420)[0])
            except subprocess.TimeoutExpired:
                p.kill()                                   # this very process, by its handle
                outs.append(p.communicate()[0])
        assert all(p.returncode == 0 for p in procs), [o[-1500:] for o in outs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        master.terminate()
        master.communicate(timeout=30)

    def losses(out):
        rows = [json.loads(line) for line in out.splitlines() if line.startswith("{") and "loss/train" in line]
        return {r["step"]: r["loss/train"] for r in rows}
    first, second = losses(outs[1]), losses(outs[3])
    both = sorted(set(first) & set(second))
    assert len(both) >= 3
    assert all(abs(first[k] - second[k]) < 1e-5 for k in both[-3:])
