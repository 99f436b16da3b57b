"""Tensor-parallel block against the unsharded block on two CPU ranks (gloo)."""
import os
import socket

import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fbamtrain_b200.models.blocks import AttentionBlock
    from fbamtrain_b200.models.init_utils import SeedSequence
    from fbamtrain_b200.parallel.tensor_parallel import TensorParallelBlock, TpContext, sync_replicated_grads
    torch.manual_seed(0)
    b, t, e, heads, mlp = 2, 8, 32, 4, 64
    full = AttentionBlock(e, heads, mlp, True, True, 1e-5, torch.float32, SeedSequence(7))
    x = torch.randn(b, t, e, requires_grad=True)
    g = torch.randn(b, t, e)
    y = full(x)
    y.backward(g)
    tp = TpContext(None, torch.device("cpu"), "nccl")
    blk = TensorParallelBlock(full, tp, b, t)
    rows = b * t // world
    xs = x.detach().reshape(b * t, e)[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
    ys = blk(xs)
    ys.backward(g.reshape(b * t, e)[rank * rows:(rank + 1) * rows])
    sync_replicated_grads([blk], tp)
    errs = {}
    errs["y"] = float((ys - y.detach().reshape(b * t, e)[rank * rows:(rank + 1) * rows]).abs().max())
    errs["dx"] = float((xs.grad - x.grad.reshape(b * t, e)[rank * rows:(rank + 1) * rows]).abs().max())
    d, hl = e // heads, heads // world
    gq = full.attn.qkv.weight.grad.view(3, heads, d, e)[:, rank * hl:(rank + 1) * hl].reshape(3 * hl * d, e)
    errs["dw_qkv"] = float((blk.w_qkv.grad - gq).abs().max())
    errs["dw_proj"] = float((blk.w_proj.grad - full.attn.proj.weight.grad[:, rank * hl * d:(rank + 1) * hl * d]).abs().max())
    fl = mlp // world
    errs["dw_fc1"] = float((blk.w_fc1.grad - full.mlp.fc1.weight.grad[rank * fl:(rank + 1) * fl]).abs().max())
    errs["db_fc1"] = float((blk.b_fc1.grad - full.mlp.fc1.bias.grad[rank * fl:(rank + 1) * fl]).abs().max())
    errs["dw_fc2"] = float((blk.w_fc2.grad - full.mlp.fc2.weight.grad[:, rank * fl:(rank + 1) * fl]).abs().max())
    errs["db_fc2"] = float((blk.b_fc2.grad - full.mlp.fc2.bias.grad).abs().max())
    errs["dln1"] = float((blk.ln1_weight.grad - full.ln1.weight.grad).abs().max())
    errs["dln2"] = float((blk.ln2_weight.grad - full.ln2.weight.grad).abs().max())
    q.put((rank, errs))
    dist.destroy_process_group()


def test_tensor_parallel_block_matches_unsharded_block():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, errs in results:
        for k, v in errs.items():
            assert v < 2e-5, (rank, k, v)
