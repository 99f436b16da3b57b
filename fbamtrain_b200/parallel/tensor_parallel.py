"""Tensor parallelism for the attention / MLP blocks of the action model (Megatron-style with
sequence-sharded activations between the parallel regions).

Activations between blocks are sharded by token rows; a *column-parallel* linear (fused QKV, MLP fc1) needs all
rows — all-gather → GEMM — and a *row-parallel* linear (attention out-projection, MLP fc2) produces partial sums
over the hidden shards — GEMM → reduce-scatter.  Two transports implement the two patterns:

``nccl``   ``all_gather_into_tensor`` / ``reduce_scatter_tensor`` around plain GEMMs (the baseline; also what
           runs on CPU ranks with gloo).
``fused``  the tcgen05 GEMM itself talks to peer memory (``csrc/gemm_tcgen05.cu``):
           *all-gather → GEMM*: every rank pushes its row shard into all peers' staging windows and raises a
           per-source flag; the consuming GEMM starts with its own rows and its TMA producer waits, tile by tile,
           for the flag of the shard a tile reads, so remote shards stream in underneath the math (the remote
           tile lands in local memory first — no TMA load ever targets a peer).
           *GEMM → reduce-scatter*: the epilogue adds each fp32 tile directly into the buffer of the rank that
           owns those rows (system-scope vector reductions over NVLink), so there is no separate collective.

The reference has no tensor parallelism (it shards positions of the sequence across frame-head workers
instead); the benchmark configurations ask for 4-way TP inside the action-model pipeline stage.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from ..models.blocks import AttentionBlock


class TpContext:
    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, transport: str = "nccl",
                 spin_limit: int = 1 << 22):
        if transport not in ("nccl", "fused"):
            raise ValueError("transport must be nccl or fused")
        self.group, self.device, self.transport = group, device, transport
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.spin_limit = spin_limit
        # GEMM -> reduce-scatter form of the fused transport: "epilogue" (partial tiles stored to the owners from
        # inside the GEMM) or "chunked" (one GEMM per owner's row block, each block copied to its owner by the copy
        # engines while the next GEMM runs)
        self.rs_mode = os.environ.get("FBAMTRAIN_TP_RS_MODE", "epilogue")
        if self.rs_mode not in ("epilogue", "chunked"):
            raise ValueError("FBAMTRAIN_TP_RS_MODE must be epilogue or chunked")
        # opt-in: 64-byte row pieces per store instruction in the reduce-scatter epilogue (see native_ops.gemm)
        self.rs_row_stores = os.environ.get("FBAMTRAIN_TP_RS_ROW_STORES", "0") == "1"
        self._copy_stream = None
        self.peers = None
        self._win: Dict[Tuple, object] = {}
        if transport == "fused":
            from .peer_window import PeerGroup
            self.peers = PeerGroup(group, device)

    # ---------------------------------------------------------------- library collectives
    def all_gather_rows(self, shard: torch.Tensor) -> torch.Tensor:
        full = torch.empty((shard.shape[0] * self.world,) + tuple(shard.shape[1:]), dtype=shard.dtype,
                           device=shard.device)
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        return full

    def reduce_scatter_rows(self, partial: torch.Tensor) -> torch.Tensor:
        out = torch.empty((partial.shape[0] // self.world,) + tuple(partial.shape[1:]), dtype=partial.dtype,
                          device=partial.device)
        dist.reduce_scatter_tensor(out, partial.contiguous(), group=self.group)
        return out

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.group)
        return t

    # ---------------------------------------------------------------- fused kernels
    def _window(self, kind: str, numel: int, dtype: torch.dtype):
        key = (kind, numel, dtype)
        if key not in self._win:
            self._win[key] = self.peers.allocate(f"tp/{kind}/{numel}/{dtype}", numel, dtype)
        return self._win[key]

    def _barrier(self, slot: int) -> None:
        from ..ops import native as nv
        epoch = self.peers.next_epoch()
        nv.check(nv.lib().fbam_peer_barrier(self.peers.flags.c_ptrs, self.rank, self.world, slot, C.c_uint(epoch),
                                            C.c_uint(self.spin_limit), nv.ptr(nv.status_word(self.device)),
                                            nv.stream_ptr()), "fbam_peer_barrier")

    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, bias, act: str, preact_out=None):
        """``act(all_gather(x_shard) · wᵀ + bias)``; returns the result and the gathered input."""
        from ..ops import native as nv
        from ..ops import native_ops as no
        rows, k = x_shard.shape
        win = self._window("ag", rows * self.world * k, x_shard.dtype)
        x_full = win.local.view(rows * self.world, k)
        self._barrier(2)                                   # everyone is done reading the previous contents
        x_full[self.rank * rows:(self.rank + 1) * rows].copy_(x_shard)
        epoch = self.peers.next_epoch()
        # The push runs BEFORE the GEMM on the same stream: a kernel that waits on flags must never share a GPU
        # with the (not yet scheduled) kernel that raises them.  What overlaps with the math is the arrival of
        # the OTHER ranks' shards: the GEMM starts with its own rows and waits per tile for remote ones.
        lo = self.rank * rows * k * x_shard.element_size()
        nv.check(nv.lib().fbam_push_shard(win.c_ptrs, self.peers.flags.c_ptrs, C.c_longlong(lo),
                                          C.c_longlong(lo + rows * k * x_shard.element_size()), self.rank,
                                          self.world, 3, C.c_uint(epoch), nv.ptr(self.peers.arrive[1:]),
                                          nv.stream_ptr()), "fbam_push_shard")
        from .peer_window import MAX_RANKS
        flags = self.peers.flags.local[3 * MAX_RANKS:4 * MAX_RANKS]
        m_full, n_out = rows * self.world, w.shape[0]
        tiles256 = ((m_full + 255) // 256) * ((n_out + 255) // 256)
        pair = n_out >= 256 and n_out % 16 == 0 and tiles256 >= 148       # CTA pairs: 256-row tiles
        tile_rows = 256 if pair or (tiles256 >= 296 and n_out >= 128) else 128
        y = no.gemm(x_full, w, bias=bias, act=act, preact_out=preact_out, ready_flags=flags, flag_rows=rows,
                    flag_epoch=epoch, flag_spin_limit=self.spin_limit, bm=tile_rows, two_cta=pair,
                    tile_m_rotate=(self.rank * rows) // tile_rows)
        return y, x_full.clone() if x_shard.requires_grad or w.requires_grad else x_full

    def gemm_rs(self, h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``reduce_scatter_rows(h · wᵀ)``: the GEMM epilogue stores every bf16 partial tile straight into this
        rank's slot of the buffer of the rank that owns the rows (plain vector stores over NVLink, remote owners
        first and in a different order on every rank so that no owner is written by two peers at once); one more
        kernel waits for all peers' tiles and sums the slots.  Returns this rank's rows in the operands' 16-bit type."""
        from ..ops import native as nv
        from ..ops import native_ops as no
        m, n = h.shape[0], w.shape[0]
        rows = m // self.world
        self._rs_round = getattr(self, "_rs_round", 0) + 1
        # two buffers in turn: a peer may still be summing the previous call's slots while this call's tiles arrive
        win = self._window(f"rs{self._rs_round & 1}", self.world * rows * n, h.dtype)
        if self.rs_mode == "chunked":
            return self._gemm_rs_chunked(h, w, win, rows, n)
        pair = n >= 256 and n % 16 == 0 and ((m + 255) // 256) * ((n + 255) // 256) >= 148
        tile_rows = 256 if pair else 128
        first = ((self.rank + 1) % self.world) * rows
        rotate = first // tile_rows if rows % tile_rows == 0 else 0
        no.gemm(h, w, out=_RsShape((m, n), h.dtype, n, win.local.data_ptr()), rs_out=list(win.ptrs),
                rs_rows_per_rank=rows, rs_slot=self.rank, tile_m_rotate=rotate, two_cta=pair, bm=tile_rows,
                rs_row_stores=self.rs_row_stores)
        out = torch.empty(rows, n, dtype=h.dtype, device=h.device)
        epoch = self.peers.next_epoch()
        nv.check(nv.lib(h).fbam_reduce_slots(nv.ptr(win.local), nv.ptr(out), C.c_longlong(rows * n), self.world,
                                            self.peers.flags.c_ptrs, self.rank, 5, C.c_uint(epoch),
                                            C.c_uint(self.spin_limit), nv.ptr(nv.status_word(self.device)),
                                            nv.stream_ptr()), "fbam_reduce_slots")
        return out

    def _gemm_rs_chunked(self, h: torch.Tensor, w: torch.Tensor, win, rows: int, n: int) -> torch.Tensor:
        """One GEMM per owner's block of rows (remote owners first, own block last, a different order on every
        rank); each finished block goes into this rank's slot of its owner's buffer as one peer-to-peer copy on a
        second stream — the copy engines move it while the tensor cores work on the next block — and the slot
        reduction waits for all peers as in the epilogue form."""
        from ..ops import native as nv
        from ..ops import native_ops as no
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        main = torch.cuda.current_stream()
        slot_elems = rows * n
        for i in range(self.world):
            owner = (self.rank + 1 + i) % self.world
            block = h[owner * rows:(owner + 1) * rows]
            if owner == self.rank:
                own = win.local[self.rank * slot_elems:(self.rank + 1) * slot_elems].view(rows, n)
                no.gemm(block, w, out=own)
                continue
            part = no.gemm(block, w)
            done = torch.cuda.Event()
            done.record(main)
            self._copy_stream.wait_event(done)
            dst = win.ptrs[owner] + self.rank * slot_elems * 2       # this rank's slot in the owner's buffer
            nv.check(nv.lib().fbam_copy_async(C.c_void_p(dst), nv.ptr(part), C.c_longlong(slot_elems * 2),
                                              C.c_void_p(self._copy_stream.cuda_stream)), "fbam_copy_async")
            part.record_stream(self._copy_stream)
        main.wait_stream(self._copy_stream)
        out = torch.empty(rows, n, dtype=h.dtype, device=h.device)
        epoch = self.peers.next_epoch()
        nv.check(nv.lib(h).fbam_reduce_slots(nv.ptr(win.local), nv.ptr(out), C.c_longlong(slot_elems), self.world,
                                            self.peers.flags.c_ptrs, self.rank, 5, C.c_uint(epoch),
                                            C.c_uint(self.spin_limit), nv.ptr(nv.status_word(self.device)),
                                            nv.stream_ptr()), "fbam_reduce_slots")
        return out


class _RsShape:
    """Stand-in output for the reduce-scatter GEMM: exposes shape, dtype, pitch and an address for the
    launcher's checks (the kernel writes to the owners' buffers instead)."""

    def __init__(self, shape, dtype, pitch: int, address: int):
        self.shape, self.dtype, self._pitch, self._address = torch.Size(shape), dtype, pitch, address

    def stride(self, i: int) -> int:
        return (self._pitch, 1)[i]

    def data_ptr(self) -> int:
        return self._address


# =================================================================================================
# autograd functions
# =================================================================================================
def _mm_nt(a, b, bias=None, act="none"):
    return ops.linear(a, b, bias, act)


class _ColumnParallel(torch.autograd.Function):
    """``y = act(AG_rows(x) · wᵀ + b)``; backward reduce-scatters the input gradient."""

    @staticmethod
    def forward(ctx, x_shard, w, b, tp: TpContext, act: str):
        fused = tp.transport == "fused" and x_shard.is_cuda
        preact = None
        if fused:
            if act == "gelu":
                preact = torch.empty((x_shard.shape[0] * tp.world, w.shape[0]), dtype=x_shard.dtype,
                                     device=x_shard.device)
            y, x_full = tp.ag_gemm(x_shard, w, b, act, preact)
        else:
            x_full = tp.all_gather_rows(x_shard)
            z = x_full.float() @ w.float().t() if not x_full.is_cuda else None
            if x_full.is_cuda:
                from ..ops import native_ops as no
                if act == "gelu":
                    preact = torch.empty((x_full.shape[0], w.shape[0]), dtype=x_full.dtype, device=x_full.device)
                y = no.gemm(x_full, w, bias=b, act=act, preact_out=preact)
            else:
                if b is not None:
                    z = z + b.float()
                preact = z.to(x_full.dtype) if act == "gelu" else None
                y = (torch.nn.functional.gelu(z) if act == "gelu" else z).to(x_full.dtype)
        ctx.save_for_backward(x_full, w, preact)
        ctx.tp, ctx.act, ctx.has_bias = tp, act, b is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, w, preact = ctx.saved_tensors
        tp: TpContext = ctx.tp
        dy = dy.contiguous()
        if ctx.act == "gelu":
            from ..ops import reference as ref
            dy = (dy.float() * ref.gelu_grad(preact)).to(dy.dtype)
        if dy.is_cuda:
            from ..ops import native_ops as no
            if tp.transport == "fused":
                dx = tp.gemm_rs(dy, w.t().contiguous())
            else:
                dx = tp.reduce_scatter_rows(no.gemm_nn(dy, w))
            dw = no.gemm_tn(dy, x_full)
            db = no._colsum(dy).to(dy.dtype) if ctx.has_bias else None
        else:
            dx = tp.reduce_scatter_rows((dy.float() @ w.float()).to(dy.dtype))
            dw = (dy.float().t() @ x_full.float()).to(w.dtype)
            db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return dx, dw, db, None, None


class _RowParallel(torch.autograd.Function):
    """``y_shard = RS_rows(h · wᵀ)``; backward all-gathers the output gradient."""

    @staticmethod
    def forward(ctx, h, w, tp: TpContext):
        if h.is_cuda:
            from ..ops import native_ops as no
            if tp.transport == "fused":
                y = tp.gemm_rs(h.contiguous(), w)
            else:
                y = tp.reduce_scatter_rows(no.gemm(h.contiguous(), w))
        else:
            y = tp.reduce_scatter_rows((h.float() @ w.float().t()).to(h.dtype))
        ctx.save_for_backward(h, w)
        ctx.tp = tp
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        h, w = ctx.saved_tensors
        tp: TpContext = ctx.tp
        if dy_shard.is_cuda:
            from ..ops import native_ops as no
            if tp.transport == "fused":
                dh, dy_full = tp.ag_gemm(dy_shard.contiguous(), w.t().contiguous(), None, "none")
            else:
                dy_full = tp.all_gather_rows(dy_shard)
                dh = no.gemm_nn(dy_full, w)
            dw = no.gemm_tn(dy_full, h)
        else:
            dy_full = tp.all_gather_rows(dy_shard)
            dh = (dy_full.float() @ w.float()).to(h.dtype)
            dw = (dy_full.float().t() @ h.float()).to(w.dtype)
        return dh, dw, None


# =================================================================================================
# tensor-parallel attention / MLP block
# =================================================================================================
class TensorParallelBlock(nn.Module):
    """One pre-norm attention + MLP block with heads and MLP columns split over the TP group.  Built from an
    unsharded :class:`AttentionBlock` so that both share initialisation (and tests can compare them).
    Input and output are row shards ``(B·T / tp, E)`` of the token matrix."""

    def __init__(self, block: AttentionBlock, tp: TpContext, batch: int, seq: int):
        super().__init__()
        self.tp, self.batch, self.seq = tp, batch, seq
        r, w = tp.rank, tp.world
        attn = block.attn
        e = attn.proj.weight.shape[0]
        self.heads_local = attn.n_head // w
        self.head_dim = e // attn.n_head
        if attn.n_head % w or (batch * seq) % w:
            raise ValueError("heads and tokens must divide by the tensor-parallel degree")
        self.causal = attn.causal
        hl, d = self.heads_local, self.head_dim
        qkv = attn.qkv.weight.detach().view(3, attn.n_head, d, e)[:, r * hl:(r + 1) * hl].reshape(3 * hl * d, e)
        self.w_qkv = nn.Parameter(qkv.clone())
        self.b_qkv = None
        if attn.qkv.bias is not None:
            self.b_qkv = nn.Parameter(attn.qkv.bias.detach().view(3, attn.n_head, d)[:, r * hl:(r + 1) * hl]
                                      .reshape(-1).clone())
        self.w_proj = nn.Parameter(attn.proj.weight.detach()[:, r * hl * d:(r + 1) * hl * d].clone())
        self.b_proj = nn.Parameter(attn.proj.bias.detach().clone()) if attn.proj.bias is not None else None
        f = block.mlp.fc1.weight.shape[0]
        fl = f // w
        self.w_fc1 = nn.Parameter(block.mlp.fc1.weight.detach()[r * fl:(r + 1) * fl].clone())
        self.b_fc1 = nn.Parameter(block.mlp.fc1.bias.detach()[r * fl:(r + 1) * fl].clone()) \
            if block.mlp.fc1.bias is not None else None
        self.w_fc2 = nn.Parameter(block.mlp.fc2.weight.detach()[:, r * fl:(r + 1) * fl].clone())
        self.b_fc2 = nn.Parameter(block.mlp.fc2.bias.detach().clone()) if block.mlp.fc2.bias is not None else None
        self.ln1_weight = nn.Parameter(block.ln1.weight.detach().clone())
        self.ln2_weight = nn.Parameter(block.ln2.weight.detach().clone())
        self.eps = block.ln1.eps

    # name -> (tensor of the unsharded block, how it is cut): "qkv" = per-head rows of the fused projection,
    # "rows" / "cols" = a contiguous range of rows / columns, None = replicated
    def _layout(self, block: AttentionBlock):
        attn, mlp = block.attn, block.mlp
        return [("w_qkv", attn.qkv.weight, "qkv"), ("b_qkv", attn.qkv.bias, "qkv"),
                ("w_proj", attn.proj.weight, "cols"), ("b_proj", attn.proj.bias, None),
                ("w_fc1", mlp.fc1.weight, "rows"), ("b_fc1", mlp.fc1.bias, "rows"),
                ("w_fc2", mlp.fc2.weight, "cols"), ("b_fc2", mlp.fc2.bias, None),
                ("ln1_weight", block.ln1.weight, None), ("ln2_weight", block.ln2.weight, None)]

    @torch.no_grad()
    def gather_into(self, block: AttentionBlock) -> None:
        """Writes the full parameters into the unsharded ``block`` (inverse of the constructor's slicing).
        Collective over the TP group."""
        w, hl, d = self.tp.world, self.heads_local, self.head_dim
        for name, full, cut in self._layout(block):
            mine = getattr(self, name)
            if mine is None or full is None:
                continue
            if cut is None:
                full.data.copy_(mine.data)
                continue
            parts = [torch.empty_like(mine.data) for _ in range(w)]
            dist.all_gather(parts, mine.data.contiguous(), group=self.tp.group)
            if cut == "qkv":      # rank r holds (3, hl, d, ...) of the (3, heads, d, ...) tensor
                tail = mine.shape[1:]
                merged = torch.cat([q.view(3, hl, d, *tail) for q in parts], dim=1)
                full.data.copy_(merged.reshape(full.shape))
            else:
                full.data.copy_(torch.cat(parts, dim=0 if cut == "rows" else 1))

    @torch.no_grad()
    def load_from(self, block: AttentionBlock) -> None:
        """Takes this rank's shards from the unsharded ``block`` again (after a checkpoint was loaded into it)."""
        r, w, hl, d = self.tp.rank, self.tp.world, self.heads_local, self.head_dim
        for name, full, cut in self._layout(block):
            mine = getattr(self, name)
            if mine is None or full is None:
                continue
            src = full.data
            if cut == "qkv":
                tail = src.shape[1:]
                src = src.view(3, w * hl, d, *tail)[:, r * hl:(r + 1) * hl].reshape(mine.shape)
            elif cut == "rows":
                n = mine.shape[0]
                src = src[r * n:(r + 1) * n]
            elif cut == "cols":
                n = mine.shape[1]
                src = src[:, r * n:(r + 1) * n]
            mine.data.copy_(src)

    def replicated_parameters(self):
        """Parameters every TP rank holds in full; their gradients are partial sums over row shards and must be
        all-reduced over the TP group after backward (:func:`sync_replicated_grads`)."""
        return [p for p in (self.ln1_weight, self.ln2_weight, self.b_proj, self.b_fc2) if p is not None]

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        tp = self.tp
        h = ops.rms_norm(x_shard, self.ln1_weight, self.eps)
        qkv = _ColumnParallel.apply(h, self.w_qkv, self.b_qkv, tp, "none")
        qkv = qkv.view(self.batch, self.seq, 3, self.heads_local, self.head_dim)
        o = ops.attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], self.causal)
        a = _RowParallel.apply(o.reshape(self.batch * self.seq, -1), self.w_proj, tp)
        if self.b_proj is not None:
            a = a + self.b_proj
        x_shard = x_shard + a
        h = ops.rms_norm(x_shard, self.ln2_weight, self.eps)
        u = _ColumnParallel.apply(h, self.w_fc1, self.b_fc1, tp, "gelu")
        m = _RowParallel.apply(u, self.w_fc2, tp)
        if self.b_fc2 is not None:
            m = m + self.b_fc2
        return x_shard + m


def sync_replicated_grads(blocks, tp: TpContext) -> None:
    for blk in blocks:
        for p in blk.replicated_parameters():
            if p.grad is not None:
                tp.all_reduce(p.grad)
