"""Data parallelism over flat gradient buckets.

Three ways to turn per-rank gradients into updated parameters, all with identical mathematics
(sum of gradients, no averaging — the loss is already divided by the global batch; reference:
``src/main.cpp:2501-2502, 3585-3659``):

``allreduce``  NCCL all-reduce of every bucket, then every rank runs the full optimizer (what the
               reference does; optimizer state is replicated).
``zero1``      NCCL reduce-scatter → AdamW on this rank's slice of m / v / master → NCCL all-gather of
               the parameters.  This is the library baseline of the fused path.
``fused``      one hand-written kernel per bucket (``csrc/comm.cu``: ``fbam_rs_adamw_ag``) reads this rank's slice
               of every peer's gradient bucket over NVLink, sums in fp32, applies AdamW to its slice and
               stores the rounded parameters into every peer's parameter bucket.  Buckets live in
               peer-memory windows; the action-model buckets are reduced on a side stream as soon as the
               action model's backward has finished, i.e. while the frame head's backward (the bulk of
               the step) is still running.

The buckets are the trainer's flat groups (frame-head 16-bit, frame-head fp32 embeddings,
action-model 16-bit, action-model fp32 LSTM), the grouping the reference uses for its all-reduces
(reference: ``src/main.cpp:745-807``).
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..optim import AdamwOptimizer
from ..utils.flat import FlatGroup
from ..utils.nvtx import gputx_range


class DataParallel:
    def __init__(self, mode: str = "allreduce", group: Optional[dist.ProcessGroup] = None,
                 use_multicast: bool = False, overlap: bool = True, spin_limit: int = 1 << 22,
                 window_transport: str = "symm"):
        if mode not in ("allreduce", "zero1", "fused"):
            raise ValueError("mode must be allreduce, zero1 or fused")
        self.mode, self.group = mode, group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self.use_multicast, self.overlap, self.spin_limit = use_multicast, overlap, spin_limit
        # "symm": torch's symmetric-memory allocator (multicast address available); "ipc": CUDA IPC handles exchanged
        # over the group, usable when the members of the group change while the job runs
        if window_transport not in ("symm", "ipc"):
            raise ValueError("window_transport must be symm or ipc")
        self.window_transport = window_transport
        self.peers = None
        self.grad_scale = 1.0
        self._windows: Dict[str, tuple] = {}
        self._side = None
        self.stats = {"bytes_reduced": 0}

    # ------------------------------------------------------------------------------------------
    def attach(self, trainer) -> None:
        """Called once by the trainer after the flat groups exist: broadcasts rank 0's parameters and,
        for the fused mode, moves every bucket into a peer-memory window."""
        for g in trainer.all_groups():
            dist.broadcast(g.data, src=self._global(0), group=self.group)
            if g.numel % self.world_size != 0:
                raise ValueError("flat groups must be padded to a multiple of the world size")
        for opt in self._adamw_optimizers(trainer):
            for fs, g in zip(opt.flat_state, opt.groups):
                if "master" in fs:
                    fs["master"].copy_(g.data.float())
        for opt in trainer.optimizers.values():       # per-parameter master copies (Muon, SGD)
            for sub in (opt, getattr(opt, "muon", None)):
                if sub is None or isinstance(sub, AdamwOptimizer) or not hasattr(sub, "named_params"):
                    continue
                for n, p in sub.named_params:
                    st = sub.state.get(n, {}) if isinstance(sub.state, dict) else {}
                    if "master" in st:
                        st["master"].copy_(p.data.float())
        if self.mode == "fused":
            if trainer.device.type != "cuda":
                raise ValueError("the fused mode needs CUDA peer memory")
            self._build_windows(trainer)
            self._side = torch.cuda.Stream(device=trainer.device)
            # Early start of the action-model buckets: count gradient accumulations of the action model's
            # parameters during the last micro-batch; when all have landed, the frame head's backward is
            # still ahead and the fused kernel can run beside it.
            self._am_params = [p for _, p in trainer.model.action_model.named_parameters() if p.requires_grad]
            self._pending = 0
            self._armed = False

            def _hook(_p, dp=self, tr=trainer):
                if not dp._armed:
                    return
                dp._pending -= 1
                if dp._pending == 0:
                    dp._armed = False
                    dp.action_model_grads_ready(tr)

            for p in self._am_params:
                p.register_post_accumulate_grad_hook(_hook)

    def attach_windows_only(self, trainer) -> None:
        """For callers that synchronise the parameters themselves (fault-tolerant DP): set up the peer windows
        and the early-start hooks without the initial broadcast."""
        if trainer.device.type != "cuda":
            raise ValueError("the fused mode needs CUDA peer memory")
        self._build_windows(trainer)
        self._side = torch.cuda.Stream(device=trainer.device)
        self._am_params = [p for _, p in trainer.model.action_model.named_parameters() if p.requires_grad]
        self._pending, self._armed, self.overlap = 0, False, False

    def _global(self, rank_in_group: int) -> int:
        return rank_in_group if self.group is None else dist.get_global_rank(self.group, rank_in_group)

    @staticmethod
    def _adamw_optimizers(trainer) -> List[AdamwOptimizer]:
        out = []
        for opt in trainer.optimizers.values():
            if isinstance(opt, AdamwOptimizer) and opt.groups is not None:
                out.append(opt)
            elif hasattr(opt, "adam") and isinstance(opt.adam, AdamwOptimizer) and opt.adam.groups is not None:
                out.append(opt.adam)
        return out

    def _build_windows(self, trainer) -> None:
        from .peer_window import IpcPeerGroup, PeerGroup
        if self.peers is None:
            cls = IpcPeerGroup if self.window_transport == "ipc" else PeerGroup
            self.peers = cls(self.group, trainer.device, self.use_multicast)
        self._windows.clear()
        for g in trainer.all_groups():
            wg = self.peers.allocate(g.name + "/grad", g.numel, g.dtype)
            wp = self.peers.allocate(g.name + "/param", g.numel, g.dtype)
            wp.local.copy_(g.data)
            wg.local.zero_()
            g.data, g.grad = wp.local, wg.local
            for n, p in g.named_params:                       # re-point parameters at the window
                o = g.offsets[n]
                p.data = g.data[o:o + p.numel()].view_as(p)
            g.rebind_grads()
            self._windows[g.name] = (wg, wp)
        torch.cuda.synchronize(trainer.device)
        dist.barrier(group=self.group)

    def rebuild(self, trainer, group: Optional[dist.ProcessGroup]) -> None:
        """After a membership change: adopt the new group and re-create the peer windows."""
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        self._owners = None               # the matrix-to-owner map of the fused Muon path depends on the world size
        if self.mode == "fused":
            # buckets are padded to the NOMINAL world; with fewer ranks the slice size must still divide
            for g in trainer.all_groups():
                if g.numel % self.world_size != 0:
                    raise ValueError(f"bucket '{g.name}' ({g.numel} elements) does not divide by world size "
                                     f"{self.world_size}; pad buckets to the least common multiple")
            saved = {g.name: g.data.clone() for g in trainer.all_groups()}
            self.peers.rebuild(group)
            self._build_windows(trainer)
            for g in trainer.all_groups():
                g.data.copy_(saved[g.name])

    # ------------------------------------------------------------------------------------------
    def reduce_and_step(self, trainer) -> bool:
        """Reduces gradients over the group and applies the optimizers.  Returns True (step committed)."""
        if self.mode == "fused":
            self._fused_step(trainer)
            return True
        if self.mode == "zero1":
            self._zero1_step(trainer)
            return True
        with gputx_range("fbamtrain::action_model_grad_allreduce"):
            for g in trainer.groups["action_model"]:
                dist.all_reduce(g.grad, group=self.group)
                self.stats["bytes_reduced"] += g.grad.numel() * g.grad.element_size()
        with gputx_range("fbamtrain::frame_head_grad_allreduce"):
            for g in trainer.groups["frame_head"]:
                dist.all_reduce(g.grad, group=self.group)
                self.stats["bytes_reduced"] += g.grad.numel() * g.grad.element_size()
        with gputx_range("fbamtrain::action_model_optim_step"):
            trainer.optimizers["action_model"].step()
        with gputx_range("fbamtrain::frame_head_optim_step"):
            trainer.optimizers["frame_head"].step()
        return True

    def _zero1_step(self, trainer) -> None:
        shard = (self.rank, self.world_size)
        for opt in self._adamw_optimizers(trainer):
            for g in opt.groups:
                per = g.numel // self.world_size
                reduced = torch.empty(per, dtype=g.grad.dtype, device=g.grad.device)   # must not alias the input
                dist.reduce_scatter_tensor(reduced, g.grad, group=self.group)
                g.grad[self.rank * per:(self.rank + 1) * per].copy_(reduced)
            opt.step(shard=shard)
            for g in opt.groups:
                per = g.numel // self.world_size
                dist.all_gather_into_tensor(g.data, g.data[self.rank * per:(self.rank + 1) * per].clone(),
                                            group=self.group)
        self._step_non_adamw(trainer)

    # -- Muon over peer memory --------------------------------------------------------------------
    def _muon_owner_map(self, muon):
        """Greedy balance of the matrices over the ranks (largest first); identical on every rank."""
        if getattr(self, "_owners", None) is None:
            self._owners = {}
        key = id(muon)
        if key not in self._owners:
            load = [0] * self.world_size
            owners = {}
            for name, p in sorted(muon.named_params, key=lambda np_: -np_[1].numel()):
                r = min(range(self.world_size), key=lambda i: (load[i], i))
                owners[name] = r
                load[r] += p.numel()
            self._owners[key] = owners
        return self._owners[key]

    def _fused_muon(self, trainer, muon, groups) -> None:
        """Muon under data parallelism without NCCL: the owner of each matrix pulls and sums all peers' gradients
        for it (fused with the momentum update, the bf16 cast and Σx²), orthogonalises it with Newton–Schulz on
        the tensor-core GEMM, updates its master copy and pushes the new parameter into every peer's window."""
        from ..ops import native as nv
        from ..ops.native_ops import newton_schulz as native_ns
        dev = trainer.device
        owners = self._muon_owner_map(muon)
        by_param = {}
        for g in groups:
            for n, p in g.named_params:
                by_param[n] = (g, g.offsets[n])
        muon.step_count += 1
        flags = self.peers.flags.c_ptrs
        status = nv.ptr(nv.status_word(dev))
        # Every rank must tag the same event with the same epoch although each pushes only the matrices it owns:
        # the step reserves one epoch per matrix (in the optimizer's order) plus two for its barriers.
        ordered = [name for name, _ in muon.named_params]
        base = self.peers.epoch
        self.peers.epoch = base + len(ordered) + 2

        def barrier(slot, epoch):
            nv.check(nv.lib().fbam_peer_barrier(flags, self.rank, self.world_size, slot, C.c_uint(epoch),
                                                C.c_uint(self.spin_limit), status, nv.stream_ptr()),
                     "fbam_peer_barrier")

        barrier(6, base + 1)                         # every rank's gradients are complete
        for index, (name, p) in enumerate(muon.named_params):
            if owners[name] != self.rank:
                continue
            g, off = by_param[name]
            wg, wp = self._windows[g.name]
            n = p.numel()
            is_elem = g.dtype in nv.ELEM_DTYPES
            esize = 2 if is_elem else 4
            if (not is_elem and g.dtype != torch.float32) or n % (16 // esize) != 0:
                raise ValueError(f"fused Muon needs bf16/fp16/fp32 matrices whose size is a multiple of 16 bytes ('{name}')")
            buf = muon.state[name]["momentum"].view(-1)
            u = torch.empty(n, dtype=g.dtype if is_elem else torch.bfloat16, device=dev)
            sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
            nv.check(nv.lib(g.dtype).fbam_reduce_pull(wg.c_ptrs, nv.ptr(buf), nv.ptr(u), nv.ptr(sumsq), C.c_longlong(off),
                                               C.c_longlong(off + n), int(is_elem), C.c_float(muon.momentum),
                                               int(muon.nesterov), C.c_float(self.grad_scale), self.world_size,
                                               nv.stream_ptr()),
                     "fbam_reduce_pull")
            u2 = native_ns(u.view(p.shape[0], -1), muon.ns_steps, norm=sumsq.sqrt())
            muon.apply_update(name, p, u2)          # writes the local window (p.data is a view of it)
            lo_b = off * esize
            nv.check(nv.lib().fbam_push_shard(wp.c_ptrs, flags, C.c_longlong(lo_b), C.c_longlong(lo_b + n * esize),
                                              self.rank, self.world_size, 7, C.c_uint(base + 2 + index),
                                              nv.ptr(self.peers.arrive[2:]), nv.stream_ptr()), "fbam_push_shard")
            self.stats["bytes_reduced"] += n * esize
        barrier(8, base + len(ordered) + 2)          # all pushes have landed everywhere

    def _step_non_adamw(self, trainer) -> None:
        """Optimizers without a sharded form (SGD, Muon matrices): all-reduce their buckets, step replicated —
        except Muon in the fused mode, which runs matrix-parallel over peer memory."""
        handled = {id(g) for opt in self._adamw_optimizers(trainer) for g in opt.groups}
        if self.mode == "fused":
            for scope, opt in trainer.optimizers.items():
                if hasattr(opt, "muon") and opt.muon.named_params:
                    groups = [g for g in trainer.groups[scope] if id(g) not in handled]
                    opt.step_count += 1
                    self._fused_muon(trainer, opt.muon, groups)
                    handled.update(id(g) for g in groups)
                    if not (isinstance(opt.adam, AdamwOptimizer) and opt.adam.groups is not None):
                        opt.adam.step()
            if all(id(g) in handled for g in trainer.all_groups()):
                return
        for g in trainer.all_groups():
            if id(g) not in handled:
                dist.all_reduce(g.grad, group=self.group)
        for opt in trainer.optimizers.values():
            if isinstance(opt, AdamwOptimizer):
                continue
            if hasattr(opt, "muon") and self.mode == "fused":
                continue
            if hasattr(opt, "muon"):
                opt.step_count += 1
                opt.muon.step()
                if not (isinstance(opt.adam, AdamwOptimizer) and opt.adam.groups is not None):
                    opt.adam.step()
            else:
                opt.step()

    # -- fused path ----------------------------------------------------------------------------
    def launch_fused_bucket(self, opt: AdamwOptimizer, g: FlatGroup, fs, bc1: float, bc2: float, device) -> None:
        from ..ops import native as nv
        wg, wp = self._windows[g.name]
        per = g.numel // self.world_size
        lo, hi = self.rank * per, (self.rank + 1) * per
        epoch = self.peers.next_epoch()
        is_elem = g.dtype in nv.ELEM_DTYPES
        if not is_elem and g.dtype != torch.float32:
            raise TypeError("fused buckets are bf16, fp16 or fp32")
        master = fs.get("master")
        code = nv.lib(g.dtype).fbam_rs_adamw_ag(
            wg.c_ptrs, wp.c_ptrs, self.peers.flags.c_ptrs,
            C.c_void_p(wg.multicast_ptr), C.c_void_p(wp.multicast_ptr),
            nv.ptr(fs["m"]), nv.ptr(fs["v"]), nv.ptr(master), C.c_longlong(lo), C.c_longlong(hi), int(is_elem),
            C.c_float(opt.lr), C.c_float(opt.beta1), C.c_float(opt.beta2), C.c_float(opt.eps),
            C.c_float(opt.weight_decay), C.c_float(bc1), C.c_float(bc2), C.c_float(self.grad_scale), self.rank,
            self.world_size,
            C.c_uint(epoch), 1, C.c_uint(self.spin_limit), nv.ptr(nv.status_word(device)), nv.ptr(self.peers.arrive),
            0, nv.stream_ptr())
        nv.check(code, "fbam_rs_adamw_ag")
        self.stats["bytes_reduced"] += g.numel * g.grad.element_size()

    def _fused_scope(self, trainer, scope: str) -> None:
        opt = trainer.optimizers[scope]
        adam = opt if isinstance(opt, AdamwOptimizer) else getattr(opt, "adam", None)
        if not (isinstance(adam, AdamwOptimizer) and adam.groups is not None):
            return
        adam.step_count += 1
        bc1 = 1.0 - adam.beta1 ** adam.step_count
        bc2 = 1.0 - adam.beta2 ** adam.step_count
        for g, fs in zip(adam.groups, adam.flat_state):
            self.launch_fused_bucket(adam, g, fs, bc1, bc2, trainer.device)

    def arm(self) -> None:
        """Called by the trainer right before the backward pass of the step's last micro-batch."""
        if self.mode == "fused" and self.overlap:
            self._pending = len(self._am_params)
            self._armed = True

    def action_model_grads_ready(self, trainer) -> None:
        """Hook: the action model's backward is complete while the frame head's is still to run.  Starts
        the fused reduce-scatter / AdamW / all-gather of the action-model buckets on the side stream."""
        if self.mode != "fused" or not self.overlap:
            return
        self._side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._side), gputx_range("fbamtrain::action_model_grad_allreduce"):
            self._fused_scope(trainer, "action_model")
        self._early = True

    def _fused_step(self, trainer) -> None:
        cur = torch.cuda.current_stream()
        if getattr(self, "_early", False):
            # The action-model buckets went out on the side stream under the frame head's backward.  All fused
            # kernels share the entry/exit flag slots, so the frame head's buckets queue behind them rather than
            # beside them (by now the side stream has long finished; this only fixes the order).
            cur.wait_stream(self._side)
            self._early = False
        else:
            with gputx_range("fbamtrain::action_model_grad_allreduce"):
                self._fused_scope(trainer, "action_model")
        with gputx_range("fbamtrain::frame_head_grad_allreduce"):
            self._fused_scope(trainer, "frame_head")
        self._step_non_adamw(trainer)

    # ------------------------------------------------------------------------------------------
    def gather_optimizer_state(self, trainer) -> None:
        """Before a checkpoint: make every rank's m / v / master complete (each rank only maintains its slice)."""
        if self.mode == "allreduce":
            return
        for opt in self._adamw_optimizers(trainer):
            for g, fs in zip(opt.groups, opt.flat_state):
                per = g.numel // self.world_size
                for t in fs.values():
                    dist.all_gather_into_tensor(t, t[self.rank * per:(self.rank + 1) * per].clone(), group=self.group)
        if self.mode == "fused":
            for opt in trainer.optimizers.values():
                if hasattr(opt, "muon"):
                    owners = self._muon_owner_map(opt.muon)
                    for name, _ in opt.muon.named_params:
                        for t in opt.muon.state[name].values():
                            dist.broadcast(t, src=self._global(owners[name]), group=self.group)


def recover_sharded_state(tensors_with_fallback, old: Optional[tuple], group: Optional[dist.ProcessGroup]) -> int:
    """After a membership change of a group whose members each maintained only a slice of some flat state tensors
    (the sharded AdamW moments and fp32 masters of the fused / ZeRO-1 modes): make every member hold all of it again.

    ``tensors_with_fallback``: list of ``(tensor, fallback)``; ``tensor`` is a flat state tensor of which this
    member's OLD slice ``[old_rank · n/old_world, (old_rank + 1) · n/old_world)`` is current; ``fallback`` is
    ``None`` (slices whose owner is gone restart from zero — Adam moments) or a tensor of the same length to take
    them from (masters: the current low-precision parameters, which every member holds).  ``old = (old_rank,
    old_world)``, or ``None`` for a member that just joined and owns nothing.  Collective over ``group``.
    Returns the number of old slices that had no surviving owner."""
    world = dist.get_world_size(group)
    everyone: List[Optional[tuple]] = [None] * world
    dist.all_gather_object(everyone, old, group=group)
    known = [o for o in everyone if o is not None]
    if not known:
        return 0
    old_world = known[0][1]
    if any(o[1] != old_world for o in known):
        raise ValueError("members disagree about the previous world size")
    covered = {o[0] for o in known}
    lost = [r for r in range(old_world) if r not in covered]
    for t, fallback in tensors_with_fallback:
        n = t.numel()
        per = n // old_world
        mine = torch.zeros_like(t)
        if old is not None:
            lo, hi = old[0] * per, (old[0] + 1) * per
            mine[lo:hi] = t[lo:hi]
        dist.all_reduce(mine, group=group)
        if fallback is not None:
            for r in lost:
                mine[r * per:(r + 1) * per] = fallback[r * per:(r + 1) * per].to(mine.dtype)
        t.copy_(mine)
    return len(lost)
