"""Two-stage pipeline: frame head on the first group of ranks, action model on the second.

The reference's closest mode is *frame-head parallel*: workers own positions of the sequence, run the frame head
for them and ``ncclSend`` the embeddings to a recurrence master, which sends the upstream gradients back
(rotating buffers + events on a communication stream; reference: ``src/main.cpp:3119-3123, 3204-3273,
3368-3414``).  Here the same idea is a micro-batched 1F1B pipeline:

* stage 0 ranks split every micro-batch's frames among themselves (contiguous slices), run the frame head and
  send their slice of the ``(frames, n_embed)`` embeddings to their partner rank of stage 1;
* stage 1 ranks all-gather the slices inside their tensor-parallel group, run the action model — LSTM
  replicated, attention/MLP blocks tensor-parallel over token rows, LM head + loss on the local rows —
  back-propagate, and return the matching slice of the embedding gradient;
* stage 0 back-propagates a micro-batch as soon as its gradient arrives, always keeping the next forward in
  flight first (1F1B), with sends and receives on their own stream so they overlap the convolutions.

Point-to-point traffic is NCCL (``isend`` / ``irecv``; gloo on CPU ranks).  Gradients of parameters that are
replicated inside a stage are all-reduced over that stage's group at the end of the step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from ..utils.logging import LOG
from ..utils.nvtx import gputx_range
from ..models import FbamModel
from .tensor_parallel import TensorParallelBlock, TpContext


RESERVED_SMS = 16   # SMs left to the library's send/receive kernels while a pipeline is active


@dataclass
class PipelineLayout:
    frame_ranks: List[int]
    action_ranks: List[int]

    @staticmethod
    def even_split(world: int) -> "PipelineLayout":
        if world % 2:
            raise ValueError("the two-stage pipeline needs an even number of ranks")
        half = world // 2
        return PipelineLayout(list(range(half)), list(range(half, world)))


class TensorParallelActionModel(nn.Module):
    """The action model of one pipeline stage: replicated LSTM, tensor-parallel blocks, row-sharded head/loss."""

    def __init__(self, model: FbamModel, tp: TpContext, batch: int, seq: int):
        super().__init__()
        am = model.action_model
        self.tp, self.batch, self.seq = tp, batch, seq
        self.lstm = am.lstm
        self.blocks = nn.ModuleList([TensorParallelBlock(b, tp, batch, seq) for b in am.block])
        self.ln_f = am.ln_f
        self.head_weight = am.head_weight
        self.vocab = am.vocab

    def replicated_before_shard(self):
        return list(self.lstm.parameters())

    def replicated_in_shard(self):
        ps = [p for b in self.blocks for p in b.replicated_parameters()]
        if self.ln_f is not None:
            ps += list(self.ln_f.parameters())
        ps.append(self.head_weight)
        return ps

    def forward(self, emb: torch.Tensor, targets: torch.Tensor, loss_scale: float) -> torch.Tensor:
        """``emb`` ``(B, T, E)`` full micro-batch; returns this rank's share of the scaled loss."""
        tp = self.tp
        y, _ = self.lstm(emb.transpose(0, 1).contiguous())
        x = y.transpose(0, 1).reshape(self.batch * self.seq, -1)
        rows = x.shape[0] // tp.world
        xs = x[tp.rank * rows:(tp.rank + 1) * rows]
        for blk in self.blocks:
            xs = blk(xs)
        if self.ln_f is not None:
            xs = self.ln_f(xs)
        tg = targets.reshape(-1)[tp.rank * rows:(tp.rank + 1) * rows]
        return ops.lm_head_ce(xs.contiguous(), self.head_weight, tg, self.vocab, loss_scale)


class TwoStagePipeline:
    def __init__(self, model: FbamModel, layout: PipelineLayout, device: torch.device, micro_batches: int,
                 micro_batch_size: int, seq: int, tp_transport: str = "nccl",
                 all_layouts: Optional[Sequence[PipelineLayout]] = None):
        """``all_layouts``: the layouts of every pipeline replica of the job (data parallelism over whole
        pipelines); process groups are created collectively, so every rank walks through all of them."""
        self.model, self.layout, self.device = model, layout, device
        all_layouts = list(all_layouts) if all_layouts is not None else [layout]
        self.rank = dist.get_rank()
        self.micro_batches, self.mb_size, self.seq = micro_batches, micro_batch_size, seq
        if len(layout.frame_ranks) != len(layout.action_ranks):
            raise ValueError("both stages need the same number of ranks (one partner each)")
        self.is_frame = self.rank in layout.frame_ranks
        self.stage_ranks = layout.frame_ranks if self.is_frame else layout.action_ranks
        self.index = self.stage_ranks.index(self.rank)
        self.partner = (layout.action_ranks if self.is_frame else layout.frame_ranks)[self.index]
        # every rank creates every group (collective), keeps its own
        self.stage_group = None
        for lay in all_layouts:
            g_frame = dist.new_group(lay.frame_ranks)
            g_action = dist.new_group(lay.action_ranks)
            if self.rank in lay.frame_ranks:
                self.stage_group = g_frame
            elif self.rank in lay.action_ranks:
                self.stage_group = g_action
        # One group per partner pair and direction.  NCCL runs the point-to-point operations of a group in issue
        # order on one stream; with both directions in one group, stage 0's "receive gradient k" (issued before
        # "send embeddings k+1") and stage 1's "receive embeddings k+1" (issued before "send gradient k") would
        # wait for each other forever.
        self.fwd_group = self.bwd_group = None
        for lay in all_layouts:
            for f_rank, a_rank in zip(lay.frame_ranks, lay.action_ranks):
                g_fwd, g_bwd = dist.new_group([f_rank, a_rank]), dist.new_group([f_rank, a_rank])
                if self.rank in (f_rank, a_rank):
                    self.fwd_group, self.bwd_group = g_fwd, g_bwd
        if device.type == "cuda":
            # NCCL creates the communicator of a group at the group's first operation, and that creation is a blocking
            # host-side rendezvous of both partners.  Inside the schedule the two sides reach their first operation
            # on the gradient group at different points (stage 0 posts its first gradient receive right after its
            # first forward; stage 1 touches that group only after it has received a whole group of micro-batches),
            # so stage 0 would sit in the rendezvous without ever sending the embeddings stage 1 waits for.  Create
            # both communicators here, in the same order on both sides, with a one-element exchange.
            token = torch.zeros(1, dtype=torch.float32, device=device)
            if self.is_frame:
                dist.send(token, self.partner, group=self.fwd_group)
                dist.recv(token, self.partner, group=self.bwd_group)
            else:
                dist.recv(token, self.partner, group=self.fwd_group)
                dist.send(token, self.partner, group=self.bwd_group)
            torch.cuda.synchronize(device)
        self.n_stage = len(self.stage_ranks)
        frames = micro_batch_size * seq
        if frames % self.n_stage:
            raise ValueError("frames per micro-batch must divide by the ranks of a stage")
        self.slice_rows = frames // self.n_stage
        self.comm_stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        if device.type == "cuda":
            # A posted receive is a resident kernel that spins until its partner sends.  The persistent GEMM /
            # convolution kernels are sized to the machine and could not finish next to it (their last CTAs would
            # wait for the SMs the receive holds, while the partner waits for this rank's results): keep a few
            # SMs out of their grids.  Launch with NCCL_MAX_P2P_NCHANNELS <= 4 so that the two point-to-point
            # kernels that can be resident at once (one per direction) stay within the reserve.
            from ..ops import native as nv
            if nv.available():
                nv.lib().fbam_set_reserved_sms(RESERVED_SMS)
        if not self.is_frame:
            self.tp = TpContext(self.stage_group, device, tp_transport)
            self.action = TensorParallelActionModel(model, self.tp, micro_batch_size, seq).to(device)
        self.stats = {"p2p_bytes": 0}

    # ------------------------------------------------------------------------------------------
    def parameters_of_stage(self):
        if self.is_frame:
            return list(self.model.frame_head.parameters())
        return list(self.action.parameters())

    def _isend(self, t: torch.Tensor):
        """Stage 0 sends embeddings forward, stage 1 sends gradients backward."""
        self.stats["p2p_bytes"] += t.numel() * t.element_size()
        return dist.isend(t, self.partner, group=self.fwd_group if self.is_frame else self.bwd_group)

    def _irecv(self, t: torch.Tensor):
        return dist.irecv(t, self.partner, group=self.bwd_group if self.is_frame else self.fwd_group)

    def run_step(self, cells: Optional[torch.Tensor], targets: Optional[torch.Tensor], loss_scale: float) -> float:
        """One step over ``micro_batches`` micro-batches.  Stage-0 ranks pass ``cells``
        ``(micro_batches, mb_size, T, P, 3)``; stage-1 ranks pass ``targets`` ``(micro_batches, mb_size, T)``.
        Returns this rank's share of the loss (0 on stage 0)."""
        return self._run_frame(cells) if self.is_frame else self._run_action(targets, loss_scale)

    def _run_frame(self, cells: torch.Tensor) -> float:
        fh = self.model.frame_head
        e = self.model.cfg.n_embed
        dtype = next(p for p in fh.parameters() if p.dim() == 2 and p.dtype != torch.float32).dtype \
            if any(p.dtype != torch.float32 for p in fh.parameters()) else torch.float32
        outs, grads, recvs, sends = {}, {}, {}, []
        lo = self.index * self.slice_rows

        def forward(k):
            flat = cells[k].reshape(self.mb_size * self.seq, cells.shape[-2], 3)[lo:lo + self.slice_rows]
            with gputx_range("fbamtrain::frame_head_fwd"):
                emb = fh(flat.to(self.device))
            outs[k] = emb
            payload = emb.detach().contiguous()
            with gputx_range("fbamtrain::ccl_send"):
                sends.append((self._isend(payload), payload))
            grads[k] = torch.empty(self.slice_rows, e, dtype=emb.dtype, device=self.device)
            with gputx_range("fbamtrain::ccl_recv_upstream"):
                recvs[k] = self._irecv(grads[k])

        def backward(k):
            recvs[k].wait()
            with gputx_range("fbamtrain::frame_head_bwd"):
                outs.pop(k).backward(grads.pop(k))

        # 1F1B with a lead of one micro-batch.  (A longer lead — the action stage taking several micro-batches at a
        # time, which would divide the share of its batch-size-independent recurrent kernels — passed on gloo ranks
        # but stopped making progress on NCCL ranks on two GPUs; the cause was not found by reading, so the
        # schedule keeps the lead at which every posted receive depends only on data that has already been sent.)
        forward(0)
        for k in range(1, self.micro_batches):       # next forward first, then the oldest backward
            forward(k)
            backward(k - 1)
        backward(self.micro_batches - 1)
        for work, _ in sends:
            work.wait()
        with gputx_range("fbamtrain::frame_head_grad_allreduce"):
            for p in fh.parameters():            # frame ranks are data parallel over frame slices
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=self.stage_group)
        return 0.0

    def _run_action(self, targets: torch.Tensor, loss_scale: float) -> float:
        """Receives each micro-batch's embeddings, runs the action model on it and returns its slice of the embedding
        gradient to the partner rank."""
        e = self.model.cfg.n_embed
        am = self.action
        dtype = am.head_weight.dtype
        total = torch.zeros((), dtype=torch.float32, device=self.device)   # summed on the device: no host sync
        sends = []
        buf = torch.empty(self.slice_rows, e, dtype=dtype, device=self.device)
        for k in range(self.micro_batches):
            # The receive is posted only when its data is needed: a posted receive is a resident kernel that spins
            # until the data arrives, and the recurrent kernels of this stage are cooperative launches that need
            # most of the machine at once.  The partner sent these embeddings long ago (or is about to).
            self._irecv(buf).wait()
            full = self.tp.all_gather_rows(buf).view(self.mb_size, self.seq, e).detach().requires_grad_(True)
            LOG("DEBUG", f"pipeline: action rank {self.rank} micro-batch {k}: embeddings received")
            tg = targets[k].to(self.device)
            with gputx_range("fbamtrain::action_model_fwd_bwd"):
                loss = am(full, tg, loss_scale)
                loss.backward()
            total += loss.detach().float()
            d_all = full.grad.reshape(self.mb_size * self.seq, e)
            self.tp.all_reduce(d_all)             # every TP rank saw only its rows' contribution
            payload = d_all[self.index * self.slice_rows:(self.index + 1) * self.slice_rows].contiguous()
            with gputx_range("fbamtrain::ccl_send_upstream"):
                sends.append((self._isend(payload), payload))
            LOG("DEBUG", f"pipeline: action rank {self.rank} micro-batch {k}: gradient sent")
        for work, _ in sends:
            work.wait()
        with gputx_range("fbamtrain::action_model_grad_allreduce"):
            for p in am.replicated_before_shard() + am.replicated_in_shard():
                if p.grad is not None:
                    self.tp.all_reduce(p.grad)
        return float(total)


class PipelineTrainer:
    """Training loop body for the two-stage pipeline: one model replica per rank (each rank only touches its
    stage's parameters), one optimizer per rank over its stage's parameters, ``total_batch_size / micro_batch_size``
    micro-batches per step.  Every rank draws the same seeded batch; frame ranks use its cells, action ranks its
    targets.  This is the mode the reference's ``frame_head_parallel`` configuration maps to (reference:
    ``src/main.cpp:3119-3123, 3204-3273, 3368-3414, 3588-3598``)."""

    def __init__(self, cfg, device: torch.device, vocab: int, layout: Optional[PipelineLayout] = None,
                 tp_transport: str = "nccl", replicas: int = 1, ft=None):
        """``replicas`` > 1 runs that many pipelines side by side (data parallelism over pipelines: the reference's
        combination of ``ddp_parallel`` with ``frame_head_parallel``, ``src/main.cpp:2563-2588``): consecutive
        blocks of ``world / replicas`` ranks form one pipeline each, every replica takes its share of the batch
        and the gradients of ranks in the same position are summed across replicas.

        ``ft`` (a :class:`~.ft_pipeline.FaultTolerantPipelineReplicas`): this process group is ONE pipeline of a job
        whose pipelines come and go; the batch is divided by ``ft.expected_replicas``, the pipeline takes the share
        of its current index, gradients are summed over the pipelines that are present, and a step is applied only
        when every position's exchange succeeded."""
        from ..optim import create_optimizer
        self.cfg, self.device = cfg, device
        self.ft = ft
        world, rank = dist.get_world_size(), dist.get_rank()
        if ft is not None and replicas != 1:
            raise ValueError("with dynamic membership every pipeline is a process group of its own (replicas = 1)")
        if replicas < 1 or world % replicas or (world // replicas) % 2:
            raise ValueError("the world must split into `replicas` pipelines with an even number of ranks each")
        shares = replicas if ft is None else ft.expected_replicas
        if cfg.total_batch_size % (cfg.micro_batch_size * shares):
            raise ValueError("total_batch_size must be a multiple of micro_batch_size x replicas")
        self.replicas, self.per_replica = replicas, world // replicas
        self.replica = rank // self.per_replica
        self.micro_batches = cfg.total_batch_size // (cfg.micro_batch_size * shares)
        self.seq = cfg.train_sequence_length
        torch.manual_seed(cfg.model_config.model_init_seed)
        self.model = FbamModel(cfg.model_config, vocab).to(device)
        if replicas == 1:
            layouts = [layout or PipelineLayout.even_split(world)]
        else:
            half = self.per_replica // 2
            layouts = [PipelineLayout(list(range(r * self.per_replica, r * self.per_replica + half)),
                                      list(range(r * self.per_replica + half, (r + 1) * self.per_replica)))
                       for r in range(replicas)]
        self.pipe = TwoStagePipeline(self.model, layouts[self.replica], device, self.micro_batches,
                                     cfg.micro_batch_size, self.seq, tp_transport, all_layouts=layouts,
                                     )
        self.cross_group = None            # ranks in this rank's position of every replica
        if replicas > 1:
            for pos in range(self.per_replica):
                g = dist.new_group([r * self.per_replica + pos for r in range(replicas)])
                if rank % self.per_replica == pos:
                    self.cross_group = g
        if self.pipe.is_frame:
            named = [("frame_head." + n, p) for n, p in self.model.frame_head.named_parameters()]
            prefix = "optim/frame_head"
        else:
            named = [("action_model." + n, p) for n, p in self.pipe.action.named_parameters()]
            prefix = "optim/action_model"
        self.named = named
        self.optimizer = create_optimizer(cfg.optimizer_config, named, prefix)
        self.loss_scale = 1.0 / (self.seq * cfg.total_batch_size)
        self.step_count = 0
        # (valid, RNG state of the dataset iterator at the start of the current step): part of the state a pipeline
        # receives when it is admitted to a running job, so that it continues the job's data order
        self.data_state = torch.zeros(2, dtype=torch.int64, device=device) if ft is not None else None
        if ft is not None:
            ft.attach(self)

    # -- checkpoints ---------------------------------------------------------------------------------------
    # One model file in the single-process layout (every mode can load it) written by global rank 0, plus one
    # optimizer-state file per position of a pipeline (the optimizers hold stage-local, TP-sharded tensors).
    def _optimizer_path(self, model_path: str) -> str:
        pos = dist.get_rank() % self.per_replica
        return model_path.replace(".safetensors", f".optim.pos{pos}.safetensors")

    @torch.no_grad()
    def gather_model(self) -> None:
        """Makes ``self.model`` hold the complete, current model on every rank.  Collective over all ranks."""
        layout = self.pipe.layout
        if not self.pipe.is_frame:
            for blk, full in zip(self.pipe.action.blocks, self.model.action_model.block):
                blk.gather_into(full)
        first_frame, first_action = layout.frame_ranks[0], layout.action_ranks[0]
        if self.replicas > 1:            # replicas hold identical parameters: everyone takes replica 0's
            first_frame, first_action = first_frame % self.per_replica, first_action % self.per_replica
        for p in self.model.frame_head.parameters():
            dist.broadcast(p.data, src=first_frame)
        for p in self.model.action_model.parameters():
            dist.broadcast(p.data, src=first_action)

    @torch.no_grad()
    def validation_loss(self, cells: torch.Tensor, targets: torch.Tensor) -> float:
        """Mean cross-entropy of the current model on ``cells`` / ``targets`` (one micro-batch).  Collective: the
        model is gathered, the first action-model rank evaluates it in one piece and shares the result."""
        self.gather_model()
        first_action = self.pipe.layout.action_ranks[0] % self.per_replica if self.replicas > 1 \
            else self.pipe.layout.action_ranks[0]
        out = torch.zeros(1, dtype=torch.float64, device=self.device)
        if dist.get_rank() == first_action:
            scale = 1.0 / (cells.shape[0] * cells.shape[1])
            out[0] = float(self.model(cells.to(self.device), targets.to(self.device), scale))
        dist.broadcast(out, src=first_action)
        return float(out.item())

    def save_checkpoint(self, manager, dataset_state=None) -> str:
        """Collective.  Returns the model file's path."""
        from ..utils import safetensors_io as st
        self.gather_model()
        path = manager.path_for(self.step_count)
        # with dynamic membership every pipeline holds the same state: the one with index 0 writes the files
        writer = self.ft is None or self.ft.replica_index == 0
        if dist.get_rank() == 0 and writer:
            manager.save(self.step_count, self.model, {}, dataset_state)
        if self.replica == 0 and writer:
            import os
            os.makedirs(manager.directory, exist_ok=True)
            st.save_file({k: v.detach().cpu() for k, v in self.optimizer.state_tensors().items()},
                         self._optimizer_path(path))
        dist.barrier()
        return path

    def load_checkpoint(self, manager, path: str):
        """Every rank reads the model file and takes its stage's (shards of the) parameters; optimizer state comes
        from this position's file when there is one (otherwise moments start from zero and the fp32 masters from
        the loaded parameters).  Returns the dataset state stored with the model."""
        import os
        from ..utils import safetensors_io as st
        step, dataset_state = manager.load(path, self.model, {})
        if not self.pipe.is_frame:
            for blk, full in zip(self.pipe.action.blocks, self.model.action_model.block):
                blk.load_from(full)
        opt_path = self._optimizer_path(path)
        if os.path.exists(opt_path):
            tensors = {k: v.to(self.device) for k, v in st.load_file(opt_path).items()}
            self.optimizer.load_state_tensors(tensors)
        else:
            for name, p in self.named:
                master = self.optimizer.state.get(name, {}).get("master")
                if master is not None:
                    master.copy_(p.data.float())
        self.optimizer.set_step(step)
        self.step_count = step
        return dataset_state

    def train_step(self, cells: torch.Tensor, targets: torch.Tensor) -> float:
        """``cells`` ``(total_batch, T, P, 3)`` and ``targets`` ``(total_batch, T)`` (the same on every rank).
        Returns the step loss (identical on every rank)."""
        for _, p in self.named:
            p.grad = None
        mb = self.cfg.micro_batch_size
        per = self.micro_batches * mb                      # sequences of this replica
        share_index = self.replica if self.ft is None else self.ft.replica_index
        cells, targets = cells[share_index * per:(share_index + 1) * per], \
            targets[share_index * per:(share_index + 1) * per]
        c5 = cells.view(self.micro_batches, mb, *cells.shape[1:]) if self.pipe.is_frame else None
        t3 = targets.view(self.micro_batches, mb, targets.shape[1]) if not self.pipe.is_frame else None
        share = self.pipe.run_step(c5, t3, self.loss_scale)
        if self.cross_group is not None:                   # data parallelism over pipelines: sum (loss is pre-scaled)
            for _, p in self.named:
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=self.cross_group)
        total = torch.tensor([share], dtype=torch.float64, device=self.device)
        dist.all_reduce(total)
        if self.ft is not None:
            # the loss of the whole job rides along with the leader's gradients (zero from the other positions)
            extra = total.float() if self.ft.is_leader else torch.zeros(1, device=self.device)
            if not self.ft.reduce(self, extra=extra):
                return float("nan")                        # dropped: no update, the step is not counted
            total = self._job_loss(extra)
        self.optimizer.step()
        self.step_count += 1
        return float(total.item())

    def _job_loss(self, leader_sum: torch.Tensor) -> torch.Tensor:
        """The leader holds the loss summed over the pipelines; everyone in the pipeline gets it."""
        t = leader_sum.double()
        dist.broadcast(t, src=0)
        return t
