"""Training engine: builds the model, optimizers and flat buffers from a run configuration and runs
steps.

Step structure of the reference (reference: ``src/main.cpp:3016-3869``): zero gradients → for every
micro-batch run frame head, action model forward/backward and frame-head backward → accumulate the
loss → reduce gradients across data-parallel ranks (sum; the loss is pre-divided by
``T · total_batch_size``) → step the frame-head and action-model optimizers → commit the dataset
cursor → enqueue step metrics → periodic validation → periodic checkpoint.

``Trainer.train_step(cells, targets)`` is the public per-step call.  It accepts host tensors
(pinned or not): frames are uploaded chunk by chunk on a copy stream while the frame head already
works on earlier chunks, and the step loss leaves the device through the loss ring buffer without
blocking the loop.
"""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .checkpoint import CheckpointManager
from .config import ParallelConfiguration, RunConfiguration
from .data import (Batch, DatasetCursorCommitter, DatasetCursorSnapshot, RecordingDatasetIterator,
                   PrefetchingSource, StreamTokenizationContext, SyntheticBatchSource, consume_next_token, prepare_cell_states)
from .models import FbamModel
from .ops import embconv
from .optim import AdamwOptimizer, MuonWithAuxAdam, Optimizer, create_optimizer
from .tokenizer import Tokenizer
from .utils import flops, plan
from .utils.flat import FlatGroup, build_groups
from .utils.logging import LOG, enabled as log_enabled
from .utils.metrics import AsyncStepLogger, LossRingBuffer, ProgressRecord, StepRecord
from .utils.nvtx import gputx_range


def _is_muon_param(name: str, p: torch.nn.Parameter) -> bool:
    """Matrices go to Muon; embeddings, the LM head, gains, biases and initial states to AdamW."""
    if p.dim() < 2:
        return False
    return not any(k in name for k in ("embed", "head_weight", "position_embedding"))


class Trainer:
    def __init__(self, cfg: RunConfiguration, parallel: Optional[ParallelConfiguration] = None,
                 device: Optional[torch.device] = None, dp=None, tokenizer: Optional[Tokenizer] = None,
                 frame_chunk: int = 0, working_dir: str = "."):
        self.cfg, self.parallel, self.working_dir = cfg, parallel, working_dir
        self.device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.dp = dp
        self.world = dp.world_size if dp is not None else 1
        if cfg.total_batch_size % (cfg.micro_batch_size * self.world) != 0:
            raise ValueError("total_batch_size must be a multiple of micro_batch_size x data-parallel world size")
        self.grad_accum_steps = cfg.total_batch_size // (cfg.micro_batch_size * self.world)

        self.tokenizer = tokenizer
        if tokenizer is None and cfg.tokenizer_file_path:
            self.tokenizer = Tokenizer.from_file(os.path.join(working_dir, cfg.tokenizer_file_path))
        vocab = cfg.model_config.action_vocab or (len(self.tokenizer) if self.tokenizer else 0)
        if vocab <= 0:
            raise ValueError("action vocabulary unknown: give a tokenizer file or 'action_vocab'")
        self.vocab = vocab

        self.model = FbamModel(cfg.model_config, vocab).to(self.device)
        self.model.frame_chunk = frame_chunk
        self.frame_chunk = frame_chunk

        # flat parameter / gradient buffers, grouped by scope, optimizer kind and dtype
        # buckets divide evenly by every world size up to the nominal one, so the sharded / fused update keeps
        # working after ranks have left (fault-tolerant data parallelism)
        import math
        shard_multiple = math.lcm(*range(1, self.world + 1)) if self.world > 1 else 1
        self.groups: Dict[str, List[FlatGroup]] = {}
        self.optimizers: Dict[str, Optimizer] = {}
        for scope, module in (("frame_head", self.model.frame_head), ("action_model", self.model.action_model)):
            named = [(f"{scope}.{n}", p) for n, p in module.named_parameters()]
            ocfg = cfg.optimizer_config
            prefix = f"optim/{scope}"
            if ocfg.type == "adamw":
                gs = build_groups(scope, named, shard_multiple)
                self.groups[scope] = gs
                self.optimizers[scope] = AdamwOptimizer(named, prefix, ocfg.learning_rate, ocfg.beta1, ocfg.beta2,
                                                        ocfg.eps, ocfg.weight_decay, groups=gs)
            elif ocfg.type == "muon":
                muon_named = [(n, p) for n, p in named if _is_muon_param(n, p)]
                adam_named = [(n, p) for n, p in named if not _is_muon_param(n, p)]
                g_muon = build_groups(scope + "/muon", muon_named, shard_multiple) if muon_named else []
                g_adam = build_groups(scope + "/adam", adam_named, shard_multiple) if adam_named else []
                self.groups[scope] = g_muon + g_adam
                opt = MuonWithAuxAdam(named, prefix, ocfg.learning_rate, ocfg.momentum, ocfg.nesterov,
                                      ocfg.weight_decay, ocfg.beta1, ocfg.beta2, ocfg.eps,
                                      adam_names=lambda n, _m=dict(named): not _is_muon_param(n, _m[n]))
                if g_adam:
                    opt.adam = AdamwOptimizer(adam_named, prefix + "/adam", ocfg.learning_rate, ocfg.beta1,
                                              ocfg.beta2, ocfg.eps, ocfg.weight_decay, groups=g_adam)
                self.optimizers[scope] = opt
            else:
                self.groups[scope] = build_groups(scope, named, shard_multiple)
                self.optimizers[scope] = create_optimizer(ocfg, named, prefix)
        self.step_count = 0
        self.last_upload_event = None
        # [valid, iterator RNG state] of the dataset iterator at the start of the current step: part of the shared
        # state of a fault-tolerant group, so that a process admitted mid-run continues the group's data order
        self.data_state = torch.zeros(2, dtype=torch.int64, device=self.device)
        if self.dp is not None:
            self.dp.attach(self)

        self.ring = LossRingBuffer(self.device)
        self.logger = AsyncStepLogger(self.ring)
        self.ckpt = CheckpointManager(os.path.join(working_dir, cfg.checkpointing.checkpoint_directory),
                                      cfg.max_training_steps, background=cfg.checkpointing.background_write)
        self.cursor: Optional[DatasetCursorCommitter] = None
        self._cuda = self.device.type == "cuda"
        if self._cuda:
            from .utils.streams import stream_bundle
            self.streams = stream_bundle(self.device)
            self.h2d_stream = self.streams.h2d
        self._staging: Dict[Tuple, torch.Tensor] = {}
        self._loss_events: List[Tuple[int, object]] = [(-1, None)] * 64
        self._warned_recompute = False
        self._upload_slot, self._slot_in_use, self._fresh_buffer = 0, 0, False
        self._slot_free: List[Optional[torch.cuda.Event]] = [None, None]

    @property
    def rank(self) -> int:
        """This process's current data-parallel rank (ranks are assigned, and can change, when the membership of a
        fault-tolerant group changes)."""
        return self.dp.rank if self.dp is not None else 0

    # ------------------------------------------------------------------------------------------
    def all_groups(self) -> List[FlatGroup]:
        return [g for gs in self.groups.values() for g in gs]

    def zero_grad(self) -> None:
        with gputx_range("fbamtrain::zero_grad"):
            for g in self.all_groups():
                g.grad.zero_()

    def _device_buffer(self, key, shape, dtype) -> torch.Tensor:
        buf = self._staging.get(key)
        if buf is None or tuple(buf.shape) != tuple(shape) or buf.dtype != dtype:
            buf = torch.empty(shape, dtype=dtype, device=self.device)
            self._staging[key] = buf
            self._fresh_buffer = True
        return buf

    def _upload(self, cells: torch.Tensor, targets: torch.Tensor):
        """Starts the host→device copies; returns device tensors and per-chunk ready events."""
        if cells.device == self.device or not self._cuda:
            return cells.to(self.device), targets.to(self.device), None, None
        b, t, p, _ = cells.shape
        frames = b * t
        chunk = self.frame_chunk or frames
        # Two device buffers in turn: the copies for this micro-batch only wait until the micro-batch before the
        # previous one has finished its backward (the last reader of the buffer), so a caller that queues step
        # k + 1 while step k computes gets its upload overlapped with that compute.
        slot = self._upload_slot
        self._upload_slot = 1 - slot
        self._fresh_buffer = False
        dev_cells = self._device_buffer(("cells", slot), (frames, p, 3), cells.dtype)
        dev_targets = self._device_buffer(("targets", slot), tuple(targets.shape), targets.dtype)
        flat = cells.reshape(frames, p, 3)
        events = []
        if self._fresh_buffer or self._slot_free[slot] is None:
            # new memory from the caching allocator: order the copies behind everything queued on the compute stream
            self.h2d_stream.wait_stream(torch.cuda.current_stream())
        else:
            self.h2d_stream.wait_event(self._slot_free[slot])
        self._slot_in_use = slot
        with torch.cuda.stream(self.h2d_stream):
            dev_targets.copy_(targets, non_blocking=True)
            for lo in range(0, frames, chunk):
                hi = min(frames, lo + chunk)
                dev_cells[lo:hi].copy_(flat[lo:hi], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                events.append(ev)
        self.last_upload_event = events[-1] if events else None   # all of this step's host→device copies are done
        return dev_cells.view(b, t, p, 3), dev_targets, events, chunk

    def _mark(self):
        """A point in time on the compute stream: a timing event on a GPU, wall-clock seconds on the CPU."""
        if not self._cuda:
            return time.perf_counter()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def _forward_backward(self, cells: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        loss_scale = 1.0 / (cells.shape[1] * cfg.total_batch_size)
        if self.model.cfg.frame_replay and not cells.is_cuda:
            return self._forward_backward_replayed(cells, targets, loss_scale)
        dev_cells, dev_targets, events, chunk = self._upload(cells, targets)
        b, t, p, _ = dev_cells.shape
        progress = log_enabled("INFO")          # per-chunk progress lines cost two events per chunk: only when shown
        phase0 = self._mark() if progress else None
        with gputx_range("fbamtrain::forward"):
            if events is None:
                emb = self.model.frame_embeddings(dev_cells)
                if progress:
                    self.logger.progress(ProgressRecord("Frame head: frames", b * t, b * t, phase0, self._mark()))
            else:
                flat = dev_cells.view(b * t, p, 3)
                parts = []
                with gputx_range("fbamtrain::frame_head_fwd"):
                    n_chunks = (b * t + chunk - 1) // chunk
                    recompute = None                  # None: as configured
                    for i, lo in enumerate(range(0, b * t, chunk)):
                        torch.cuda.current_stream().wait_event(events[i])
                        before = torch.cuda.memory_allocated(self.device)
                        parts.append(self.model.frame_head_chunk(flat[lo:lo + chunk], recompute))
                        if recompute is None and not self.model.cfg.frame_head_recompute:
                            # Activations kept for the backward grow by about the same amount per chunk.  When
                            # the rest would not fit, the remaining chunks keep only their inputs and are run
                            # again in the backward (the alternative is running out of memory).
                            grown = torch.cuda.memory_allocated(self.device) - before
                            free, _total = torch.cuda.mem_get_info(self.device)
                            cached = torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
                            if grown * (n_chunks - i - 1) > 0.9 * (free + cached):
                                recompute = True
                                if not self._warned_recompute:
                                    self._warned_recompute = True
                                    LOG("WARN", f"frame head: activations of {n_chunks - i - 1} of {n_chunks} chunks "
                                                "would not fit in device memory; recomputing them in the backward "
                                                "(set model key frame_head_recompute to choose this up front)")
                        if progress:
                            self.logger.progress(ProgressRecord("Frame head: frames", min(b * t, lo + chunk), b * t,
                                                                phase0, self._mark()))
                emb = (parts[0] if len(parts) == 1 else torch.cat(parts, 0)).view(b, t, -1)
            with gputx_range("fbamtrain::action_model_fwd_bwd"):
                loss = self.model.action_model(emb, dev_targets, loss_scale)
        phase1 = self._mark() if progress else None
        with gputx_range("fbamtrain::backward"):
            loss.backward()
        if progress:
            self.logger.progress(ProgressRecord("Backward: frames", b * t, b * t, phase1, self._mark()))
        if events is not None:          # the backward was the last reader of this micro-batch's device buffers
            done = torch.cuda.Event()
            done.record()
            self._slot_free[self._slot_in_use] = done
        return loss.detach()

    def _forward_backward_replayed(self, cells: torch.Tensor, targets: torch.Tensor, loss_scale: float) -> torch.Tensor:
        """Model key ``frame_replay``: the frames stay in host memory, the frame head sees one chunk at a time and
        every chunk is uploaded and run again in the backward (``utils/frame_replay.py``)."""
        from .utils.frame_replay import FrameReplay, ReplayedFrameHead
        b, t, p, _ = cells.shape
        chunk = self.frame_chunk or b * t
        replay = FrameReplay(cells.reshape(b * t, p, 3), chunk, self.device,
                             self.h2d_stream if self._cuda else None)
        self.last_replay = replay
        anchor = next(self.model.frame_head.parameters())
        dev_targets = targets.to(self.device, non_blocking=True)
        with gputx_range("fbamtrain::forward"):
            with gputx_range("fbamtrain::frame_head_fwd"):
                parts = [ReplayedFrameHead.apply(anchor, self.model.frame_head, replay, i)
                         for i in range(replay.num_chunks)]
            emb = (parts[0] if len(parts) == 1 else torch.cat(parts, 0)).view(b, t, -1)
            with gputx_range("fbamtrain::action_model_fwd_bwd"):
                loss = self.model.action_model(emb, dev_targets, loss_scale)
        with gputx_range("fbamtrain::backward"):
            loss.backward()
        return loss.detach()

    def train_step(self, cells: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimizer step (see :meth:`_train_step`).  With ``FBAMTRAIN_DUMP_PLAN=<file>`` the first step is
        recorded as a launch plan (``utils/plan.py``) and its listing written to the file."""
        path = os.environ.get("FBAMTRAIN_DUMP_PLAN", "")
        if not path or self.step_count != 0 or self.rank != 0 or plan.active() is not None:
            return self._train_step(cells, targets)
        with plan.record() as recorded:
            loss = self._train_step(cells, targets)
        with open(path, "w") as f:
            f.write(recorded.listing())
        return loss

    def _train_step(self, cells: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimizer step.  ``cells`` int32 ``(B_local, T, P, 3)`` and ``targets`` int64 ``(B_local, T)``
        hold this rank's share of the batch (``grad_accum_steps`` micro-batches).  Returns the step
        loss as a device scalar (this rank's share of the global mean)."""
        cfg = self.cfg
        micro = cfg.micro_batch_size
        if cells.shape[0] != micro * self.grad_accum_steps:
            raise ValueError(f"expected {micro * self.grad_accum_steps} sequences per rank, got {cells.shape[0]}")
        step = self.step_count
        start_ev = end_ev = None
        wall0 = time.perf_counter()
        flops_total0, flops_useful0 = flops.snapshot()
        if self._cuda:
            start_ev = torch.cuda.Event(enable_timing=True)
            start_ev.record()
        self.zero_grad()
        self.ring.begin(step)
        # parameter-derived tables of the fused first frame-head layer are valid until the optimizer runs
        self._table_epoch = getattr(self, "_table_epoch", 0) + 1
        embconv.set_cache_token((id(self), self._table_epoch))
        total = None
        for k in range(self.grad_accum_steps):
            if self.dp is not None and k == self.grad_accum_steps - 1:
                self.dp.arm()
            loss = self._forward_backward(cells[k * micro:(k + 1) * micro], targets[k * micro:(k + 1) * micro])
            self.ring.accumulate(step, loss)
            total = loss if total is None else total + loss
        committed = True
        if self.dp is not None:
            committed = self.dp.reduce_and_step(self)
            if self._cuda and getattr(self.dp, "mode", "") == "fused" and not hasattr(self.dp, "peer"):
                # plain (not fault-tolerant) fused data parallelism: a bounded device-side wait that ran out means
                # a collective did not complete; fail the run (seen one step late, without a host sync per step)
                from .ops import native as _nv
                _nv.check_status_late(self.device)
        else:
            with gputx_range("fbamtrain::action_model_optim_step"):
                self.optimizers["action_model"].step()
            with gputx_range("fbamtrain::frame_head_optim_step"):
                self.optimizers["frame_head"].step()
        embconv.set_cache_token(None)
        loss_ev = self.ring.finalize(step)
        self._loss_events[step % len(self._loss_events)] = (step, loss_ev)
        if self._cuda:
            end_ev = torch.cuda.Event(enable_timing=True)
            end_ev.record()
        flops_total1, flops_useful1 = flops.snapshot()
        self.logger.submit(StepRecord(step, start_ev, end_ev, loss_ev, cells.shape[1], cfg.total_batch_size,
                                      dropped=not committed, wall_start=wall0, wall_end=time.perf_counter(),
                                      useful_flops=flops_useful1 - flops_useful0,
                                      total_flops=flops_total1 - flops_total0))
        if committed:
            self.step_count += 1
        if self._cuda and self.step_count % 50 == 0:
            from .utils.streams import allocator_metrics
            m = allocator_metrics(self.device)
            LOG("INFO", "allocator: peak {:.2f} GiB, current {:.2f} GiB, cached {:.2f} GiB, reserved {:.2f} GiB".format(
                *(m[k] / 2 ** 30 for k in ("peak_bytes", "current_bytes", "cached_bytes", "reserved_bytes"))))
        return total

    def host_loss(self, step: int) -> float:
        """The loss of step ``step`` (this rank's share) as a host float.  Waits only for that step's own
        device→host copy — 4 bytes on the side stream, queued when the step was — and not for steps launched after
        it, so a loop can launch step k + 1 and then read the loss of step k without draining the device."""
        kept_step, event = self._loss_events[step % len(self._loss_events)]
        if kept_step != step:
            raise ValueError(f"the loss of step {step} is no longer kept (latest {self.step_count - 1})")
        if event is not None:
            event.synchronize()
        return self.ring.read(step)

    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def validation_loss(self, cells: torch.Tensor, targets: torch.Tensor) -> float:
        cells, targets = cells.to(self.device), targets.to(self.device)
        scale = 1.0 / (cells.shape[0] * cells.shape[1])
        embconv.set_cache_token(None)
        return float(self.model(cells, targets, scale))

    def validation_dump(self, cells: torch.Tensor, targets: torch.Tensor) -> Dict[str, torch.Tensor]:
        """Tensors of one forward/backward pass for numerics comparison: ``output`` (LSTM-stack
        hidden states), ``h_n``, ``c_n``, ``loss``, ``frame_embeddings``, ``logits``, ``grad_*`` and
        ``param_*`` (reference: ``src/main.cpp:3492-3564``)."""
        cells, targets = cells.to(self.device), targets.to(self.device)
        self.zero_grad()
        embconv.set_cache_token(None)
        scale = 1.0 / (cells.shape[1] * cells.shape[0])
        emb = self.model.frame_embeddings(cells)
        emb.retain_grad()
        hidden, (h_n, c_n) = self.model.action_model.features(emb)
        logits = self.model.action_model.logits(hidden)
        loss = self.model.action_model(emb, targets, scale)
        loss.backward()
        out = {"output": hidden.detach(), "h_n": h_n.detach(), "c_n": c_n.detach(), "loss": loss.detach().reshape(1),
               "frame_embeddings": emb.detach(), "logits": logits.detach()}
        for n, p in self.model.named_parameters():
            out["param_" + n] = p.detach().clone()
            if p.grad is not None:
                out["grad_" + n] = p.grad.detach().clone()
        return {k: v.float().cpu().contiguous() for k, v in out.items()}

    # ------------------------------------------------------------------------------------------
    def save_checkpoint(self, dataset_state=None) -> str:
        """Collective under data parallelism (every rank calls it: the sharded optimizer state is gathered first);
        rank 0 writes the file.  Returns the file's path on every rank."""
        if self._cuda:
            torch.cuda.synchronize()
        if self.dp is not None:
            self.dp.gather_optimizer_state(self)
        if self.rank != 0:
            return self.ckpt.path_for(self.step_count)
        return self.ckpt.save(self.step_count, self.model, self.optimizers, dataset_state)

    def load_latest_checkpoint(self):
        """Returns the restored dataset-iterator state, or None when nothing was loaded."""
        if self.cfg.checkpointing.resume_behavior != "load_latest":
            return None
        latest = self.ckpt.find_latest()
        if latest is None:
            return None
        step, ds = self.ckpt.load(latest[1], self.model, self.optimizers,
                                  self.cfg.micro_batch_size * self.grad_accum_steps * self.world)
        self.step_count = step
        LOG("INFO", f"Resumed from {latest[1]} at step {step}")
        return ds

    def close(self) -> None:
        self.ckpt.wait()
        self.logger.drain()
        self.logger.close()
        if self.cursor is not None:
            self.cursor.close()


# ----------------------------------------------------------------------------------------------
# batches from recordings
# ----------------------------------------------------------------------------------------------
def build_batch_from_recordings(batch, tokenizer: Tokenizer, seq_len: int, rows: int, cols: int, vocab: int,
                                max_code_point: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Walks each stream's keystrokes with the tokenizer and pairs every token with the frame that
    was on screen when it started; exhausted streams pad with zero frames and target 0
    (reference: ``src/main.cpp:1812-1884``)."""
    b = len(batch.recordings)
    cells = np.zeros((b, seq_len, rows * cols, 3), dtype=np.uint32)
    targets = np.zeros((b, seq_len), dtype=np.int64)
    for i, (rec, start) in enumerate(zip(batch.recordings, batch.start_positions)):
        if rec.rows != rows or rec.cols != cols:
            raise RuntimeError(f"Obtained input frame from dataset with size different from configuration: "
                               f"Expected {rows}x{cols} according to configuration, got {rec.rows}x{rec.cols}")
        ctx = StreamTokenizationContext(rec, tokenizer, int(start))
        for pos in range(seq_len):
            res = None if ctx.exhausted else consume_next_token(ctx)
            if res is None:
                ctx.exhausted = True
                continue
            token_id, frame_idx = res
            frame, _ = rec.frame(frame_idx)
            prepare_cell_states(frame, max_code_point, cells[i, pos])
            targets[i, pos] = token_id % vocab
    return torch.from_numpy(cells.view(np.int32)), torch.from_numpy(targets)


class _PinnedBatchBuffer:
    """One of the two host buffers the native loader fills in turn.  ``release(event)`` is called after the step
    that read it has queued its host→device copies; the next fill waits for that event, because the copies are
    asynchronous and the host can be several steps ahead of the device."""

    def __init__(self, batch: int, seq: int, cells_per_frame: int, pin: bool):
        self.cells = torch.empty((batch, seq, cells_per_frame, 3), dtype=torch.int32, pin_memory=pin)
        self.targets = torch.empty((batch, seq), dtype=torch.int64, pin_memory=pin)
        self._event = None

    def wait_until_free(self) -> None:
        event, self._event = self._event, None
        if event is not None:
            event.synchronize()

    def release(self, event) -> None:
        self._event = event


def _data_rank(trainer: Trainer) -> int:
    """Which share of a global batch draw this process takes: its current data-parallel rank (ranks renumber when
    the membership of a fault-tolerant group changes), within the nominal world the batch is drawn for."""
    rank = trainer.dp.rank if trainer.dp is not None else 0
    return rank % max(1, trainer.world)


def _make_assembler(trainer: Trainer, local_batch: int):
    """The batch assembler for the dataset iterator's prefetch thread, or None when the per-frame Python path has
    to be used: the native loader needs raw ``.fbrec`` recordings, a tokenizer and the runtime library."""
    from . import runtime
    from .data.recording import recording_extensions
    cfg = trainer.cfg
    folder = os.path.join(trainer.working_dir, cfg.train_data_config.recordings_directory_path)
    if trainer.tokenizer is None or not runtime.available() or not os.path.isdir(folder):
        return None
    exts = tuple(recording_extensions())
    paths = sorted(os.path.join(folder, f) for f in os.listdir(folder)
                   if f.endswith(exts) and not os.path.isdir(os.path.join(folder, f)))
    if not paths or not all(p.endswith(".fbrec") for p in paths):
        return None
    loader = runtime.NativeBatchLoader(paths, trainer.tokenizer.tokens, cfg.model_config.max_code_point, trainer.vocab)
    if (loader.rows, loader.cols) != (cfg.frame_rows, cfg.frame_cols):
        raise RuntimeError(f"Obtained input frame from dataset with size different from configuration: Expected "
                           f"{cfg.frame_rows}x{cfg.frame_cols} according to configuration, got "
                           f"{loader.rows}x{loader.cols}")
    seq = cfg.train_sequence_length
    buffers = [_PinnedBatchBuffer(local_batch, seq, cfg.frame_rows * cfg.frame_cols, trainer.device.type == "cuda")
               for _ in range(2)]

    def assemble(indices, starts, buffer_index):
        lo = _data_rank(trainer) * local_batch   # the iterator draws the global batch; this rank assembles its share
        buf = buffers[buffer_index]
        buf.wait_until_free()
        loader.fill(indices[lo:lo + local_batch], starts[lo:lo + local_batch], seq, buf.cells, buf.targets)
        return buf, buf.cells, buf.targets

    assemble.loader = loader          # keeps the mapping alive as long as the assembler
    return assemble


def _validation_source(trainer: Trainer):
    """A callable returning one validation batch per call: sequences drawn from the validation recordings with
    their own seeded iterator when the configuration names a folder (the reference runs a second dataset iterator
    for validation, ``src/main.cpp:2169-2175``), else seeded synthetic frames — the same batch every time, so the
    curve is comparable across steps."""
    cfg = trainer.cfg
    mc = cfg.model_config
    vcfg = cfg.validation_data_config
    folder = os.path.join(trainer.working_dir, vcfg.recordings_directory_path) if vcfg.recordings_directory_path else ""
    if folder and os.path.isdir(folder) and trainer.tokenizer is not None:
        iterator = RecordingDatasetIterator(folder, cfg.micro_batch_size, cfg.validation_sequence_length,
                                            vcfg.iteration_seed)

        def from_recordings():
            return build_batch_from_recordings(iterator.next_batch(), trainer.tokenizer,
                                               cfg.validation_sequence_length, cfg.frame_rows, cfg.frame_cols,
                                               trainer.vocab, mc.max_code_point)
        from_recordings.iterator = iterator
        return from_recordings

    def synthetic():
        src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, mc.max_code_point, trainer.vocab,
                                   seed=vcfg.iteration_seed, pin=False)
        return src.next_batch(cfg.micro_batch_size, cfg.validation_sequence_length)
    return synthetic


def run_training(trainer: Trainer, source=None, max_steps: Optional[int] = None) -> List[dict]:
    """The outer loop: data → ``train_step`` → cursor commit → validation → checkpoint."""
    cfg = trainer.cfg
    local_batch = cfg.micro_batch_size * trainer.grad_accum_steps
    global_batch = local_batch * trainer.world
    iterator = None
    own_source = False
    if source is None:
        if cfg.train_data_config.recordings_directory_path:
            # Every rank runs the same seeded iterator over the GLOBAL batch and takes its own share of each draw:
            # the data order does not depend on the number of ranks, and one iterator state (stored in the
            # checkpoint and the cursor file) resumes all of them.
            iterator = RecordingDatasetIterator(
                os.path.join(trainer.working_dir, cfg.train_data_config.recordings_directory_path), global_batch,
                cfg.train_sequence_length, cfg.train_data_config.iteration_seed,
                assembler=_make_assembler(trainer, local_batch))
        else:
            source = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point,
                                          trainer.vocab, seed=cfg.train_data_config.iteration_seed + trainer.rank)
            own_source = True
    validation = None
    if hasattr(trainer.dp, "peer") and trainer.step_count > 0:
        # admitted to a running fault-tolerant group: its state (received when the trainer attached) is newer than
        # any checkpoint on disk
        restored = None
    else:
        restored = trainer.load_latest_checkpoint()
    if iterator is not None and restored is not None and restored.batch_size:
        iterator.restore(restored)
    if source is not None and trainer.step_count and hasattr(source, "seek"):
        source.seek(trainer.step_count)        # synthetic batches are a function of (seed, call number)
    prefetcher = None
    if own_source:                             # generate batch k + 1 on a host thread while batch k trains
        source = prefetcher = PrefetchingSource(source, local_batch, cfg.train_sequence_length)
    cursor_path = cfg.checkpointing.dataset_cursor_path
    if cursor_path:
        cursor_path = os.path.join(trainer.working_dir, cursor_path)
        snap = DatasetCursorCommitter.load(cursor_path)
        if snap is not None and iterator is not None:
            # A cursor written under another batch or sequence length describes a different data order: refuse it,
            # as the reference does (src/main.cpp:2926-2933).  batch_size is the number of sequences the iterator
            # draws per call — the global batch here (one iterator serves all ranks), the micro-batch there.
            if snap.batch_size != global_batch:
                raise RuntimeError(f"Dataset cursor batch_size does not match run configuration "
                                   f"(cursor {snap.batch_size}, iterator draws {global_batch} sequences per step).")
            if snap.sequence_length != cfg.train_sequence_length:
                raise RuntimeError(f"Dataset cursor sequence_length does not match run configuration "
                                   f"(cursor {snap.sequence_length}, configured {cfg.train_sequence_length}).")
            if snap.step_count != trainer.step_count:
                LOG("WARN", f"dataset cursor is at step {snap.step_count}, checkpoint at {trainer.step_count}")
            from .data.iterator import DatasetIteratorState
            iterator.restore(DatasetIteratorState(rng_state=snap.rng_state, batch_size=global_batch))
        if trainer.rank == 0:                  # the iterator state is the same on every rank: one writer
            trainer.cursor = DatasetCursorCommitter(cursor_path)
    limit = cfg.max_training_steps if max_steps is None else min(cfg.max_training_steps, trainer.step_count + max_steps)
    mc = cfg.model_config
    shares_data_state = iterator is not None and hasattr(trainer.dp, "peer")     # fault-tolerant group on recordings
    if shares_data_state:
        valid, rng_state = (int(v) for v in trainer.data_state.tolist())
        if valid:                              # admitted to a running group: continue ITS data order
            from .data.iterator import DatasetIteratorState
            iterator.restore(DatasetIteratorState(rng_state=rng_state & ((1 << 64) - 1), batch_size=global_batch))
            LOG("INFO", "adopted the group's dataset iterator state")
    while trainer.step_count < limit:
        with gputx_range("fbamtrain::next_batch_wait"):
            assembled = None
            if shares_data_state:
                rng_now = iterator.cursor_checkpoint().rng_state
                trainer.data_state.copy_(torch.tensor([1, rng_now - (1 << 64) if rng_now >= (1 << 63) else rng_now],
                                                      dtype=torch.int64))
            if iterator is not None:
                batch = iterator.next_batch()
                if batch.tensors is not None:          # gathered by the native loader on the prefetch thread
                    assembled, cells, targets = batch.tensors
                else:
                    if trainer.world > 1:              # this rank's share of the global draw
                        lo = _data_rank(trainer) * local_batch
                        batch = Batch(batch.recordings[lo:lo + local_batch], batch.indices[lo:lo + local_batch],
                                      batch.start_positions[lo:lo + local_batch])
                    cells, targets = build_batch_from_recordings(batch, trainer.tokenizer, cfg.train_sequence_length,
                                                                 cfg.frame_rows, cfg.frame_cols, trainer.vocab,
                                                                 mc.max_code_point)
            else:
                cells, targets = source.next_batch(local_batch, cfg.train_sequence_length)
        trainer.train_step(cells, targets)
        if assembled is not None:
            assembled.release(trainer.last_upload_event)
        if trainer.cursor is not None and iterator is not None:
            st = iterator.cursor_checkpoint()
            trainer.cursor.commit(DatasetCursorSnapshot(trainer.step_count, st.rng_state, global_batch,
                                                        cfg.train_sequence_length))
        if cfg.enable_validation and cfg.validation_interval and trainer.step_count % cfg.validation_interval == 0:
            with gputx_range("fbamtrain::validation"):
                if validation is None:
                    validation = _validation_source(trainer)
                vc, vt = validation()
                trainer.logger.log_validation(trainer.step_count, trainer.validation_loss(vc, vt))
        if trainer.step_count % cfg.checkpointing.checkpoint_interval == 0:
            trainer.save_checkpoint(iterator.checkpoint() if iterator is not None else None)
    trainer.logger.drain()
    if iterator is not None:
        LOG("INFO", f"dataset iterator state at the end: {iterator.cursor_checkpoint().rng_state}")
        iterator.close()
    if prefetcher is not None:
        prefetcher.close()
    if validation is not None and getattr(validation, "iterator", None) is not None:
        validation.iterator.close()
    return list(trainer.logger.history)
