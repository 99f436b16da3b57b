"""Checkpoint save / find-latest / load.

One safetensors file per checkpoint, named ``checkpoint_step_<step>.safetensors`` with the step
zero-padded to the number of digits of ``max_training_steps``.  Tensors: ``step_count`` (U64[1]),
``dataset_rng_state`` (U64[1]), ``dataset_prefetch_indices`` (U32[B]), ``dataset_prefetch_starts``
(U64[B]), ``dataset_prefetch_buffer_index`` (U32[1]), ``param/<name>`` in the reference's storage
layout, and the optimizer state under ``optim/frame_head/…`` and ``optim/action_model/…``.  The
latest checkpoint is the one with the largest step not above ``max_training_steps``; on load the
step in the file name must equal the stored ``step_count`` (reference:
``src/checkpointing.cpp:14-67, 180-422``; load order ``src/main.cpp:91-160``).
"""
from __future__ import annotations

import os
import threading
import re
from typing import Dict, Optional, Tuple

import torch

from .data.iterator import DatasetIteratorState
from .models.fbam import FbamModel, checkpoint_name_map
from .optim.base import Optimizer
from .utils import safetensors_io as st
from .utils.logging import LOG

_NAME_RE = re.compile(r"^checkpoint_step_(\d+)\.safetensors$")


def _u64(values) -> torch.Tensor:
    return torch.tensor([int(v) & ((1 << 64) - 1) for v in values], dtype=torch.uint64)


def _u32(values) -> torch.Tensor:
    return torch.tensor([int(v) for v in values], dtype=torch.uint32)


def model_param_tensors(model: FbamModel) -> Dict[str, torch.Tensor]:
    """``param/<reference name>`` → tensor in the reference's storage layout."""
    named = dict(model.named_parameters())
    out: Dict[str, torch.Tensor] = {}
    for internal, entries in checkpoint_name_map(model).items():
        for ck_name, to_ckpt, _ in entries:
            out["param/" + ck_name] = to_ckpt(named[internal].detach()).contiguous()
    return out


def load_model_params(model: FbamModel, tensors: Dict[str, torch.Tensor]) -> None:
    named = dict(model.named_parameters())
    for internal, entries in checkpoint_name_map(model).items():
        p = named[internal]
        for row, (ck_name, to_ckpt, from_ckpt) in enumerate(entries):
            key = "param/" + ck_name
            if key not in tensors:
                raise KeyError(f"checkpoint lacks tensor '{key}'")
            src = tensors[key]
            expect = to_ckpt(p.detach())
            if src.dtype != expect.dtype or tuple(src.shape) != tuple(expect.shape):
                raise ValueError(f"checkpoint tensor '{key}' is {src.dtype}{tuple(src.shape)}, "
                                 f"expected {expect.dtype}{tuple(expect.shape)}")
            with torch.no_grad():
                if len(entries) > 1:
                    p.data[row].copy_(src)
                else:
                    p.data.copy_(from_ckpt(src))


class CheckpointManager:
    def __init__(self, directory: str, max_training_steps: int, background: bool = False):
        """``background``: ``save`` snapshots the tensors into host memory on the calling thread (device→host copies
        only) and leaves the file write — the slow part for multi-gigabyte states — to a worker thread; training
        continues meanwhile.  A later ``save``, ``find_latest``, ``load`` or ``wait`` first waits for the pending
        write, and a write error is raised there.  The file appears under its final name only when complete
        (temporary file, fsync, rename), in either mode."""
        self.directory = directory
        self.max_training_steps = int(max_training_steps)
        self.pad = len(str(self.max_training_steps))
        self.background = background
        self._writer: Optional[threading.Thread] = None
        self._write_error: Optional[BaseException] = None

    def wait(self) -> None:
        """Blocks until the pending background write (if any) is on disk; raises what it raised."""
        writer, self._writer = self._writer, None
        if writer is not None:
            writer.join()
        error, self._write_error = self._write_error, None
        if error is not None:
            raise RuntimeError(f"background checkpoint write failed: {error}") from error

    def _write(self, tensors: Dict[str, torch.Tensor], path: str) -> None:
        try:
            st.save_file(tensors, path)
        except BaseException as e:  # noqa: BLE001 - reported by wait()
            self._write_error = e

    def path_for(self, step: int) -> str:
        return os.path.join(self.directory, f"checkpoint_step_{int(step):0{self.pad}d}.safetensors")

    def find_latest(self) -> Optional[Tuple[int, str]]:
        self.wait()
        if not os.path.isdir(self.directory):
            return None
        best: Optional[Tuple[int, str]] = None
        for f in os.listdir(self.directory):
            m = _NAME_RE.match(f)
            if not m:
                continue
            step = int(m.group(1))
            if step <= self.max_training_steps and (best is None or step > best[0]):
                best = (step, os.path.join(self.directory, f))
        return best

    def save(self, step: int, model: FbamModel, optimizers: Dict[str, Optimizer],
             dataset_state: Optional[DatasetIteratorState]) -> str:
        os.makedirs(self.directory, exist_ok=True)
        tensors: Dict[str, torch.Tensor] = {"step_count": _u64([step])}
        ds = dataset_state or DatasetIteratorState()
        tensors["dataset_rng_state"] = _u64([ds.rng_state])
        tensors["dataset_prefetch_indices"] = _u32(ds.prepared_indices)
        tensors["dataset_prefetch_starts"] = _u64(ds.prepared_start_positions)
        tensors["dataset_prefetch_buffer_index"] = _u32([ds.prefetch_buffer_index])
        tensors.update(model_param_tensors(model))
        for opt in optimizers.values():
            for name, t in opt.state_tensors().items():
                if name.endswith("__optimizer/step"):
                    t = _u64([int(t.reshape(-1)[0])])
                tensors[name] = t
        path = self.path_for(step)
        self.wait()
        if not self.background:
            st.save_file({k: v.detach().cpu() for k, v in tensors.items()}, path)
            return path
        # the snapshot must not alias live training state: .cpu() copies device tensors, host tensors are cloned
        snapshot = {k: (v.detach().cpu() if v.device.type != "cpu" else v.detach().clone()) for k, v in tensors.items()}
        self._writer = threading.Thread(target=self._write, args=(snapshot, path), name="fbam-checkpoint-writer")
        self._writer.start()
        return path

    def load(self, path: str, model: FbamModel, optimizers: Dict[str, Optimizer],
             batch_size: Optional[int] = None) -> Tuple[int, DatasetIteratorState]:
        self.wait()
        m = _NAME_RE.match(os.path.basename(path))
        tensors = st.load_file(path)
        if "step_count" not in tensors:
            raise KeyError(f"{path}: tensor 'step_count' missing")
        step = int(tensors["step_count"].view(torch.int64).reshape(-1)[0])
        if m and int(m.group(1)) != step:
            raise ValueError(f"{path}: file name says step {int(m.group(1))} but step_count is {step}")
        load_model_params(model, tensors)
        dev = next(model.parameters()).device
        for opt in optimizers.values():
            as_i64 = {k: (v.view(torch.int64) if v.dtype == torch.uint64 else v).to(dev) for k, v in tensors.items()
                      if k.startswith(opt.prefix + "/")}
            if as_i64:
                opt.load_state_tensors(as_i64)
            else:
                # a model-only file (e.g. written by the pipeline trainer, whose optimizer state lives in files of
                # its own): moments start from zero, the fp32 masters from the parameters just loaded
                LOG("WARN", f"{path} holds no state under '{opt.prefix}/': optimizer moments start from zero")
                opt.reset_masters_from_params()
            opt.set_step(step)
        ds = DatasetIteratorState()
        if "dataset_rng_state" in tensors:
            ds.rng_state = int(tensors["dataset_rng_state"].view(torch.int64).reshape(-1)[0]) & ((1 << 64) - 1)
            ds.prepared_indices = [int(v) for v in tensors["dataset_prefetch_indices"].view(torch.int32).reshape(-1)]
            ds.prepared_start_positions = [int(v) for v in
                                           tensors["dataset_prefetch_starts"].view(torch.int64).reshape(-1)]
            ds.prefetch_buffer_index = int(tensors["dataset_prefetch_buffer_index"].view(torch.int32).reshape(-1)[0])
            ds.batch_size = batch_size if batch_size is not None else len(ds.prepared_indices)
        return step, ds
