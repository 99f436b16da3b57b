"""Command-line trainer: ``python -m fbamtrain_b200.cli -c run.json [--parallel-config p.json ...]``.

Flags follow the reference binary (reference: ``src/main.cpp:970-1003``): ``-c/--config``,
``--parallel-config``, ``--master``, ``--worker_id``, ``--world-size``, ``--ddp-world-size``,
``--validation-dump``, ``--validation-dump-file``, ``--validation-dump-steps``, ``-v``.  Additions:
``--synthetic`` (seeded synthetic frames instead of recordings), ``--steps`` (stop early),
``--ftccl-master`` (run the membership master of the fault-tolerant transport and nothing else),
``--device``.

Role resolution: with a parallel configuration whose ``ddp_parallel.use_ddp_parallel`` is true, ``--worker_id``
is the data-parallel rank and ``--ddp-world-size`` the world size; transport ``ccl`` rendezvouses at
``ccl_rendezvous`` and reduces gradients as ``grad_reduce`` says (all-reduce, ZeRO-1 or the fused peer-memory
kernels); transport ``ftccl`` joins the membership master at ``ftccl_master``.  ``frame_head_parallel`` maps to
the two-stage pipeline over ``--world-size`` ranks; together with transport ``ftccl`` every pipeline is a job of its
own that joins the membership master (``--replica-id`` tells pipelines started by hand apart).  Under ``torch.distributed.run`` the RANK / WORLD_SIZE
environment takes the place of the flags.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch

from .config import ParallelConfiguration, RunConfiguration
from .utils.logging import LOG


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="fbamtrain", description="Train a frame-based action model.")
    ap.add_argument("-c", "--config", required=False, help="run configuration JSON")
    ap.add_argument("--parallel-config", default=None)
    ap.add_argument("--master", action="store_true", help="this process is the recurrence master (pipeline stage 1)")
    ap.add_argument("--worker_id", "--worker-id", type=int, default=None)
    ap.add_argument("--world-size", type=int, default=1)
    ap.add_argument("--ddp-world-size", type=int, default=1)
    ap.add_argument("--replica-id", type=int, default=None,
                    help="frame_head_parallel with transport ftccl, processes started by hand: which pipeline this "
                         "process belongs to (its pipeline rendezvouses at the configured port + this number)")
    ap.add_argument("--validation-dump", action="store_true")
    ap.add_argument("--validation-dump-file", default="validation_dump.safetensors")
    ap.add_argument("--validation-dump-steps", type=int, default=1)
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--device", default=None)
    ap.add_argument("--frame-chunk", type=int, default=1024)
    ap.add_argument("--ftccl-master", action="store_true")
    return ap


def _run_ftccl_master(par: ParallelConfiguration) -> int:
    from .parallel.ftccl import create_master
    ep = par.ddp_parallel.ftccl_master
    if ep is None:
        LOG("FATAL", "--ftccl-master needs ddp_parallel.transport = \"ftccl\" with an ftccl_master endpoint")
    master = create_master(ep.ip, ep.port)
    if master.port == 0:          # the native service binds when started
        master.start()
    LOG("INFO", f"ftccl master listening on {ep.ip}:{master.port}")
    try:
        master.run()
    except KeyboardInterrupt:
        master.interrupt()
    return 0


def _run_pipeline(cfg: RunConfiguration, par: ParallelConfiguration, args, device: torch.device) -> int:
    """``frame_head_parallel``: the first half of ``--world-size`` ranks runs the frame head, the second half the
    action model (tensor-parallel blocks); ``--master`` marks the first action-model rank, as the reference marks
    its recurrence master."""
    import torch.distributed as dist
    from .data import SyntheticBatchSource
    from .parallel import rendezvous
    from .parallel.pipeline import PipelineLayout, PipelineTrainer
    env_rank = os.environ.get("RANK")
    ddp = par.ddp_parallel
    dynamic = ddp.use_ddp_parallel and ddp.transport == "ftccl"
    if dynamic:
        # pipelines come and go: ranks may vanish while their memory is mapped by peers, so nothing in this job binds
        # memory to NVLink multicast objects
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    if env_rank is not None:
        rank, world = int(env_rank), int(os.environ["WORLD_SIZE"])
        kwargs = {"device_id": device} if device.type == "cuda" else {}
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo", **kwargs)
    elif dynamic:
        # every pipeline is a job of its own: --world-size ranks, --worker_id counts inside the pipeline
        rank, world = (args.worker_id or 0), args.world_size
        ep = par.frame_head_parallel.ccl_rendezvous
        rendezvous.perform_ccl_rendezvous(ep.ip, ep.port + (args.replica_id or 0), rank, world, device)
    else:
        # --world-size ranks per pipeline, --ddp-world-size pipelines side by side; --worker_id counts over all
        rank, world = (args.worker_id or 0), args.world_size * max(1, args.ddp_world_size)
        ep = par.frame_head_parallel.ccl_rendezvous
        rendezvous.perform_ccl_rendezvous(ep.ip, ep.port, rank, world, device)
    replicas = 1 if dynamic else max(1, args.ddp_world_size)
    if world % replicas or (world // replicas) % 2:
        LOG("FATAL", f"{world} ranks do not split into {replicas} pipelines of an even number of ranks")
    per = world // replicas
    layout = PipelineLayout(list(range(per // 2)), list(range(per // 2, per)))   # positions inside one pipeline
    if args.master and rank % per != layout.action_ranks[0]:
        LOG("FATAL", f"--master belongs to position {layout.action_ranks[0]} (the first action-model rank) of a pipeline")
    vocab = cfg.model_config.action_vocab
    if vocab <= 0:
        from .tokenizer import Tokenizer
        vocab = len(Tokenizer.from_file(os.path.join(os.path.dirname(os.path.abspath(args.config)),
                                                     cfg.tokenizer_file_path)))
    fused_tp = device.type == "cuda" and per // 2 > 1        # peer-memory kernels need at least two TP ranks
    ft = None
    if dynamic:
        # Data parallelism over pipelines with dynamic membership: this process group is one pipeline; its leader
        # talks to the membership master, same-position ranks of the pipelines that are present exchange gradients.
        # A pipeline started while the job runs receives the state from the others (the highest revision wins).
        from .parallel.ft_pipeline import FaultTolerantPipelineReplicas
        ft = FaultTolerantPipelineReplicas(ddp.ftccl_master.ip, ddp.ftccl_master.port, device,
                                           expected_replicas=max(1, args.ddp_world_size), min_replicas=1)
    trainer = PipelineTrainer(cfg, device, vocab, tp_transport="fused" if fused_tp else "nccl", replicas=replicas,
                              ft=ft)
    working_dir = os.path.dirname(os.path.abspath(args.config))
    rec_dir = cfg.train_data_config.recordings_directory_path
    if rec_dir and not args.synthetic:
        # Every rank draws the same batches (same seed): frame-head ranks use the frames, action-model ranks the
        # targets of the sequences of their pipeline.
        from .data import RecordingDatasetIterator
        from .tokenizer import Tokenizer
        from .train import build_batch_from_recordings
        tokenizer = Tokenizer.from_file(os.path.join(working_dir, cfg.tokenizer_file_path))
        iterator = RecordingDatasetIterator(os.path.join(working_dir, rec_dir), cfg.total_batch_size,
                                            cfg.train_sequence_length, cfg.train_data_config.iteration_seed)

        def next_batch():
            return build_batch_from_recordings(iterator.next_batch(), tokenizer, cfg.train_sequence_length,
                                               cfg.frame_rows, cfg.frame_cols, vocab, cfg.model_config.max_code_point)
    else:
        iterator = None
        src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, vocab,
                                   seed=cfg.train_data_config.iteration_seed, pin=device.type == "cuda")

        prefetch = None

        def next_batch():
            nonlocal prefetch
            if prefetch is None:               # started after a resume has positioned the source
                from .data import PrefetchingSource
                prefetch = PrefetchingSource(src, cfg.total_batch_size, cfg.train_sequence_length)
            return prefetch.next_batch(cfg.total_batch_size, cfg.train_sequence_length)
        next_batch.close = lambda: prefetch.close() if prefetch is not None else None
    from .checkpoint import CheckpointManager
    manager = CheckpointManager(os.path.join(working_dir, cfg.checkpointing.checkpoint_directory),
                                cfg.max_training_steps)
    if cfg.checkpointing.resume_behavior == "load_latest":
        latest = manager.find_latest()
        if latest is not None:
            restored = trainer.load_checkpoint(manager, latest[1])
            LOG("INFO", f"Resumed from {latest[1]} at step {trainer.step_count}")
            if iterator is not None and restored is not None and restored.prepared_indices:
                restored.batch_size = cfg.total_batch_size
                iterator.restore(restored)
            elif iterator is None:
                src.seek(trainer.step_count)
    if ft is not None and iterator is None and trainer.step_count > 0:
        src.seek(trainer.step_count)     # a pipeline admitted to a running job continues at the job's position
    if ft is not None and iterator is not None:
        valid, rng_state = (int(v) for v in trainer.data_state.tolist())
        if valid:                        # ... and on recordings it adopts the job's iterator state
            from .data.iterator import DatasetIteratorState
            iterator.restore(DatasetIteratorState(rng_state=rng_state & ((1 << 64) - 1), batch_size=cfg.total_batch_size))
            LOG("INFO", "adopted the job's dataset iterator state")
    limit = cfg.max_training_steps if args.steps is None else min(cfg.max_training_steps,
                                                                  trainer.step_count + args.steps)
    interval = cfg.checkpointing.checkpoint_interval
    while trainer.step_count < limit:
        step = trainer.step_count
        if ft is not None and iterator is not None:
            rng_now = iterator.cursor_checkpoint().rng_state
            trainer.data_state.copy_(torch.tensor([1, rng_now - (1 << 64) if rng_now >= (1 << 63) else rng_now],
                                                  dtype=torch.int64))
        cells, targets = next_batch()
        t0 = time.perf_counter()
        loss = trainer.train_step(cells.to(device), targets.to(device))
        if rank == layout.action_ranks[0]:                 # the first pipeline's recurrence master reports
            LOG("INFO", f"Step {step} took {time.perf_counter() - t0:.4f} seconds; loss/train = {loss:.6f}")
            if os.environ.get("FBAMTRAIN_METRICS_JSON"):
                import json
                sys.stdout.write(json.dumps({"step": step, "step_time_sec": time.perf_counter() - t0,
                                             "loss/train": loss}) + "\n")
                sys.stdout.flush()
        if cfg.enable_validation and cfg.validation_interval and trainer.step_count % cfg.validation_interval == 0:
            vsrc = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, vocab,
                                        seed=cfg.validation_data_config.iteration_seed, pin=False)
            vloss = trainer.validation_loss(*vsrc.next_batch(cfg.micro_batch_size, cfg.validation_sequence_length))
            if rank == layout.action_ranks[0]:
                LOG("INFO", f"Step {trainer.step_count} validation loss = {vloss:.6f}")
                if os.environ.get("FBAMTRAIN_METRICS_JSON"):
                    import json
                    sys.stdout.write(json.dumps({"step": trainer.step_count, "loss/validation": vloss}) + "\n")
                    sys.stdout.flush()
        if interval > 0 and trainer.step_count % interval == 0:
            trainer.save_checkpoint(manager, iterator.checkpoint() if iterator is not None else None)
    if iterator is not None:
        LOG("INFO", f"dataset iterator state at the end: {iterator.cursor_checkpoint().rng_state}")
        iterator.close()
    if hasattr(next_batch, "close"):
        next_batch.close()
    if ft is not None:
        ft.leave()               # orderly departure: the remaining pipelines re-form their groups at the next gate
    dist.destroy_process_group()
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.verbose:
        os.environ["FBAMTRAIN_LOG_LEVEL"] = "INFO"
    par = None
    if args.parallel_config:
        par = ParallelConfiguration.from_json_file(args.parallel_config)
        if par is None:
            LOG("FATAL", f"parallel configuration {args.parallel_config} not found")
    if args.ftccl_master:
        if par is None:
            LOG("FATAL", "--ftccl-master needs --parallel-config")
        return _run_ftccl_master(par)
    if not args.config:
        LOG("FATAL", "a run configuration is required (-c)")
    cfg = RunConfiguration.from_json_file(args.config)
    if cfg is None:
        LOG("FATAL", f"run configuration {args.config} not found")
    working_dir = os.path.dirname(os.path.abspath(args.config))

    from .train import Trainer, run_training
    env_rank, env_world = os.environ.get("RANK"), os.environ.get("WORLD_SIZE")
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.device:
        device = torch.device(args.device)
        if device.type == "cuda" and device.index is not None:
            torch.cuda.set_device(device)
    elif torch.cuda.is_available():
        device = torch.device("cuda", local_rank if env_rank is not None else (args.worker_id or 0) % max(
            1, torch.cuda.device_count()))
        torch.cuda.set_device(device)
    else:
        device = torch.device("cpu")

    fhp = par.frame_head_parallel if par is not None else None
    if fhp is not None and fhp.use_frame_head_parallel:
        return _run_pipeline(cfg, par, args, device)

    dp = None
    ddp = par.ddp_parallel if par is not None else None
    if ddp is not None and ddp.use_ddp_parallel and ddp.grad_reduce == "fused" and device.type != "cuda":
        # the fused reduction runs in kernels over peer GPU memory; CPU ranks take the sharded library path
        LOG("WARN", "grad_reduce 'fused' needs GPUs; using 'zero1' on this device")
        ddp.grad_reduce = "zero1"
    if env_rank is not None and int(env_world) > 1:
        import torch.distributed as dist
        from .parallel.dp import DataParallel
        kwargs = {"device_id": device} if device.type == "cuda" else {}
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo", **kwargs)
        dp = DataParallel(mode=(ddp.grad_reduce if ddp is not None and ddp.use_ddp_parallel else "allreduce"))
    elif ddp is not None and ddp.use_ddp_parallel:
        rank = args.worker_id if args.worker_id is not None else 0
        if ddp.transport == "ccl":
            from .parallel import rendezvous
            from .parallel.dp import DataParallel
            rendezvous.perform_ccl_rendezvous(ddp.ccl_rendezvous.ip, ddp.ccl_rendezvous.port, rank,
                                              args.ddp_world_size, device)
            dp = DataParallel(mode=ddp.grad_reduce)
        else:
            from .parallel.ft_dp import FaultTolerantDataParallel
            from .parallel.ftccl import FtPeer
            # the peer announces itself to the master when the trainer attaches, i.e. after the model is built, so
            # that a process joining a running group does not hold the members at their gate while it initialises
            peer = FtPeer(ddp.ftccl_master.ip, ddp.ftccl_master.port, device)
            dp = FaultTolerantDataParallel(peer, expected_world=args.ddp_world_size, min_world=1,
                                           mode="fused" if ddp.grad_reduce == "fused" else "allreduce")

    if cfg.model_config.dtype == "fp16" and cfg.model_config.use_fp16_accumulation and device.type == "cuda":
        LOG("INFO", "use_fp16_accumulation: the half-precision kernels of this package accumulate in fp32 "
                    "(tensor-memory accumulators); the flag changes nothing here")
    trainer = Trainer(cfg, parallel=par, device=device, dp=dp, frame_chunk=args.frame_chunk, working_dir=working_dir)
    if args.synthetic:
        cfg.train_data_config.recordings_directory_path = ""

    if args.validation_dump:
        from .data import SyntheticBatchSource
        from .utils import safetensors_io as st
        src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, trainer.vocab,
                                   seed=cfg.validation_data_config.iteration_seed, pin=False)
        for step in range(args.validation_dump_steps):
            cells, targets = src.next_batch(cfg.micro_batch_size, cfg.validation_sequence_length)
            dump = trainer.validation_dump(cells, targets)
            path = args.validation_dump_file if args.validation_dump_steps == 1 else \
                args.validation_dump_file.replace(".safetensors", f"_{step}.safetensors")
            st.save_file(dump, path)
            LOG("INFO", f"wrote {path}")
            trainer.train_step(cells, targets)
        trainer.close()
        return 0

    t0 = time.time()
    history = run_training(trainer, max_steps=args.steps)
    trainer.close()
    if dp is not None and hasattr(dp, "peer"):
        dp.peer.leave()          # orderly departure: the remaining members re-form the group at their next gate
    if history:
        LOG("INFO", f"finished {len(history)} steps in {time.time() - t0:.1f} s; last loss {history[-1]['loss/train']:.4f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
