"""Two-stage pipeline (2 frame-head ranks → 2 action-model ranks with 2-way tensor parallelism) on CPU ranks,
against the same model trained in one process."""
import os

import pytest
import socket

import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _setup():
    from fbamtrain_b200 import RunConfiguration, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.models import FbamModel
    d = presets.tiny()
    d["model_config"].update({"action_heads": 2, "lstm_layers": 1})
    cfg = RunConfiguration.from_json(d)
    model = FbamModel(cfg.model_config, 32)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=9, pin=False)
    micro_batches, mb, seq = 3, 2, 16
    cells, targets = src.next_batch(micro_batches * mb, seq)
    return cfg, model, cells.view(micro_batches, mb, seq, -1, 3), targets.view(micro_batches, mb, seq), (micro_batches, mb, seq)


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fbamtrain_b200.parallel.pipeline import PipelineLayout, TwoStagePipeline
    cfg, model, cells, targets, (nmb, mb, seq) = _setup()
    pipe = TwoStagePipeline(model, PipelineLayout.even_split(world), torch.device("cpu"), nmb, mb, seq)
    scale = 1.0 / (seq * nmb * mb)
    loss = pipe.run_step(cells, targets, scale)
    out = {"loss": loss, "frame": pipe.is_frame, "index": pipe.index}
    if pipe.is_frame:
        out["grads"] = {n: p.grad.clone() for n, p in model.frame_head.named_parameters()}
    else:
        out["grads"] = {"lstm." + n: p.grad.clone() for n, p in pipe.action.lstm.named_parameters()}
        out["grads"]["head"] = pipe.action.head_weight.grad.clone()
        out["grads"]["blk0.w_fc1"] = pipe.action.blocks[0].w_fc1.grad.clone()
        out["grads"]["blk0.ln1"] = pipe.action.blocks[0].ln1_weight.grad.clone()
    q.put((rank, out))
    dist.destroy_process_group()


def test_pipeline_matches_single_process():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=180) for _ in range(4))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    cfg, model, cells, targets, (nmb, mb, seq) = _setup()
    scale = 1.0 / (seq * nmb * mb)
    total = 0.0
    for k in range(nmb):
        loss = model(cells[k], targets[k], scale)
        loss.backward()
        total += float(loss)
    assert abs(results[2]["loss"] + results[3]["loss"] - total) < 1e-5
    ref_fh = {n: p.grad for n, p in model.frame_head.named_parameters()}
    for r in (0, 1):
        for n, g in results[r]["grads"].items():
            assert torch.allclose(g, ref_fh[n], atol=2e-6), (r, n)
    am = model.action_model
    for r in (2, 3):
        g = results[r]["grads"]
        for n, p in am.lstm.named_parameters():
            assert torch.allclose(g["lstm." + n], p.grad, atol=2e-6), (r, n)
        assert torch.allclose(g["head"], am.head_weight.grad, atol=2e-6)
        assert torch.allclose(g["blk0.ln1"], am.block[0].ln1.weight.grad, atol=2e-6)
        fl = am.block[0].mlp.fc1.weight.shape[0] // 2
        i = results[r]["index"]
        assert torch.allclose(g["blk0.w_fc1"], am.block[0].mlp.fc1.weight.grad[i * fl:(i + 1) * fl], atol=2e-6)


def _trainer_worker(rank, world, port, q, replicas=1, micro=2):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fbamtrain_b200 import RunConfiguration, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.parallel.pipeline import PipelineTrainer
    d = presets.tiny()
    d["model_config"].update({"action_heads": 2, "lstm_layers": 1})
    d["micro_batch_size"], d["total_batch_size"] = micro, 4
    d["optimizer"]["learning_rate"] = 3e-3
    cfg = RunConfiguration.from_json(d)
    tr = PipelineTrainer(cfg, torch.device("cpu"), vocab=32, replicas=replicas)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=5, pin=False)
    cells, targets = src.next_batch(4, cfg.train_sequence_length)
    losses = [tr.train_step(cells, targets) for _ in range(6)]
    q.put((rank, losses))
    dist.destroy_process_group()


def test_pipeline_trainer_reduces_the_loss():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_trainer_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=240) for _ in range(4))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for r in range(1, 4):
        assert results[r] == results[0]                 # every rank reports the same global loss
    assert results[0][-1] < results[0][0] - 0.05        # and training on one batch brings it down


def test_data_parallel_over_pipelines_matches_one_pipeline():
    """Two one-plus-one pipelines side by side (4 ranks) against a single one-plus-one pipeline (2 ranks) on the
    same total batch: identical loss curves."""
    ctx = mp.get_context("spawn")
    curves = {}
    for world, replicas in ((2, 1), (4, 2)):
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_trainer_worker, args=(r, world, port, q, replicas)) for r in range(world)]
        for p in procs:
            p.start()
        results = dict(q.get(timeout=240) for _ in range(world))
        for p in procs:
            p.join(60)
            assert p.exitcode == 0
        curves[replicas] = results[0]
    assert curves[1] == pytest.approx(curves[2], abs=2e-5)


def _checkpoint_worker(rank, world, port, q, directory):
    """Trains 3 steps, saves, trains 2 more; then a fresh trainer loads the checkpoint and repeats those 2 steps.
    Also loads the model file into a plain single-process model (the file is in the single-process layout)."""
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fbamtrain_b200 import RunConfiguration, presets
    from fbamtrain_b200.checkpoint import CheckpointManager, load_model_params
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.models import FbamModel
    from fbamtrain_b200.parallel.pipeline import PipelineTrainer
    from fbamtrain_b200.utils import safetensors_io as st
    d = presets.tiny()
    d["model_config"].update({"action_heads": 2, "lstm_layers": 1})
    d["micro_batch_size"], d["total_batch_size"] = 2, 4
    d["optimizer"]["learning_rate"] = 3e-3
    cfg = RunConfiguration.from_json(d)
    manager = CheckpointManager(directory, cfg.max_training_steps)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=5, pin=False)
    batches = [src.next_batch(4, cfg.train_sequence_length) for _ in range(5)]
    tr = PipelineTrainer(cfg, torch.device("cpu"), vocab=32)
    for k in range(3):
        tr.train_step(*batches[k])
    path = tr.save_checkpoint(manager)
    first = [tr.train_step(*batches[k]) for k in (3, 4)]
    tr2 = PipelineTrainer(cfg, torch.device("cpu"), vocab=32)
    tr2.load_checkpoint(manager, path)
    assert tr2.step_count == 3
    again = [tr2.train_step(*batches[k]) for k in (3, 4)]
    plain = FbamModel(cfg.model_config, 32)
    load_model_params(plain, st.load_file(path))            # strict names, dtypes and shapes
    if rank == 0:
        # the single-process trainer resumes from the pipeline's model file (optimizer moments restart)
        import copy
        from fbamtrain_b200 import Trainer
        d2 = copy.deepcopy(d)
        d2["checkpointing"] = {"checkpoint_interval": 100, "checkpoint_directory": directory,
                               "resume_behavior": "load_latest"}
        d2["model_config"]["action_vocab"] = 32
        single = Trainer(RunConfiguration.from_json(d2), device=torch.device("cpu"), working_dir="/")
        single.load_latest_checkpoint()
        assert single.step_count == 3
        got = dict(single.model.named_parameters())
        for n, p in plain.named_parameters():
            assert torch.equal(got[n].detach(), p.detach()), n
        single.train_step(*batches[3])
        single.close()
    q.put((rank, first, again, sorted(os.listdir(directory))))
    dist.destroy_process_group()


def test_pipeline_checkpoint_resume_repeats_the_same_steps(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    directory = str(tmp_path / "ck")
    procs = [ctx.Process(target=_checkpoint_worker, args=(r, 4, port, q, directory)) for r in range(4)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(4)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for _, first, again, files in results:
        assert again == pytest.approx(first, rel=1e-6, abs=1e-7)
    files = results[0][3]
    assert any(f.endswith(".safetensors") and ".optim." not in f for f in files)
    assert sum(".optim.pos" in f for f in files) == 4           # one optimizer file per position of the pipeline
