import json
import os
import subprocess
import sys

import torch

from fbamtrain_b200 import presets
from fbamtrain_b200.utils import safetensors_io as st

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, **kw):
    env = dict(os.environ, PYTHONPATH=ROOT, FBAMTRAIN_LOG_LEVEL="INFO")
    return subprocess.run([sys.executable, "-m"] + args, capture_output=True, text=True, env=env, timeout=300, **kw)


def test_cli_trains_synthetic_and_dumps(tmp_path):
    cfg = presets.tiny()
    cfg["checkpointing"]["checkpoint_directory"] = "ckpt"
    cfg["checkpointing"]["checkpoint_interval"] = 2
    cfg["checkpointing"]["resume_behavior"] = "load_latest"
    p = tmp_path / "run.json"
    p.write_text(json.dumps(cfg))
    r = _run(["fbamtrain_b200.cli", "-c", str(p), "--synthetic", "--steps", "3", "--device", "cpu", "-v"])
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Step 2 took" in r.stdout and os.path.exists(tmp_path / "ckpt" / "checkpoint_step_02.safetensors")
    dump = tmp_path / "d.safetensors"
    r = _run(["fbamtrain_b200.cli", "-c", str(p), "--device", "cpu", "--validation-dump", "--validation-dump-file",
              str(dump)])
    assert r.returncode == 0, r.stdout + r.stderr
    keys = set(st.load_file(str(dump)))
    assert {"output", "h_n", "c_n", "loss", "frame_embeddings", "logits"} <= keys


def test_tenscmp_cli(tmp_path):
    a, b = str(tmp_path / "a.safetensors"), str(tmp_path / "b.safetensors")
    t = torch.randn(4, 4)
    st.save_file({"x": t}, a)
    st.save_file({"x": t + 0.01}, b)
    assert _run(["fbamtrain_b200.tenscmp", a, b, "-t", "0.1"]).returncode == 0
    r = _run(["fbamtrain_b200.tenscmp", a, b, "-t", "0.001"])
    assert r.returncode == 1 and "x: max |a-b|" in r.stdout


def test_wandb_wrapper_collects_metric_lines():
    from fbamtrain_b200.wandb_log_wrapper import parse_metric_line
    assert parse_metric_line('{"step": 3, "loss/train": 1.5}') == {"step": 3, "loss/train": 1.5}
    assert parse_metric_line("Step 3 took 1 s") is None and parse_metric_line('{"no_step": 1}') is None
    code = "import json;print('hello');print(json.dumps({'step': 1, 'loss/train': 2.0}))"
    r = _run(["fbamtrain_b200.wandb_log_wrapper", "--dry-run", "--", sys.executable, "-c", code])
    assert r.returncode == 0 and "hello" in r.stdout
    assert json.loads(r.stdout.strip().splitlines()[-1])["metrics_logged"] == 1


def test_cli_frame_head_parallel_runs_the_two_stage_pipeline(tmp_path):
    """Two processes launched the way the reference's launcher script does it (``--worker_id`` / ``--world-size``
    / ``--master`` plus a parallel configuration): rank 0 runs the frame head, rank 1 the action model."""
    import socket
    cfg = presets.tiny()
    cfg["model_config"].update({"action_heads": 2, "lstm_layers": 1})
    cfg["micro_batch_size"], cfg["total_batch_size"] = 2, 4
    cfg["enable_validation"], cfg["validation_interval"] = True, 2
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    par = {"frame_head_parallel": {"use_frame_head_parallel": True, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": port}},
           "ddp_parallel": {"use_ddp_parallel": False}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    env = dict(os.environ, PYTHONPATH=ROOT, FBAMTRAIN_LOG_LEVEL="INFO")
    base = [sys.executable, "-m", "fbamtrain_b200.cli", "-c", str(run), "--parallel-config", str(parallel),
            "--synthetic", "--steps", "2", "--device", "cpu", "--world-size", "2"]
    procs = [subprocess.Popen(base + ["--worker_id", "0"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                              env=env),
             subprocess.Popen(base + ["--worker_id", "1", "--master"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True, env=env)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "Step 1 took" in outs[1] and "loss/train" in outs[1]
    assert "Step 2 validation loss" in outs[1]


def test_launcher_starts_data_parallel_ranks(tmp_path):
    """``fbamtrain_b200.launch`` with a ccl data-parallel configuration: two CPU ranks rendezvous and train."""
    import socket
    cfg = presets.tiny()
    cfg["micro_batch_size"], cfg["total_batch_size"] = 1, 2
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ep = {"ip": "127.0.0.1", "port": port}
    par = {"frame_head_parallel": {"use_frame_head_parallel": False, "transport": "ccl", "ccl_rendezvous": ep},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ccl", "ccl_rendezvous": ep}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    r = _run(["fbamtrain_b200.launch", "--nproc", "2", "--", "-c", str(run), "--parallel-config", str(parallel),
              "--synthetic", "--steps", "2", "--device", "cpu", "-v"])
    assert r.returncode == 0, r.stdout + r.stderr
    assert "[rank 0]" in r.stdout and "[rank 1]" in r.stdout and "Step 1 took" in r.stdout


def test_validate_numerics_flow_on_cpu(tmp_path):
    """Both arms are the PyTorch definitions on a CPU, so the dumps must be identical: checks the plumbing of the
    end-to-end comparison (step, dump, native tenscmp)."""
    from fbamtrain_b200 import validate_numerics
    bad = validate_numerics.run(steps=2, threshold=0.3, preset="tiny", device=torch.device("cpu"),
                                out_dir=str(tmp_path))
    assert bad == 0
    assert any(name.endswith(".safetensors") for name in os.listdir(tmp_path))


def test_cli_pipeline_reads_recordings(tmp_path):
    """The two-stage pipeline launched on a recordings folder: every rank draws the same seeded batches; the
    frame-head rank uses the frames, the action-model rank the tokenised keystrokes."""
    import socket
    import numpy as np
    from fbamtrain_b200.data import ArrayRecording, SyntheticRecording
    from fbamtrain_b200.tokenizer import Tokenizer
    rec_dir = tmp_path / "rec"
    rec_dir.mkdir()
    for i in range(2):
        r = SyntheticRecording(8, 16, 50, seed=i)
        cells = np.stack([r.frame(t)[0] for t in range(50)])
        ArrayRecording(cells, [r.frame(t)[1] for t in range(50)]).save(str(rec_dir / f"r{i}.fbrec.npz"))
    Tokenizer(list("abcdefghijklmnopqrstuvwxyz") + ["ab", "th"]).save(str(tmp_path / "tok.txt"))
    cfg = presets.tiny()
    cfg["model_config"].update({"action_heads": 2, "lstm_layers": 1, "action_vocab": 0})
    cfg["micro_batch_size"], cfg["total_batch_size"] = 2, 4
    cfg["tokenizer_file_path"] = "tok.txt"
    cfg["train_data_config"]["recordings_directory_path"] = "rec"
    cfg["checkpointing"] = {"checkpoint_interval": 2, "checkpoint_directory": "ck", "resume_behavior": "load_latest"}
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    par = {"frame_head_parallel": {"use_frame_head_parallel": True, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": port}},
           "ddp_parallel": {"use_ddp_parallel": False}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    env = dict(os.environ, PYTHONPATH=ROOT, FBAMTRAIN_LOG_LEVEL="INFO")
    base = [sys.executable, "-m", "fbamtrain_b200.cli", "-c", str(run), "--parallel-config", str(parallel),
            "--steps", "2", "--device", "cpu", "--world-size", "2"]
    procs = [subprocess.Popen(base + ["--worker_id", "0"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                              env=env),
             subprocess.Popen(base + ["--worker_id", "1", "--master"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True, env=env)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "Step 1 took" in outs[1] and "loss/train" in outs[1]
    # a second launch resumes from the checkpoint written after step 2 (model gathered from the stages, optimizer
    # state per position, dataset iterator state) and continues with step 2
    base[base.index("--steps") + 1] = "1"
    procs = [subprocess.Popen(base + ["--worker_id", "0"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                              env=env),
             subprocess.Popen(base + ["--worker_id", "1", "--master"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True, env=env)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "Resumed from" in outs[1] and "Step 2 took" in outs[1] and "Step 0 took" not in outs[1], outs[1]


def test_launcher_with_fault_tolerant_transport(tmp_path):
    """``transport: "ftccl"`` through the launcher: it starts the membership master and two CPU ranks; the rank that
    forms the group first must take the other in at the step gate, after which both train in lockstep (same
    committed losses, no dropped step)."""
    import socket
    cfg = presets.tiny()
    cfg["micro_batch_size"], cfg["total_batch_size"] = 1, 2
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    ports = []
    for _ in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    par = {"frame_head_parallel": {"use_frame_head_parallel": False, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": ports[0]}},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ftccl",
                            "ftccl_master": {"ip": "127.0.0.1", "port": ports[1]}}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    r = _run(["fbamtrain_b200.launch", "--nproc", "2", "--", "-c", str(run), "--parallel-config", str(parallel),
              "--synthetic", "--steps", "3", "--device", "cpu", "-v"])
    assert r.returncode == 0, r.stdout + r.stderr
    assert "dropping step" not in r.stdout and "failed" not in r.stdout, r.stdout
    for rank in (0, 1):
        assert f"[rank {rank}]" in r.stdout
    assert r.stdout.count("Step 2 took") == 2


def test_launcher_stops_the_other_ranks_when_one_fails(tmp_path):
    """Rank 1 gets a bad argument and exits at once; rank 0 would wait at the rendezvous for it: the launcher ends
    it after the grace period and reports the failure."""
    import socket
    import time
    cfg = presets.tiny()
    cfg["micro_batch_size"], cfg["total_batch_size"] = 1, 2
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ep = {"ip": "127.0.0.1", "port": port}
    par = {"frame_head_parallel": {"use_frame_head_parallel": False, "transport": "ccl", "ccl_rendezvous": ep},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ccl", "ccl_rendezvous": ep}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    from fbamtrain_b200 import launch
    real_popen = launch.subprocess.Popen
    count = {"n": 0}

    def popen(cmd, **kw):                       # second rank: an interpreter that fails immediately
        count["n"] += 1
        if count["n"] == 2:
            cmd = [sys.executable, "-c", "import sys; print('boom'); sys.exit(3)"]
        return real_popen(cmd, **kw)
    launch.subprocess.Popen = popen
    t0 = time.time()
    try:
        code = launch.main(["--nproc", "2", "--grace", "1", "--", "-c", str(run), "--parallel-config", str(parallel),
                            "--synthetic", "--steps", "2", "--device", "cpu"])
    finally:
        launch.subprocess.Popen = real_popen
    assert code == 3
    assert time.time() - t0 < 60


def test_fault_tolerant_cli_ranks_outlive_an_early_leaver(tmp_path):
    """Master plus three fault-tolerant CLI ranks; one trains two steps and leaves in an orderly way, the others
    re-form the group at their next gate and finish their six steps without dropping one."""
    import socket
    import time
    cfg = presets.tiny()
    cfg["micro_batch_size"], cfg["total_batch_size"] = 1, 3
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    ports = []
    for _ in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    par = {"frame_head_parallel": {"use_frame_head_parallel": False, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": ports[0]}},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ftccl",
                            "ftccl_master": {"ip": "127.0.0.1", "port": ports[1]}}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    env = dict(os.environ, PYTHONPATH=ROOT, FBAMTRAIN_LOG_LEVEL="INFO")
    master = subprocess.Popen([sys.executable, "-m", "fbamtrain_b200.cli", "--parallel-config", str(parallel),
                               "--ftccl-master"], env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    try:
        time.sleep(1.0)
        base = [sys.executable, "-m", "fbamtrain_b200.cli", "-c", str(run), "--parallel-config", str(parallel),
                "--synthetic", "--device", "cpu", "--ddp-world-size", "3"]
        procs = [subprocess.Popen(base + ["--worker_id", str(r), "--steps", "2" if r == 2 else "6"], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(3)]
        outs = [p.communicate(timeout=280)[0] for p in procs]
    finally:
        master.terminate()
        master.wait(10)
    assert all(p.returncode == 0 for p in procs), outs
    assert "finished 2 steps" in outs[2]
    for r in (0, 1):
        assert "finished 6 steps" in outs[r] and "dropping step" not in outs[r], outs[r]


def test_fault_tolerant_cli_admits_a_late_joiner(tmp_path):
    """Two fault-tolerant CLI ranks are training when a third process starts: it builds its model, announces
    itself, receives the shared state (adopting the group's step) and trains the remaining steps with them."""
    import socket
    import time
    cfg = presets.tiny()
    cfg["micro_batch_size"], cfg["total_batch_size"] = 1, 3
    cfg["max_training_steps"] = 20
    # on recordings: the newcomer must also continue the group's data order (one seeded iterator for the group)
    import numpy as np
    from fbamtrain_b200.data import ArrayRecording, SyntheticRecording
    from fbamtrain_b200.tokenizer import Tokenizer
    (tmp_path / "rec").mkdir()
    for i in range(3):
        r = SyntheticRecording(8, 16, 60, seed=i)
        cells = np.stack([r.frame(t)[0] for t in range(60)])
        ArrayRecording(cells, [r.frame(t)[1] for t in range(60)]).save(str(tmp_path / "rec" / f"r{i}.fbrec.npz"))
    Tokenizer(list("abcdefghijklmnopqrstuvwxyz") + ["ab", "th"]).save(str(tmp_path / "tok.txt"))
    cfg["tokenizer_file_path"] = "tok.txt"
    cfg["train_data_config"]["recordings_directory_path"] = "rec"
    cfg["model_config"]["action_vocab"] = 0
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    ports = []
    for _ in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    par = {"frame_head_parallel": {"use_frame_head_parallel": False, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": ports[0]}},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ftccl",
                            "ftccl_master": {"ip": "127.0.0.1", "port": ports[1]}}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    env = dict(os.environ, PYTHONPATH=ROOT, FBAMTRAIN_LOG_LEVEL="INFO")
    master = subprocess.Popen([sys.executable, "-m", "fbamtrain_b200.cli", "--parallel-config", str(parallel),
                               "--ftccl-master"], env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    try:
        time.sleep(1.0)
        base = [sys.executable, "-m", "fbamtrain_b200.cli", "-c", str(run), "--parallel-config", str(parallel),
                "--device", "cpu", "--ddp-world-size", "3"]
        procs = [subprocess.Popen(base + ["--worker_id", str(r)], env=env, stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True) for r in range(2)]
        # the third process starts once the group is demonstrably training (not after a fixed delay)
        head = []
        for line in procs[0].stdout:
            head.append(line)
            if "Step 1 took" in line:
                break
        procs.append(subprocess.Popen(base + ["--worker_id", "2"], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
        outs = [p.communicate(timeout=280)[0] for p in procs]
        outs[0] = "".join(head) + outs[0]
    finally:
        master.terminate()
        master.wait(10)
    assert all(p.returncode == 0 for p in procs), outs
    assert "adopting shared-state revision" in outs[2] and "Step 19 took" in outs[2], outs[2]
    assert "Step 0 took" not in outs[2]                       # it did not start from scratch
    for r in (0, 1):
        assert "Step 19 took" in outs[r] and "dropping step" not in outs[r], outs[r]
    assert "adopted the group's dataset iterator state" in outs[2]
    ends = [[ln.split(": ")[-1] for ln in o.splitlines() if "dataset iterator state at the end" in ln] for o in outs]
    assert all(len(e) == 1 for e in ends) and ends[0] == ends[1] == ends[2], ends


def test_fault_tolerant_cli_survives_a_killed_rank(tmp_path):
    """Host-side failure: one of three fault-tolerant CLI ranks is killed without a goodbye after its third step;
    the other two notice at their next gate, re-form the group and finish all steps."""
    import socket
    import time
    cfg = presets.tiny()
    cfg["micro_batch_size"], cfg["total_batch_size"] = 1, 3
    cfg["max_training_steps"] = 10
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    ports = []
    for _ in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    par = {"frame_head_parallel": {"use_frame_head_parallel": False, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": ports[0]}},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ftccl",
                            "ftccl_master": {"ip": "127.0.0.1", "port": ports[1]}}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    env = dict(os.environ, PYTHONPATH=ROOT, FBAMTRAIN_LOG_LEVEL="INFO")
    master = subprocess.Popen([sys.executable, "-m", "fbamtrain_b200.cli", "--parallel-config", str(parallel),
                               "--ftccl-master"], env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    procs = []
    try:
        time.sleep(1.0)
        base = [sys.executable, "-m", "fbamtrain_b200.cli", "-c", str(run), "--parallel-config", str(parallel),
                "--synthetic", "--device", "cpu", "--ddp-world-size", "3"]
        procs = [subprocess.Popen(base + ["--worker_id", str(r)], env=env, stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True) for r in range(3)]
        for line in procs[2].stdout:
            if "Step 2 took" in line:
                break
        procs[2].kill()                                    # this test's own child, by handle
        procs[2].wait(30)
        outs = [p.communicate(timeout=280)[0] for p in procs[:2]]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        master.terminate()
        master.wait(10)
    assert all(p.returncode == 0 for p in procs[:2]), outs
    for out in outs:
        assert "finished 10 steps" in out, out


def test_cli_pipelines_with_dynamic_membership(tmp_path):
    """``frame_head_parallel`` together with ``ddp_parallel`` on transport ``ftccl``: the membership master and two
    pipelines of two CPU processes each, every pipeline started by hand as a job of its own (``--replica-id``).  The
    pipeline that forms the group first takes the other in at its step gate; afterwards both report the same
    committed losses."""
    import socket
    cfg = presets.tiny()
    cfg["model_config"].update({"action_heads": 2, "lstm_layers": 1})
    cfg["micro_batch_size"], cfg["total_batch_size"] = 1, 2
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    ports = []
    for _ in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    # the two pipelines rendezvous at ports[0] and ports[0] + 1; keep the second one free as well
    par = {"frame_head_parallel": {"use_frame_head_parallel": True, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": ports[0]}},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ftccl",
                            "ftccl_master": {"ip": "127.0.0.1", "port": ports[1]}}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    env = dict(os.environ, PYTHONPATH=ROOT, FBAMTRAIN_LOG_LEVEL="INFO", FBAMTRAIN_METRICS_JSON="1")
    master = subprocess.Popen([sys.executable, "-m", "fbamtrain_b200.cli", "--parallel-config", str(parallel),
                               "--ftccl-master"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    try:
        base = [sys.executable, "-m", "fbamtrain_b200.cli", "-c", str(run), "--parallel-config", str(parallel),
                "--synthetic", "--steps", "6", "--device", "cpu", "--world-size", "2", "--ddp-world-size", "2"]
        procs = []
        for replica in (0, 1):
            for worker, extra in ((0, []), (1, ["--master"])):
                procs.append(subprocess.Popen(base + ["--replica-id", str(replica), "--worker_id", str(worker)] + extra,
                                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env))
        outs = [p.communicate(timeout=400)[0] for p in procs]
        assert all(p.returncode == 0 for p in procs), outs
    finally:
        master.terminate()
        master.communicate(timeout=30)

    def losses(out):
        rows = [json.loads(line) for line in out.splitlines() if line.startswith("{") and "loss/train" in line]
        return {r["step"]: r["loss/train"] for r in rows}
    first, second = losses(outs[1]), losses(outs[3])         # the recurrence masters report
    both = sorted(set(first) & set(second))
    assert len(both) >= 3
    assert all(abs(first[k] - second[k]) < 1e-6 for k in both[-3:])      # in lockstep once both are in the group


def test_launcher_starts_pipelines_with_dynamic_membership(tmp_path):
    """``launch --pipelines 2`` with ``frame_head_parallel`` + transport ``ftccl``: the launcher starts the membership
    master and two pipelines of two CPU ranks, each pipeline as a job of its own (ranks numbered inside the pipeline,
    ``--replica-id`` per pipeline)."""
    import socket
    cfg = presets.tiny()
    cfg["model_config"].update({"action_heads": 2, "lstm_layers": 1})
    cfg["micro_batch_size"], cfg["total_batch_size"] = 1, 2
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    ports = []
    for _ in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    par = {"frame_head_parallel": {"use_frame_head_parallel": True, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": ports[0]}},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ftccl",
                            "ftccl_master": {"ip": "127.0.0.1", "port": ports[1]}}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    r = _run(["fbamtrain_b200.launch", "--nproc", "4", "--pipelines", "2", "--", "-c", str(run), "--parallel-config",
              str(parallel), "--synthetic", "--steps", "4", "--device", "cpu", "-v"])
    assert r.returncode == 0, r.stdout + r.stderr
    for pipeline in (0, 1):
        assert f"[pipeline {pipeline} rank 1]" in r.stdout
    assert r.stdout.count("Step 3 took") == 2          # the recurrence master of each pipeline reports


def test_pipelines_with_dynamic_membership_share_the_data_order_on_recordings(tmp_path):
    """Two pipelines under the membership master on a recordings folder, the second started after the first has
    trained for a while: it adopts the job's step AND the dataset iterator's state, so both end on the same iterator
    state (same data order from the step of admission on)."""
    import socket
    import time
    import numpy as np
    from fbamtrain_b200.data import ArrayRecording, SyntheticRecording
    from fbamtrain_b200.tokenizer import Tokenizer
    rec_dir = tmp_path / "rec"
    rec_dir.mkdir()
    for i in range(2):
        r = SyntheticRecording(8, 16, 50, seed=i)
        cells = np.stack([r.frame(t)[0] for t in range(50)])
        ArrayRecording(cells, [r.frame(t)[1] for t in range(50)]).save(str(rec_dir / f"r{i}.fbrec.npz"))
    Tokenizer(list("abcdefghijklmnopqrstuvwxyz") + ["ab", "th"]).save(str(tmp_path / "tok.txt"))
    cfg = presets.tiny()
    cfg["model_config"].update({"action_heads": 2, "lstm_layers": 1, "action_vocab": 0})
    cfg["micro_batch_size"], cfg["total_batch_size"] = 1, 2
    cfg["tokenizer_file_path"] = "tok.txt"
    cfg["train_data_config"]["recordings_directory_path"] = "rec"
    cfg["max_training_steps"] = 240
    run = tmp_path / "run.json"
    run.write_text(json.dumps(cfg))
    ports = []
    for _ in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    par = {"frame_head_parallel": {"use_frame_head_parallel": True, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": ports[0]}},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ftccl",
                            "ftccl_master": {"ip": "127.0.0.1", "port": ports[1]}}}
    parallel = tmp_path / "parallel.json"
    parallel.write_text(json.dumps(par))
    env = dict(os.environ, PYTHONPATH=ROOT, FBAMTRAIN_LOG_LEVEL="INFO", OMP_NUM_THREADS="1")   # five processes share the cores
    master = subprocess.Popen([sys.executable, "-m", "fbamtrain_b200.cli", "--parallel-config", str(parallel),
                               "--ftccl-master"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    procs = []
    try:
        base = [sys.executable, "-m", "fbamtrain_b200.cli", "-c", str(run), "--parallel-config", str(parallel),
                "--device", "cpu", "--world-size", "2", "--ddp-world-size", "2"]

        logs = []

        def start(replica):
            for worker, extra in ((0, []), (1, ["--master"])):
                log = tmp_path / f"out_{replica}_{worker}.log"
                logs.append(log)
                procs.append(subprocess.Popen(base + ["--replica-id", str(replica), "--worker_id", str(worker)] + extra,
                                              stdout=open(log, "w"), stderr=subprocess.STDOUT, env=env))
        start(0)
        deadline = time.time() + 120
        while "Step 2 took" not in logs[1].read_text() and time.time() < deadline:
            time.sleep(0.2)                    # the first pipeline is training: now start the second
        start(1)
        for p in procs:
            p.wait(timeout=500)
        outs = [log.read_text() for log in logs]
        assert all(p.returncode == 0 for p in procs), [o[-2000:] for o in outs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        master.terminate()
        master.communicate(timeout=30)
    assert "adopted the job's dataset iterator state" in outs[2] + outs[3]
    assert "Step 0 took" not in outs[3]                                  # the late pipeline joined mid-run
    ends = [line.split("end: ")[1] for o in outs for line in o.splitlines() if "iterator state at the end" in line]
    assert len(ends) == 4 and len(set(ends)) == 1                         # one data order for the whole job
