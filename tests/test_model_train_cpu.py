import copy
import math
import os

import pytest
import torch

from fbamtrain_b200 import RunConfiguration, Trainer, presets, run_training
from fbamtrain_b200.checkpoint import CheckpointManager, model_param_tensors
from fbamtrain_b200.data import SyntheticBatchSource
from fbamtrain_b200.models import FbamModel, checkpoint_name_map
from fbamtrain_b200.ops import reference as ref
from fbamtrain_b200.optim import AdamwOptimizer, MuonOptimizer, MuonWithAuxAdam, SgdOptimizer, newton_schulz
from fbamtrain_b200.utils import safetensors_io as st
from fbamtrain_b200.utils.flat import build_groups

CPU = torch.device("cpu")


def _tiny(**over):
    d = presets.tiny()
    d.update(over)
    return RunConfiguration.from_json(d)


def _batch(cfg, seed=0, batch=None):
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point,
                               cfg.model_config.action_vocab, seed=seed, pin=False)
    return src.next_batch(batch or cfg.micro_batch_size, cfg.train_sequence_length)


def test_model_shapes_and_causality():
    cfg = _tiny()
    model = FbamModel(cfg.model_config, 32)
    cells, _ = _batch(cfg)
    emb = model.frame_embeddings(cells)
    assert emb.shape == (2, 16, 64)
    hidden, (h, c) = model.action_model.features(emb)
    assert hidden.shape == (2, 16, 64) and h.shape == (2, 2, 64)
    # changing a late frame must not change earlier hidden states (LSTM + causal attention)
    cells2 = cells.clone()
    cells2[:, 10:, :, 0] = (cells2[:, 10:, :, 0] + 1) % 256
    hidden2, _ = model.action_model.features(model.frame_embeddings(cells2))
    assert torch.allclose(hidden[:, :10], hidden2[:, :10], atol=1e-6)
    assert not torch.allclose(hidden[:, 10:], hidden2[:, 10:], atol=1e-6)


def test_reference_structure_model_builds():
    # reference-style head: RMSNorm + stride-1 dilated conv + pool, attention blocks in the frame head, 1-layer LSTM
    d = presets.tiny()
    m = d["model_config"]
    for k in ("cell_embed_dim", "downsample_channels", "downsample_conv_stride", "downsample_norm", "frame_proj",
              "lstm_layers", "lstm_hidden", "action_blocks", "action_heads", "action_mlp_dim"):
        m.pop(k)
    m.update({"n_layer": 1, "downsample_blocks": 2, "downsample_conv_dilation": 2, "n_embed": 32,
              "frame_head_reduction_strategy": "last_pos"})
    cfg = RunConfiguration.from_json(d)
    model = FbamModel(cfg.model_config, 32)
    cells, tg = _batch(cfg)
    loss = model(cells, tg, 1.0 / 32)
    loss.backward()
    names = {e[0][0] for e in checkpoint_name_map(model).values()} | {
        x[0] for e in checkpoint_name_map(model).values() for x in e}
    for expect in ("frame_head.codepoint_embedding", "frame_head.fg_r_embed", "frame_head.bg_b_embed",
                   "frame_head.position_embedding.weight", "frame_head.downsample_block.1.ln.weight",
                   "frame_head.downsample_block.0.conv.weight", "frame_head.block.0.attn.w_qkv",
                   "frame_head.block.0.attn.b_proj", "frame_head.block.0.mlp.fc1.weight",
                   "frame_head.block.0.ln2.weight", "action_model.lstm.weights_ih", "action_model.lstm.h0",
                   "action_model.head.weight"):
        assert expect in names, expect
    pt = model_param_tensors(model)
    assert pt["param/action_model.lstm.weights_ih"].shape == (32, 128)       # stored (in, 4H)
    assert pt["param/action_model.head.weight"].shape == (32, 32)            # stored (H, V_pad)
    assert pt["param/frame_head.block.0.attn.w_qkv"].shape == (32, 96)       # stored (in, out)
    assert pt["param/frame_head.downsample_block.0.conv.weight"].shape == (32, 3, 3, 32)  # OHWI


def test_geglu_mode():
    d = presets.tiny()
    d["model_config"]["downsample_conv_mode"] = "geglu"
    cfg = RunConfiguration.from_json(d)
    model = FbamModel(cfg.model_config, 32)
    assert model.frame_head.downsample_block[0].conv_weight.shape[0] == 128
    cells, tg = _batch(cfg)
    model(cells, tg, 1.0).backward()


def test_loss_decreases_on_fixed_batch():
    cfg = _tiny()
    cfg.optimizer_config.learning_rate = 3e-3
    tr = Trainer(cfg, device=CPU)
    cells, tg = _batch(cfg)
    losses = [float(tr.train_step(cells, tg)) for _ in range(12)]
    tr.close()
    assert losses[-1] < losses[0] - 0.05, losses


def test_grad_accumulation_equals_large_batch():
    big = _tiny(micro_batch_size=4, total_batch_size=4)
    acc = _tiny(micro_batch_size=2, total_batch_size=4)
    for c in (big, acc):      # SGD: the update is proportional to the gradient (Adam's is not near zero)
        c.optimizer_config.type, c.optimizer_config.momentum = "sgd", 0.0
    cells, tg = _batch(big, batch=4)
    ta, tb = Trainer(big, device=CPU), Trainer(acc, device=CPU)
    la, lb = float(ta.train_step(cells, tg)), float(tb.train_step(cells, tg))
    assert abs(la - lb) < 1e-5
    for (n, p), (_, q) in zip(ta.model.named_parameters(), tb.model.named_parameters()):
        assert torch.allclose(p, q, atol=2e-6), n
    ta.close()
    tb.close()


@pytest.mark.parametrize("opt", ["adamw", "muon", "sgd"])
def test_checkpoint_roundtrip_and_identical_resume(tmp_path, opt):
    d = presets.tiny()
    d["optimizer"]["type"] = opt
    d["checkpointing"] = {"checkpoint_interval": 3, "checkpoint_directory": "ckpt", "resume_behavior": "load_latest"}
    d["max_training_steps"] = 100
    cfg = RunConfiguration.from_json(d)
    batches = [_batch(cfg, seed=s) for s in range(6)]
    tr = Trainer(cfg, device=CPU, working_dir=str(tmp_path))
    for i in range(3):
        tr.train_step(*batches[i])
    path = tr.save_checkpoint()
    assert os.path.basename(path) == "checkpoint_step_003.safetensors"
    cont = [float(tr.train_step(*batches[i])) for i in range(3, 6)]
    tr.close()

    tr2 = Trainer(cfg, device=CPU, working_dir=str(tmp_path))
    tr2.load_latest_checkpoint()
    assert tr2.step_count == 3
    resumed = [float(tr2.train_step(*batches[i])) for i in range(3, 6)]
    tr2.close()
    assert resumed == pytest.approx(cont, abs=1e-6)

    header, _ = st.read_header(path)
    keys = set(header)
    assert {"step_count", "dataset_rng_state", "dataset_prefetch_indices", "dataset_prefetch_starts",
            "dataset_prefetch_buffer_index"} <= keys
    assert header["step_count"]["dtype"] == "U64" and header["dataset_prefetch_indices"]["dtype"] == "U32"
    if opt == "adamw":
        assert "optim/action_model/action_model.lstm.layers.0.weights_ih/m" in keys
        assert "optim/frame_head/__optimizer/step" in keys
    if opt == "muon":
        assert any(k.startswith("optim/action_model/muon/") and k.endswith("/momentum") for k in keys)
        assert "optim/action_model/adam/__optimizer/step" in keys


def test_checkpoint_step_mismatch_and_latest_selection(tmp_path):
    cfg = _tiny()
    tr = Trainer(cfg, device=CPU, working_dir=str(tmp_path))
    mgr = CheckpointManager(str(tmp_path / "c"), 50)
    tr.step_count = 7
    p7 = mgr.save(7, tr.model, tr.optimizers, None)
    mgr.save(12, tr.model, tr.optimizers, None)
    mgr.save(60, tr.model, tr.optimizers, None)       # beyond max_training_steps: ignored
    assert mgr.find_latest()[0] == 12
    os.rename(p7, mgr.path_for(8))
    with pytest.raises(ValueError, match="step"):
        mgr.load(mgr.path_for(8), tr.model, tr.optimizers)
    tr.close()


def test_run_training_with_recordings_and_cursor(tmp_path):
    import numpy as np
    from fbamtrain_b200.data import ArrayRecording, SyntheticRecording
    from fbamtrain_b200.tokenizer import Tokenizer
    rec_dir = tmp_path / "train_recordings"
    rec_dir.mkdir()
    for i in range(3):
        r = SyntheticRecording(8, 16, 60, seed=i)
        ArrayRecording(np.stack([r.frame(t)[0] for t in range(60)]), [r.frame(t)[1] for t in range(60)]).save(
            str(rec_dir / f"r{i}.fbrec.npz"))
    Tokenizer(list("abcdefghijklmnopqrstuvwxyz") + ["ab", "th"]).save(str(tmp_path / "tok.txt"))
    d = presets.tiny()
    d["tokenizer_file_path"] = "tok.txt"
    d["train_data_config"]["recordings_directory_path"] = "train_recordings"
    d["model_config"]["action_vocab"] = 0
    d["checkpointing"] = {"checkpoint_interval": 2, "checkpoint_directory": "ck", "resume_behavior": "load_latest",
                          "dataset_cursor_path": "ck/cursor.json"}
    cfg = RunConfiguration.from_json(d)
    tr = Trainer(cfg, device=CPU, working_dir=str(tmp_path))
    assert tr.vocab == 28
    hist = run_training(tr, max_steps=3)
    tr.cursor.flush()
    tr.close()
    assert len(hist) == 3 and all(h["loss/train"] > 0 for h in hist)
    assert os.path.exists(tmp_path / "ck" / "cursor.json")
    assert os.path.exists(tmp_path / "ck" / "checkpoint_step_02.safetensors")


def test_validation_dump_contents():
    cfg = _tiny()
    tr = Trainer(cfg, device=CPU)
    dump = tr.validation_dump(*_batch(cfg))
    for k in ("output", "h_n", "c_n", "loss", "frame_embeddings", "logits"):
        assert k in dump
    assert any(k.startswith("grad_") for k in dump) and any(k.startswith("param_") for k in dump)
    assert dump["logits"].shape == (32, 32)
    tr.close()


# ----------------------------------------------------------------------------- optimizers
def test_adamw_matches_torch_reference():
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(37, 5))
    q = torch.nn.Parameter(p.detach().clone())
    mine = AdamwOptimizer([("w", p)], "optim/x", lr=1e-2, beta1=0.9, beta2=0.99, eps=1e-8, weight_decay=0.1)
    theirs = torch.optim.AdamW([q], lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    for _ in range(5):
        g = torch.randn_like(p)
        p.grad, q.grad = g.clone(), g.clone()
        mine.step()
        theirs.step()
    assert torch.allclose(p, q, atol=1e-6)


def test_adamw_flat_groups_shards_and_master_weights():
    torch.manual_seed(1)
    ps = [("a", torch.nn.Parameter(torch.randn(10, 7).bfloat16())), ("b", torch.nn.Parameter(torch.randn(33).bfloat16()))]
    qs = [(n, torch.nn.Parameter(p.detach().clone())) for n, p in ps]
    groups = build_groups("s", ps, shard_multiple=2)
    flat = AdamwOptimizer(ps, "o", 1e-2, weight_decay=0.1, groups=groups)
    plain = AdamwOptimizer(qs, "o", 1e-2, weight_decay=0.1)
    for _ in range(3):
        for (_, p), (_, q) in zip(ps, qs):
            g = torch.randn(p.shape).bfloat16()
            p.grad.copy_(g)
            q.grad = g.clone()
        # two shard updates together cover the whole group
        flat.step(shard=(0, 2))
        flat.step_count -= 1
        flat.step(shard=(1, 2))
        plain.step()
    for (n, p), (_, q) in zip(ps, qs):
        assert torch.equal(p, q), n
        assert torch.allclose(flat.state[n]["master"], plain.state[n]["master"], atol=1e-7)
    assert groups[0].data.data_ptr() <= ps[1][1].data_ptr() < groups[0].data.data_ptr() + groups[0].numel * 2
    assert ps[1][1].data_ptr() % 256 == groups[0].data.data_ptr() % 256


def test_sgd_nesterov_matches_torch():
    torch.manual_seed(2)
    p = torch.nn.Parameter(torch.randn(11))
    q = torch.nn.Parameter(p.detach().clone())
    mine = SgdOptimizer([("w", p)], "o", lr=0.1, momentum=0.9, nesterov=True, weight_decay=0.01)
    theirs = torch.optim.SGD([q], lr=0.1, momentum=0.9, nesterov=True, weight_decay=0.01)
    for _ in range(4):
        g = torch.randn_like(p)
        p.grad, q.grad = g.clone(), g.clone()
        mine.step()
        theirs.step()
    assert torch.allclose(p, q, atol=1e-6)


def test_newton_schulz_orthogonalises_and_muon_step():
    torch.manual_seed(3)
    g = torch.randn(48, 32)
    u = newton_schulz(g, 5, torch.float32)
    s = torch.linalg.svdvals(u)
    assert s.min() > 0.5 and s.max() < 1.3      # singular values pushed towards 1
    # reference-style oracle written independently: tall matrices are transposed first
    x = g.t() / (g.norm() + 1e-7)
    for _ in range(5):
        a = x @ x.t()
        x = 3.4445 * x + (-4.7750 * a + 2.0315 * a @ a) @ x
    assert torch.allclose(u, x.t(), atol=1e-5)
    p = torch.nn.Parameter(torch.randn(48, 32))
    before = p.detach().clone()
    opt = MuonOptimizer([("w", p)], "o/muon", lr=0.02, momentum=0.0, nesterov=False, weight_decay=0.01)
    p.grad = g.clone()
    opt.step()
    expect = before * (1 - 0.02 * 0.01) - 0.02 * newton_schulz(g, 5).float() * (48 / 32) ** 0.5
    assert torch.allclose(p, expect, atol=5e-3)
    aux = MuonWithAuxAdam([("w", torch.nn.Parameter(torch.randn(4, 4))), ("b", torch.nn.Parameter(torch.randn(4)))],
                          "o", 0.01, 0.9, True, 0.0, 0.9, 0.999, 1e-8)
    assert [n for n, _ in aux.muon.named_params] == ["w"] and [n for n, _ in aux.adam.named_params] == ["b"]


def test_muon_momentum_is_the_reference_moving_average():
    """The stored momentum tensor follows the reference's rule ``m = β·m + (1 − β)·g`` with the update
    ``(1 − β)·g + β·m`` (reference: ``src/optimizers.cpp:1204-1226``), so a momentum tensor written by the reference
    continues correctly here: the step taken from such a tensor equals the step computed by hand from that rule."""
    torch.manual_seed(5)
    beta, lr = 0.95, 0.02
    p = torch.nn.Parameter(torch.randn(24, 40))
    opt = MuonOptimizer([("w", p)], "o/muon", lr=lr, momentum=beta, nesterov=True, weight_decay=0.0)
    m_ref = torch.zeros(24, 40)
    for g in (torch.randn(24, 40), torch.randn(24, 40)):            # two steps of the reference's rule, by hand
        m_ref = beta * m_ref + (1 - beta) * g
    opt.state["w"]["momentum"].copy_(m_ref)                          # as if loaded from a reference checkpoint
    g3 = torch.randn(24, 40)
    before = p.detach().clone()
    p.grad = g3.clone()
    opt.step()
    m3 = beta * m_ref + (1 - beta) * g3
    assert torch.allclose(opt.state["w"]["momentum"], m3, atol=1e-6)
    upd = (1 - beta) * g3 + beta * m3
    expect = before - lr * newton_schulz(upd, 5).float() * max(1.0, 24 / 40) ** 0.5
    assert torch.allclose(p, expect, atol=5e-3)


# ----------------------------------------------------------------------------- reference ops
def test_cell_embed_formula():
    torch.manual_seed(4)
    cp, pos, col = torch.randn(8, 5), torch.randn(6, 5), torch.randn(6, 5)
    cells = torch.tensor([[[3, 0xFF0080, 0x000000], [9, 0, 0x0000FF]]], dtype=torch.int32)  # cp 9 is out of range
    out = ref.cell_embed(cells, cp, pos, col, torch.float32)
    e0 = cp[3] + pos[0] + 1.0 * col[0] + (128 / 255) * col[2]
    e1 = pos[1] + 1.0 * col[5]
    assert torch.allclose(out[0, 0], e0, atol=1e-6) and torch.allclose(out[0, 1], e1, atol=1e-6)


def test_lstm_matches_torch_nn_lstm():
    torch.manual_seed(5)
    lstm = torch.nn.LSTM(6, 8)
    x = torch.randn(7, 3, 6)
    h0, c0 = torch.randn(8), torch.randn(8)
    y, (h, c) = lstm(x, (h0.expand(1, 3, 8).contiguous(), c0.expand(1, 3, 8).contiguous()))
    y2, h2, c2 = ref.lstm_sequence(x, lstm.weight_ih_l0, lstm.weight_hh_l0, lstm.bias_ih_l0, lstm.bias_hh_l0,
                                   h0, c0, torch.float32)
    assert torch.allclose(y, y2, atol=1e-5) and torch.allclose(c[0], c2, atol=1e-5)


def test_embedding_and_mean_modules():
    import torch
    from fbamtrain_b200.models import Embedding, Mean
    from fbamtrain_b200.models.init_utils import SeedSequence
    emb = Embedding(10, 4, torch.float32, SeedSequence(7))
    ids = torch.tensor([[0, 3, 9], [10, -1, 3]])
    out = emb(ids)
    assert out.shape == (2, 3, 4)
    assert torch.equal(out[0, 1], emb.weight[3]) and torch.equal(out[1, 2], emb.weight[3])
    assert float(out[1, 0].abs().sum()) == 0.0 and float(out[1, 1].abs().sum()) == 0.0   # out of range -> zero row
    out.sum().backward()
    assert float(emb.weight.grad[3].sum()) == 8.0 and float(emb.weight.grad[5].abs().sum()) == 0.0
    x = torch.arange(24, dtype=torch.float32).view(2, 3, 4).requires_grad_(True)
    m = Mean(1)(x)
    assert torch.allclose(m, x.detach().mean(1))
    m.sum().backward()
    assert torch.allclose(x.grad, torch.full_like(x, 1.0 / 3))


def test_frame_head_recompute_gives_identical_gradients():
    import copy
    import torch
    from fbamtrain_b200 import RunConfiguration, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.models import FbamModel
    from fbamtrain_b200.utils import flops
    d = presets.tiny()
    cfg = RunConfiguration.from_json(d)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=4, pin=False)
    cells, targets = src.next_batch(2, cfg.train_sequence_length)
    grads = {}
    for recompute in (False, True):
        mc = copy.deepcopy(cfg.model_config)
        mc.frame_head_recompute = recompute
        torch.manual_seed(0)
        model = FbamModel(mc, 32)
        model.frame_chunk = 8                      # 32 frames -> four chunks
        flops.reset()
        model(cells, targets, 1.0 / 32).backward()
        grads[recompute] = {n: p.grad.clone() for n, p in model.named_parameters()}
    for n, g in grads[False].items():
        assert torch.allclose(g, grads[True][n], atol=1e-7), n


def test_oracle_ops_agree_with_torch_builtins():
    """The PyTorch definitions every kernel is compared against, checked against independent torch formulations."""
    import torch
    import torch.nn.functional as F
    torch.manual_seed(3)
    q, k, v = (torch.randn(2, 9, 3, 8) for _ in range(3))
    for causal in (False, True):
        want = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                              is_causal=causal).transpose(1, 2)
        assert torch.allclose(ref.attention(q, k, v, causal), want, atol=1e-5)
    x = torch.randn(5, 7, requires_grad=True)
    (g,) = torch.autograd.grad(ref.gelu(x).sum(), x)
    assert torch.allclose(g, ref.gelu_grad(x.detach()), atol=1e-6)
    img = torch.randn(2, 6, 8, 4)
    want = F.avg_pool2d(img.permute(0, 3, 1, 2), 2).permute(0, 2, 3, 1)
    assert torch.allclose(ref.avg_pool2x2_nhwc(img), want, atol=1e-6)
    w = torch.randn(5, 3, 3, 4)
    for stride, pad, dil in ((1, 1, 1), (2, 1, 1), (1, 2, 2)):
        want = F.conv2d(img.permute(0, 3, 1, 2), w.permute(0, 3, 1, 2), None, stride, pad, dil).permute(0, 2, 3, 1)
        assert torch.allclose(ref.conv2d_nhwc(img, w, stride, pad, dil), want, atol=1e-5)
    xr = torch.randn(4, 16)
    gamma = torch.rand(16) + 0.5
    want = xr / torch.sqrt((xr * xr).mean(-1, keepdim=True) + 1e-5) * gamma
    assert torch.allclose(ref.rms_norm(xr, gamma, 1e-5), want, atol=1e-6)
    hdn, head = torch.randn(6, 16), torch.randn(24, 16)
    tg = torch.randint(0, 20, (6,))
    want = F.cross_entropy(hdn @ head[:20].t(), tg, reduction="sum") * 0.25
    assert torch.allclose(ref.lm_head_ce(hdn, head, tg, 20, 0.25), want, atol=1e-5)
    gate_in = torch.randn(3, 10)
    vv, gg = gate_in.chunk(2, -1)
    assert torch.allclose(ref.geglu(gate_in), vv * F.gelu(gg), atol=1e-6)


def test_training_on_raw_recordings_uses_native_loader_and_matches_python_path(tmp_path):
    """The same recordings as ``.fbrec`` (native loader on the prefetch thread, two host buffers in turn) and as
    ``.fbrec.npz`` (per-frame Python assembly) give the same loss curve, also across a checkpoint resume."""
    import numpy as np
    from fbamtrain_b200.data import ArrayRecording, SyntheticRecording
    from fbamtrain_b200.data.recording import write_raw_recording
    from fbamtrain_b200.tokenizer import Tokenizer
    curves = {}
    for kind in ("raw", "npz"):
        root = tmp_path / kind
        rec_dir = root / "rec"
        rec_dir.mkdir(parents=True)
        for i in range(3):
            r = SyntheticRecording(8, 16, 60, seed=i)
            cells = np.stack([r.frame(t)[0] for t in range(60)])
            keys = [r.frame(t)[1] for t in range(60)]
            if kind == "raw":
                write_raw_recording(str(rec_dir / f"r{i}.fbrec"), cells, keys)
            else:
                ArrayRecording(cells, keys).save(str(rec_dir / f"r{i}.fbrec.npz"))
        Tokenizer(list("abcdefghijklmnopqrstuvwxyz") + ["ab", "th"]).save(str(root / "tok.txt"))
        d = presets.tiny()
        d["tokenizer_file_path"] = "tok.txt"
        d["train_data_config"]["recordings_directory_path"] = "rec"
        d["model_config"]["action_vocab"] = 0
        d["checkpointing"] = {"checkpoint_interval": 2, "checkpoint_directory": "ck", "resume_behavior": "load_latest"}
        cfg = RunConfiguration.from_json(d)
        tr = Trainer(cfg, device=CPU, working_dir=str(root))
        from fbamtrain_b200.train import _make_assembler
        assert (_make_assembler(tr, cfg.micro_batch_size) is not None) == (kind == "raw")
        hist = run_training(tr, max_steps=3)
        tr.close()
        tr = Trainer(cfg, device=CPU, working_dir=str(root))         # resumes from step 2's checkpoint
        hist2 = run_training(tr, max_steps=2)
        tr.close()
        curves[kind] = [h["loss/train"] for h in hist] + [h["loss/train"] for h in hist2]
    assert len(curves["raw"]) == 5
    assert curves["raw"] == pytest.approx(curves["npz"], abs=1e-6)
    assert curves["raw"][2] == pytest.approx(curves["raw"][3], abs=1e-6)   # step 2 replayed identically after resume


def test_host_loss_returns_each_steps_loss_without_the_returned_tensor():
    """``Trainer.host_loss(step)`` reads the step's slot of the loss ring: same value as the returned scalar, also
    when it is read one step late, and an error once the slot has been reused."""
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    cfg = RunConfiguration.from_json(presets.tiny())
    tr = Trainer(cfg, device=torch.device("cpu"))
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, tr.vocab, seed=3,
                               pin=False)
    returned, read_late = [], []
    previous = None
    for _ in range(3):
        step = tr.step_count
        returned.append(float(tr.train_step(*src.next_batch(2, cfg.train_sequence_length))))
        if previous is not None:
            read_late.append(tr.host_loss(previous))
        previous = step
    read_late.append(tr.host_loss(previous))
    assert read_late == pytest.approx(returned, rel=1e-6)
    with pytest.raises(ValueError):
        tr.host_loss(99)
    tr.close()


def test_progress_lines_at_info_level(monkeypatch, capsys):
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    monkeypatch.setenv("FBAMTRAIN_LOG_LEVEL", "INFO")
    cfg = RunConfiguration.from_json(presets.tiny())
    tr = Trainer(cfg, device=torch.device("cpu"))
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, tr.vocab, seed=3,
                               pin=False)
    tr.train_step(*src.next_batch(2, cfg.train_sequence_length))
    tr.logger.drain()
    tr.close()
    out = capsys.readouterr().out
    frames = 2 * cfg.train_sequence_length
    assert f"Frame head: frames {frames}/{frames} processed | FPS:" in out
    assert f"Backward: frames {frames}/{frames} processed | FPS:" in out
    assert "Step 0 took" in out


def test_validation_reads_the_validation_recordings(tmp_path):
    """With a validation folder configured, the periodic validation draws its sequences from those recordings
    through a second seeded iterator; without one it falls back to seeded synthetic frames."""
    import numpy as np
    from fbamtrain_b200.data import ArrayRecording, SyntheticRecording
    from fbamtrain_b200.tokenizer import Tokenizer
    from fbamtrain_b200.train import _validation_source
    for name, seeds in (("rec", (0, 1)), ("val", (7,))):
        (tmp_path / name).mkdir()
        for i in seeds:
            r = SyntheticRecording(8, 16, 50, seed=i)
            cells = np.stack([r.frame(t)[0] for t in range(50)])
            ArrayRecording(cells, [r.frame(t)[1] for t in range(50)]).save(str(tmp_path / name / f"r{i}.fbrec.npz"))
    Tokenizer(list("abcdefghijklmnopqrstuvwxyz") + ["ab", "th"]).save(str(tmp_path / "tok.txt"))
    d = presets.tiny()
    d["tokenizer_file_path"] = "tok.txt"
    d["model_config"]["action_vocab"] = 0
    d["train_data_config"]["recordings_directory_path"] = "rec"
    d["validation_data_config"]["recordings_directory_path"] = "val"
    d["enable_validation"], d["validation_interval"] = True, 1
    cfg = RunConfiguration.from_json(d)
    tr = Trainer(cfg, device=CPU, working_dir=str(tmp_path))
    source = _validation_source(tr)
    assert source.__name__ == "from_recordings"
    vc, vt = source()
    assert tuple(vc.shape[:2]) == (cfg.micro_batch_size, cfg.validation_sequence_length)
    source.iterator.close()
    lines = []
    tr.logger.log_validation = lambda step, loss: lines.append((step, loss))
    run_training(tr, max_steps=2)
    tr.close()
    assert [s for s, _ in lines] == [1, 2] and all(np.isfinite(l) for _, l in lines)
    d["validation_data_config"]["recordings_directory_path"] = ""
    tr = Trainer(RunConfiguration.from_json(d), device=CPU, working_dir=str(tmp_path))
    assert _validation_source(tr).__name__ == "synthetic"
    tr.close()


def test_background_checkpoint_write_snapshots_before_training_continues(tmp_path, monkeypatch):
    """With ``background_write`` the file is written by a worker thread from a snapshot taken inside ``save``:
    steps taken while the (artificially slow) write is in flight do not leak into the file, the file name appears
    only when complete, and resuming from it repeats the continued run."""
    import threading
    from fbamtrain_b200.utils import safetensors_io
    d = presets.tiny()
    d["checkpointing"] = {"checkpoint_interval": 3, "checkpoint_directory": "ckpt", "resume_behavior": "load_latest",
                          "background_write": True}
    d["max_training_steps"] = 100
    cfg = RunConfiguration.from_json(d)
    assert cfg.checkpointing.background_write
    batches = [_batch(cfg, seed=s) for s in range(6)]
    gate = threading.Event()
    real_save = safetensors_io.save_file

    def slow_save(tensors, path, metadata=None):
        gate.wait(30)
        real_save(tensors, path, metadata)
    monkeypatch.setattr(safetensors_io, "save_file", slow_save)
    tr = Trainer(cfg, device=CPU, working_dir=str(tmp_path))
    for i in range(3):
        tr.train_step(*batches[i])
    path = tr.save_checkpoint()
    assert not os.path.exists(path)                                    # still being written
    cont = [float(tr.train_step(*batches[i])) for i in range(3, 6)]   # training goes on meanwhile
    gate.set()
    tr.close()                                                         # waits for the writer
    assert os.path.exists(path) and not os.path.exists(path + ".tmp")
    monkeypatch.setattr(safetensors_io, "save_file", real_save)
    tr2 = Trainer(cfg, device=CPU, working_dir=str(tmp_path))
    tr2.load_latest_checkpoint()
    assert tr2.step_count == 3
    resumed = [float(tr2.train_step(*batches[i])) for i in range(3, 6)]
    tr2.close()
    assert resumed == pytest.approx(cont, abs=1e-6)


def test_background_checkpoint_write_errors_surface(tmp_path, monkeypatch):
    from fbamtrain_b200.checkpoint import CheckpointManager
    from fbamtrain_b200.models import FbamModel
    from fbamtrain_b200.utils import safetensors_io
    cfg = RunConfiguration.from_json(presets.tiny())
    model = FbamModel(cfg.model_config, 32)

    def failing_save(tensors, path, metadata=None):
        raise OSError("disk full")
    monkeypatch.setattr(safetensors_io, "save_file", failing_save)
    manager = CheckpointManager(str(tmp_path / "ck"), 100, background=True)
    manager.save(1, model, {}, None)
    with pytest.raises(RuntimeError, match="disk full"):
        manager.wait()
    manager.wait()                                                     # reported once


@pytest.mark.parametrize("opt", ["muon", "adamw", "sgd"])
@pytest.mark.parametrize("mode,reduction", [("dilated", "last_pos"), ("geglu", "mean")])
def test_scaled_down_reference_sample_configuration_trains(opt, mode, reduction):
    """The reference's sample run configuration (its own architecture: attention layers inside the frame head,
    dilated or GeGLU downsampling, last-position or mean reduction, one LSTM layer straight into the head), scaled
    down to CPU size, trains with every optimizer."""
    import copy
    from test_config import DEBUG_JSON
    d = copy.deepcopy(DEBUG_JSON)
    d["micro_batch_size"] = d["total_batch_size"] = 2
    d["train_sequence_length"] = d["validation_sequence_length"] = 8
    d["frame_rows"], d["frame_cols"] = 8, 16
    d["tokenizer_file_path"] = ""
    d["optimizer"]["type"] = opt
    d["model_config"].update({"n_embed": 64, "n_layer": 1, "n_head": 2, "frame_rows": 8, "frame_cols": 16,
                              "dtype": "fp32", "use_fp16_accumulation": False, "action_vocab": 48,
                              "downsample_conv_mode": mode, "frame_head_reduction_strategy": reduction})
    cfg = RunConfiguration.from_json(d)
    tr = Trainer(cfg, device=CPU)
    cells, targets = _batch(cfg, seed=2)
    losses = [float(tr.train_step(cells, targets)) for _ in range(4)]
    tr.close()
    assert all(math.isfinite(x) for x in losses) and losses[-1] < losses[0]


def test_frame_replay_gives_the_same_loss_and_gradients():
    """Model key ``frame_replay``: frames stay on the host, every chunk is fetched twice (forward and backward) and the
    frame head runs again in the backward — same loss, same gradients as keeping everything."""
    import torch
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    results = {}
    for replay in (False, True):
        d = presets.tiny()
        d["model_config"]["frame_replay"] = replay
        cfg = RunConfiguration.from_json(d)
        tr = Trainer(cfg, device=torch.device("cpu"), frame_chunk=5)
        src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=3, pin=False)
        cells, tg = src.next_batch(cfg.micro_batch_size, cfg.train_sequence_length)
        tr.zero_grad()
        loss = tr._forward_backward(cells, tg)
        results[replay] = (float(loss), {n: p.grad.detach().clone() for n, p in tr.model.named_parameters()})
        if replay:
            chunks = (cells.shape[0] * cells.shape[1] + 4) // 5
            assert tr.last_replay.num_chunks == chunks and tr.last_replay.uploads == 2 * chunks
        tr.close()
    assert results[True][0] == results[False][0]
    for name, g in results[False][1].items():
        assert torch.allclose(results[True][1][name], g, atol=1e-7), name
