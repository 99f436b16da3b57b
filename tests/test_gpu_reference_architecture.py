"""The reference's own architecture (its sample run configuration scaled down: attention layers inside the frame
head, dilated / GeGLU downsampling convolutions followed by 2x2 average pooling, last-position / mean reduction, one
LSTM layer straight into the LM head) on the native kernels against the PyTorch op definitions."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,reduction", [("dilated", "last_pos"), ("geglu", "mean")])
def test_reference_architecture_native_vs_reference_path(mode, reduction):
    from test_config import DEBUG_JSON
    from fbamtrain_b200 import RunConfiguration, Trainer, ops
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.ops import native as nv
    d = copy.deepcopy(DEBUG_JSON)
    d["micro_batch_size"] = d["total_batch_size"] = 2
    d["train_sequence_length"] = d["validation_sequence_length"] = 16
    d["frame_rows"], d["frame_cols"] = 8, 16
    d["tokenizer_file_path"] = ""
    d["optimizer"]["type"] = "adamw"
    d["model_config"].update({"n_embed": 128, "n_layer": 1, "n_head": 2, "frame_rows": 8, "frame_cols": 16,
                              "dtype": "bf16", "use_fp16_accumulation": False, "action_vocab": 64,
                              "downsample_conv_mode": mode, "frame_head_reduction_strategy": reduction})
    cfg = RunConfiguration.from_json(d)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 64, seed=0, pin=False)
    cells, tg = src.next_batch(2, 16)
    losses = {}
    for backend in ("auto", "torch"):
        ops.set_backend(backend)
        try:
            tr = Trainer(cfg, device=torch.device("cuda"))
            losses[backend] = [float(tr.train_step(cells, tg)) for _ in range(3)]
            nv.check_status(torch.device("cuda"))
            tr.close()
        finally:
            ops.set_backend("auto")
    assert losses["auto"] == pytest.approx(losses["torch"], abs=5e-2)
    assert losses["auto"][-1] < losses["auto"][0]
