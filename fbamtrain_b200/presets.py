"""Named run configurations for the benchmark model family.

``fbam_toy`` (fp32, CPU oracle), ``fbam_small`` (bf16, pure data parallel, AdamW), ``fbam_1b``
(bf16, Muon on matrices + AdamW elsewhere).  Each returns a run-configuration JSON object that
:class:`fbamtrain_b200.config.RunConfiguration` parses; the keys beyond the reference's schema are the
optional additions documented in :mod:`fbamtrain_b200.config`.
"""
from __future__ import annotations

import copy
from typing import Any, Dict


def _base(rows, cols, seq, micro, total, steps, opt, model) -> Dict[str, Any]:
    return {
        "micro_batch_size": micro, "total_batch_size": total,
        "train_sequence_length": seq, "validation_sequence_length": seq,
        "validation_interval": 0, "enable_validation": False, "max_training_steps": steps,
        "frame_rows": rows, "frame_cols": cols, "tokenizer_file_path": "",
        "train_data_config": {"recordings_directory_path": "", "iteration_seed": 0},
        "validation_data_config": {"recordings_directory_path": "", "iteration_seed": 1},
        "optimizer": opt,
        "checkpointing": {"checkpoint_interval": 1000000, "checkpoint_directory": "checkpoints",
                          "resume_behavior": "none"},
        "model_config": model,
    }


def _opt(kind, lr, wd, momentum=0.95, nesterov=True):
    return {"type": kind, "learning_rate": lr, "weight_decay": wd, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8,
            "momentum": momentum, "nesterov": nesterov}


def fbam_toy() -> Dict[str, Any]:
    model = {"frame_rows": 24, "frame_cols": 80, "n_embed": 256, "n_layer": 0, "n_head": 4, "downsample_blocks": 1,
             "max_code_point": 256, "rms_norm_eps": 1e-5, "bias": True, "dtype": "fp32",
             "downsample_conv_mode": "dilated", "downsample_conv_dilation": 1, "model_init_seed": 0,
             "use_fp16_accumulation": False, "streaming_chunk_size": 16, "recompute_interval": 1,
             "frame_head_reduction_strategy": "mean",
             "cell_embed_dim": 64, "downsample_channels": [128], "downsample_conv_stride": 2,
             "downsample_norm": False, "frame_proj": True, "lstm_layers": 1, "lstm_hidden": 256,
             "action_blocks": 2, "action_heads": 4, "action_mlp_dim": 1024, "action_vocab": 64}
    return _base(24, 80, 64, 4, 4, 10, _opt("adamw", 3e-4, 0.1), model)


def fbam_small(micro_batch: int = 8, world: int = 1) -> Dict[str, Any]:
    model = {"frame_rows": 48, "frame_cols": 160, "n_embed": 1024, "n_layer": 0, "n_head": 16,
             "downsample_blocks": 2, "max_code_point": 512, "rms_norm_eps": 1e-5, "bias": True, "dtype": "bf16",
             "downsample_conv_mode": "dilated", "downsample_conv_dilation": 1, "model_init_seed": 0,
             "use_fp16_accumulation": False, "streaming_chunk_size": 64, "recompute_interval": 1,
             "frame_head_reduction_strategy": "mean",
             "cell_embed_dim": 128, "downsample_channels": [256, 512], "downsample_conv_stride": 2,
             "downsample_norm": False, "frame_proj": True, "lstm_layers": 2, "lstm_hidden": 1024,
             "action_blocks": 8, "action_heads": 16, "action_mlp_dim": 4096, "action_vocab": 4096}
    return _base(48, 160, 1024, micro_batch, micro_batch * world, 1000, _opt("adamw", 3e-4, 0.1), model)


def fbam_1b(micro_batch: int = 4, world: int = 8) -> Dict[str, Any]:
    cfg = fbam_small(micro_batch, world)
    cfg["train_sequence_length"] = cfg["validation_sequence_length"] = 2048
    cfg["optimizer"] = _opt("muon", 2e-3, 0.01)
    m = cfg["model_config"]
    m.update({"n_embed": 2048, "lstm_hidden": 2048, "action_blocks": 16, "action_heads": 16,
              "action_mlp_dim": 8192, "action_vocab": 8192})
    return cfg


def tiny(dtype: str = "fp32") -> Dict[str, Any]:
    """A seconds-scale configuration for tests and smoke runs (same structure as ``fbam_small``)."""
    cfg = copy.deepcopy(fbam_toy())
    cfg["train_sequence_length"] = cfg["validation_sequence_length"] = 16
    cfg["micro_batch_size"] = cfg["total_batch_size"] = 2
    cfg["frame_rows"], cfg["frame_cols"] = 8, 16
    m = cfg["model_config"]
    m.update({"frame_rows": 8, "frame_cols": 16, "n_embed": 64, "n_head": 2, "cell_embed_dim": 32,
              "downsample_channels": [64], "lstm_hidden": 64, "lstm_layers": 2, "action_blocks": 1,
              "action_heads": 2, "action_mlp_dim": 128, "action_vocab": 32, "dtype": dtype,
              "streaming_chunk_size": 4})
    return cfg


PRESETS = {"fbam_toy": fbam_toy, "fbam_small": fbam_small, "fbam_1b": fbam_1b, "tiny": tiny}
