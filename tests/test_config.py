import copy
import json
import os

import pytest
from conftest import reference_path

from fbamtrain_b200 import presets
from fbamtrain_b200.config import ConfigError, ParallelConfiguration, RunConfiguration

# The reference's sample run configuration, reproduced as data (working_dir/run-configs/debug.json).
DEBUG_JSON = {
    "micro_batch_size": 32, "total_batch_size": 32, "train_sequence_length": 1024,
    "validation_sequence_length": 1024, "validation_interval": 100, "enable_validation": False,
    "max_training_steps": 100000, "frame_cols": 160, "frame_rows": 48, "tokenizer_file_path": "tokenizer.txt",
    "train_data_config": {"recordings_directory_path": "train_recordings", "iteration_seed": 42},
    "validation_data_config": {"recordings_directory_path": "validation_recordings", "iteration_seed": 42},
    "optimizer": {"type": "muon", "learning_rate": 0.002, "weight_decay": 0.01, "beta1": 0.9, "beta2": 0.999,
                  "eps": 1e-08, "momentum": 0.0, "nesterov": False},
    "checkpointing": {"checkpoint_interval": 1000, "checkpoint_directory": "checkpoints",
                      "resume_behavior": "load_latest", "dataset_cursor_path": "checkpoints/dataset_cursor.json"},
    "model_config": {"dtype": "fp16", "n_embed": 1024, "n_layer": 3, "n_head": 8, "downsample_blocks": 2,
                     "max_code_point": 256, "rms_norm_eps": 1e-05, "bias": True, "downsample_conv_mode": "dilated",
                     "downsample_conv_dilation": 2, "frame_cols": 160, "frame_rows": 48, "model_init_seed": 42,
                     "use_fp16_accumulation": True, "streaming_chunk_size": 1, "recompute_interval": 1,
                     "frame_head_reduction_strategy": "last_pos"},
}
FHP_DDP = {"frame_head_parallel": {"use_frame_head_parallel": True, "transport": "ccl",
                                   "ccl_rendezvous": {"ip": "127.0.0.1", "port": 29500}},
           "ddp_parallel": {"use_ddp_parallel": True, "transport": "ftccl",
                            "ftccl_master": {"ip": "127.0.0.1", "port": 48148}}}
FHP_ONLY = {"frame_head_parallel": {"use_frame_head_parallel": True, "transport": "ccl",
                                    "ccl_rendezvous": {"ip": "127.0.0.1", "port": 29500}},
            "ddp_parallel": {"use_ddp_parallel": False}}


def test_reference_debug_config_parses():
    cfg = RunConfiguration.from_json(copy.deepcopy(DEBUG_JSON))
    assert cfg.micro_batch_size == 32 and cfg.grad_accum_steps == 1
    m = cfg.model_config
    assert (m.dtype, m.n_layer, m.frame_head_reduction_strategy) == ("fp16", 3, "last_pos")
    # defaults of the added keys reproduce the reference's model
    assert m.lstm_layers == 1 and m.action_blocks == 0 and m.downsample_conv_stride == 1 and not m.frame_proj
    assert m.block_channels() == [(1024, 1024), (1024, 1024)]
    assert cfg.optimizer_config.type == "muon" and cfg.checkpointing.resume_behavior == "load_latest"


def test_reference_file_on_disk_if_present():
    path = reference_path("working_dir", "run-configs", "debug.json")
    if not os.path.exists(path):
        pytest.skip("reference tree not mounted")
    assert RunConfiguration.from_json_file(path) is not None
    assert RunConfiguration.from_json_file(path + ".missing") is None


@pytest.mark.parametrize("key", ["micro_batch_size", "train_data_config", "optimizer", "checkpointing",
                                 "model_config", "tokenizer_file_path", "max_training_steps"])
def test_missing_required_run_key(key):
    bad = copy.deepcopy(DEBUG_JSON)
    del bad[key]
    with pytest.raises(ConfigError, match=key):
        RunConfiguration.from_json(bad)


@pytest.mark.parametrize("key", ["n_embed", "rms_norm_eps", "use_fp16_accumulation", "streaming_chunk_size",
                                 "recompute_interval", "downsample_conv_mode"])
def test_missing_required_model_key(key):
    bad = copy.deepcopy(DEBUG_JSON)
    del bad["model_config"][key]
    with pytest.raises(ConfigError, match=key):
        RunConfiguration.from_json(bad)


def test_cross_field_rules():
    bad = copy.deepcopy(DEBUG_JSON)
    bad["total_batch_size"] = 33
    with pytest.raises(ConfigError, match="multiple"):
        RunConfiguration.from_json(bad)
    bad = copy.deepcopy(DEBUG_JSON)
    bad["model_config"]["dtype"] = "bf16"
    with pytest.raises(ConfigError, match="use_fp16_accumulation"):
        RunConfiguration.from_json(bad)
    bad = copy.deepcopy(DEBUG_JSON)
    bad["checkpointing"]["resume_behavior"] = "sometimes"
    with pytest.raises(ConfigError):
        RunConfiguration.from_json(bad)
    ok = copy.deepcopy(DEBUG_JSON)
    ok["checkpointing"]["resume_behavior"] = "disabled"
    assert RunConfiguration.from_json(ok).checkpointing.resume_behavior == "none"
    bad = copy.deepcopy(DEBUG_JSON)
    bad["micro_batch_size"] = -1
    with pytest.raises(ConfigError):
        RunConfiguration.from_json(bad)


def test_parallel_configs():
    a = ParallelConfiguration.from_json(copy.deepcopy(FHP_DDP))
    assert a.ddp_parallel.transport == "ftccl" and a.ddp_parallel.ftccl_master.port == 48148
    assert a.frame_head_parallel.ccl_rendezvous.ip == "127.0.0.1"
    b = ParallelConfiguration.from_json(copy.deepcopy(FHP_ONLY))
    assert not b.ddp_parallel.use_ddp_parallel
    bad = copy.deepcopy(FHP_ONLY)
    bad["ddp_parallel"]["transport"] = "ccl"
    with pytest.raises(ConfigError, match="illegal"):
        ParallelConfiguration.from_json(bad)
    bad = copy.deepcopy(FHP_DDP)
    bad["ddp_parallel"]["ccl_rendezvous"] = {"ip": "1.2.3.4", "port": 1}
    with pytest.raises(ConfigError, match="illegal"):
        ParallelConfiguration.from_json(bad)
    bad = copy.deepcopy(FHP_DDP)
    bad["frame_head_parallel"]["transport"] = "ftccl"
    with pytest.raises(ConfigError):
        ParallelConfiguration.from_json(bad)


@pytest.mark.parametrize("name", ["fbam_toy", "fbam_small", "fbam_1b", "tiny"])
def test_presets_parse(name):
    cfg = RunConfiguration.from_json(json.loads(json.dumps(presets.PRESETS[name]())))
    assert cfg.model_config.frame_proj and cfg.model_config.downsample_conv_stride == 2


def test_shipped_sample_configurations_parse():
    import glob
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")
    runs = sorted(glob.glob(os.path.join(root, "*.json")))
    pars = sorted(glob.glob(os.path.join(root, "parallel", "*.json")))
    assert len(runs) >= 4 and len(pars) >= 3
    for p in runs:
        assert RunConfiguration.from_json_file(p) is not None
    for p in pars:
        assert ParallelConfiguration.from_json_file(p) is not None


def test_shipped_sample_configurations_parse():
    """Every file under ``configs/`` is a valid run / parallel configuration."""
    import glob
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")
    runs = sorted(glob.glob(os.path.join(root, "*.json")))
    pars = sorted(glob.glob(os.path.join(root, "parallel", "*.json")))
    assert runs and pars
    for f in runs:
        cfg = RunConfiguration.from_json_file(f)
        assert cfg is not None and cfg.total_batch_size % cfg.micro_batch_size == 0, f
    for f in pars:
        assert ParallelConfiguration.from_json_file(f) is not None, f
