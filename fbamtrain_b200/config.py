"""Run-configuration and parallel-configuration JSON schemas.

The JSON format is the one the reference trainer reads (reference:
``include/config.h:28-166``, ``src/config.cpp:105-829``): every key listed there is
accepted with the same required/optional status and the same cross-field rules, so
``working_dir/run-configs/debug.json`` and the two sample parallel configs parse verbatim.

The model built here has parts the reference lacks (conv stride, frame-vector projection,
multi-layer LSTM, causal action-model blocks, an explicit action vocabulary).  Those are
driven by *additional optional keys* whose defaults reproduce the reference's behaviour.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, Optional


class ConfigError(ValueError):
    """Raised for a malformed configuration; the message names the offending key."""


def _is_uint(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v >= 0


def _is_number(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _require(obj: Dict[str, Any], key: str, ctx: str) -> Any:
    if key not in obj:
        raise ConfigError(f"Missing '{key}' property in {ctx} JSON.")
    return obj[key]


def _uint(obj: Dict[str, Any], key: str, ctx: str) -> int:
    v = _require(obj, key, ctx)
    if not _is_uint(v):
        raise ConfigError(f"'{key}' property must be an unsigned integer in {ctx} JSON.")
    return int(v)


def _opt_uint(obj: Dict[str, Any], key: str, ctx: str, default: int) -> int:
    if key not in obj:
        return default
    return _uint(obj, key, ctx)


def _num(obj: Dict[str, Any], key: str, ctx: str) -> float:
    v = _require(obj, key, ctx)
    if not _is_number(v):
        raise ConfigError(f"'{key}' property must be a floating point number in {ctx} JSON.")
    return float(v)


def _bool(obj: Dict[str, Any], key: str, ctx: str) -> bool:
    v = _require(obj, key, ctx)
    if not isinstance(v, bool):
        raise ConfigError(f"'{key}' property must be a boolean in {ctx} JSON.")
    return v


def _str(obj: Dict[str, Any], key: str, ctx: str, non_empty: bool = False) -> str:
    v = _require(obj, key, ctx)
    if not isinstance(v, str):
        raise ConfigError(f"'{key}' property must be a string in {ctx} JSON.")
    if non_empty and not v:
        raise ConfigError(f"'{key}' property must be a non-empty string in {ctx} JSON.")
    return v


def _obj(obj: Dict[str, Any], key: str, ctx: str) -> Dict[str, Any]:
    v = _require(obj, key, ctx)
    if not isinstance(v, dict):
        raise ConfigError(f"'{key}' property must be a JSON object in {ctx} JSON.")
    return v


_DTYPES = {"fp16": "fp16", "float16": "fp16", "half": "fp16",
           "bf16": "bf16", "bfloat16": "bf16",
           # fp32 is an addition for the CPU oracle configuration
           "fp32": "fp32", "float32": "fp32"}
_REDUCTIONS = ("mean", "last_pos")
_RESUME = {"load_latest": "load_latest", "none": "none", "disabled": "none"}


@dataclass
class DatasetConfiguration:
    recordings_directory_path: str
    iteration_seed: int

    @staticmethod
    def from_json(o: Dict[str, Any]) -> "DatasetConfiguration":
        ctx = "dataset configuration"
        return DatasetConfiguration(_str(o, "recordings_directory_path", ctx), _uint(o, "iteration_seed", ctx))


@dataclass
class FbamModelConfiguration:
    # --- keys of the reference (src/config.cpp:132-267) ---
    frame_rows: int
    frame_cols: int
    n_embed: int
    n_layer: int
    n_head: int
    downsample_blocks: int
    max_code_point: int
    rms_norm_eps: float
    bias: bool
    downsample_conv_mode: str
    downsample_conv_dilation: int
    model_init_seed: int
    use_fp16_accumulation: bool
    streaming_chunk_size: int
    recompute_interval: int
    dtype: str = "fp16"
    frame_head_reduction_strategy: str = "mean"
    # --- additional keys (defaults reproduce the reference's model) ---
    cell_embed_dim: int = 0            # 0 -> n_embed (reference: cells embedded at n_embed)
    downsample_channels: tuple = ()    # per-block conv output channels; () -> n_embed (2x for geglu)
    downsample_conv_stride: int = 1    # 1 = reference (conv s1 + 2x2 pool); 2 = strided conv, no per-block pool
    downsample_norm: bool = True       # RMSNorm before each downsample conv (reference does)
    frame_proj: bool = False           # linear projection of the pooled frame vector to n_embed
    lstm_layers: int = 1
    lstm_hidden: int = 0               # 0 -> n_embed
    action_blocks: int = 0             # causal MHA/MLP blocks after the LSTM (0 = reference: none)
    action_heads: int = 0              # 0 -> n_head
    action_mlp_dim: int = 0            # 0 -> 4 * n_embed
    action_vocab: int = 0              # 0 -> tokenizer size (reference)
    frame_head_recompute: bool = False  # recompute the frame head's activations in the backward, chunk by chunk
    frame_replay: bool = False          # frames stay in host memory; chunks are uploaded again for the backward

    @staticmethod
    def from_json(o: Dict[str, Any]) -> "FbamModelConfiguration":
        ctx = "model configuration"
        kw: Dict[str, Any] = dict(
            frame_rows=_uint(o, "frame_rows", ctx), frame_cols=_uint(o, "frame_cols", ctx),
            n_embed=_uint(o, "n_embed", ctx), n_layer=_uint(o, "n_layer", ctx),
            n_head=_uint(o, "n_head", ctx), downsample_blocks=_uint(o, "downsample_blocks", ctx),
            max_code_point=_uint(o, "max_code_point", ctx), rms_norm_eps=_num(o, "rms_norm_eps", ctx),
            bias=_bool(o, "bias", ctx),
            downsample_conv_mode=_str(o, "downsample_conv_mode", ctx, non_empty=True),
            downsample_conv_dilation=_uint(o, "downsample_conv_dilation", ctx),
            model_init_seed=_uint(o, "model_init_seed", ctx),
            use_fp16_accumulation=_bool(o, "use_fp16_accumulation", ctx),
            streaming_chunk_size=_uint(o, "streaming_chunk_size", ctx),
            recompute_interval=_uint(o, "recompute_interval", ctx),
        )
        if "dtype" in o:
            raw = _str(o, "dtype", ctx, non_empty=True)
            if raw.lower() not in _DTYPES:
                raise ConfigError(f"Unsupported model dtype '{raw}' (expected fp16, bf16 or fp32).")
            kw["dtype"] = _DTYPES[raw.lower()]
        if "frame_head_reduction_strategy" in o:
            raw = _str(o, "frame_head_reduction_strategy", ctx, non_empty=True)
            if raw not in _REDUCTIONS:
                raise ConfigError(f"Unsupported frame_head_reduction_strategy '{raw}' (expected mean or last_pos).")
            kw["frame_head_reduction_strategy"] = raw
        if kw.get("dtype", "fp16") == "bf16" and kw["use_fp16_accumulation"]:
            raise ConfigError("use_fp16_accumulation cannot be true when dtype is bf16.")
        if kw["downsample_conv_mode"] not in ("dilated", "geglu"):
            raise ConfigError("'downsample_conv_mode' must be \"dilated\" or \"geglu\".")
        for key in ("cell_embed_dim", "downsample_conv_stride", "lstm_layers", "lstm_hidden",
                    "action_blocks", "action_heads", "action_mlp_dim", "action_vocab"):
            if key in o:
                kw[key] = _uint(o, key, ctx)
        for key in ("downsample_norm", "frame_proj", "frame_head_recompute", "frame_replay"):
            if key in o:
                kw[key] = _bool(o, key, ctx)
        if "downsample_channels" in o:
            v = o["downsample_channels"]
            if not isinstance(v, list) or not all(_is_uint(c) and c > 0 for c in v):
                raise ConfigError("'downsample_channels' must be a list of positive integers.")
            if len(v) != kw["downsample_blocks"]:
                raise ConfigError("'downsample_channels' needs one entry per downsample block.")
            kw["downsample_channels"] = tuple(int(c) for c in v)
        cfg = FbamModelConfiguration(**kw)
        if cfg.downsample_conv_stride not in (1, 2):
            raise ConfigError("'downsample_conv_stride' must be 1 or 2.")
        if cfg.lstm_layers < 1:
            raise ConfigError("'lstm_layers' must be at least 1.")
        return cfg

    # resolved views of the optional keys ------------------------------------------------
    @property
    def embed_dim(self) -> int:
        return self.cell_embed_dim or self.n_embed

    @property
    def hidden(self) -> int:
        return self.lstm_hidden or self.n_embed

    @property
    def heads_action(self) -> int:
        return self.action_heads or self.n_head

    @property
    def mlp_dim(self) -> int:
        return self.action_mlp_dim or 4 * self.n_embed

    def block_channels(self):
        """(in, out) channel pairs of the downsample convolutions (geglu doubles the conv output)."""
        outs = list(self.downsample_channels) or [self.embed_dim] * self.downsample_blocks
        pairs, cin = [], self.embed_dim
        for c in outs:
            pairs.append((cin, c))
            cin = c
        return pairs

    @property
    def frame_feature_dim(self) -> int:
        pairs = self.block_channels()
        return pairs[-1][1] if pairs else self.embed_dim


@dataclass
class OptimizerConfiguration:
    type: str
    learning_rate: float
    weight_decay: float
    beta1: float
    beta2: float
    eps: float
    momentum: float
    nesterov: bool

    @staticmethod
    def from_json(o: Dict[str, Any]) -> "OptimizerConfiguration":
        ctx = "optimizer configuration"
        t = _str(o, "type", ctx)
        if t not in ("sgd", "adamw", "muon"):
            raise ConfigError(f"Unsupported optimizer type '{t}' (expected sgd, adamw or muon).")
        return OptimizerConfiguration(t, _num(o, "learning_rate", ctx), _num(o, "weight_decay", ctx),
                                      _num(o, "beta1", ctx), _num(o, "beta2", ctx), _num(o, "eps", ctx),
                                      _num(o, "momentum", ctx), _bool(o, "nesterov", ctx))


@dataclass
class CheckpointingConfiguration:
    checkpoint_interval: int
    checkpoint_directory: str
    resume_behavior: str = "load_latest"
    dataset_cursor_path: str = ""
    background_write: bool = False       # addition: write checkpoint files on a worker thread (see checkpoint.py)

    @staticmethod
    def from_json(o: Dict[str, Any]) -> "CheckpointingConfiguration":
        ctx = "checkpointing configuration"
        interval = _uint(o, "checkpoint_interval", ctx)
        if interval == 0:
            raise ConfigError("'checkpoint_interval' must be greater than zero.")
        directory = _str(o, "checkpoint_directory", ctx, non_empty=True)
        raw = _str(o, "resume_behavior", ctx, non_empty=True)
        if raw not in _RESUME:
            raise ConfigError(f"Unsupported resume_behavior '{raw}' (expected load_latest, none or disabled).")
        cursor = ""
        if "dataset_cursor_path" in o:
            cursor = _str(o, "dataset_cursor_path", ctx)
        background = _bool(o, "background_write", ctx) if "background_write" in o else False
        return CheckpointingConfiguration(interval, directory, _RESUME[raw], cursor, background)


@dataclass
class RunConfiguration:
    micro_batch_size: int
    total_batch_size: int
    train_sequence_length: int
    validation_sequence_length: int
    max_training_steps: int
    frame_rows: int
    frame_cols: int
    tokenizer_file_path: str
    train_data_config: DatasetConfiguration
    validation_data_config: DatasetConfiguration
    optimizer_config: OptimizerConfiguration
    checkpointing: CheckpointingConfiguration
    model_config: FbamModelConfiguration
    validation_interval: int = 0
    enable_validation: bool = True

    @staticmethod
    def from_json(o: Dict[str, Any]) -> "RunConfiguration":
        ctx = "run configuration"
        train = _obj(o, "train_data_config", ctx)
        val = _obj(o, "validation_data_config", ctx)
        model = _obj(o, "model_config", ctx)
        micro = _uint(o, "micro_batch_size", ctx)
        total = _uint(o, "total_batch_size", ctx)
        tsl = _uint(o, "train_sequence_length", ctx)
        vsl = _uint(o, "validation_sequence_length", ctx)
        vint = _opt_uint(o, "validation_interval", ctx, 0)
        ev = _bool(o, "enable_validation", ctx) if "enable_validation" in o else True
        steps = _uint(o, "max_training_steps", ctx)
        rows = _uint(o, "frame_rows", ctx)
        cols = _uint(o, "frame_cols", ctx)
        tok = _str(o, "tokenizer_file_path", ctx)
        opt = _obj(o, "optimizer", ctx)
        ckpt = _obj(o, "checkpointing", ctx)
        if total <= 0:
            raise ConfigError("'total_batch_size' must be greater than zero.")
        if micro <= 0 or total % micro != 0:
            raise ConfigError("'total_batch_size' must be a multiple of 'micro_batch_size'.")
        return RunConfiguration(
            micro_batch_size=micro, total_batch_size=total, train_sequence_length=tsl,
            validation_sequence_length=vsl, max_training_steps=steps, frame_rows=rows, frame_cols=cols,
            tokenizer_file_path=tok, train_data_config=DatasetConfiguration.from_json(train),
            validation_data_config=DatasetConfiguration.from_json(val),
            optimizer_config=OptimizerConfiguration.from_json(opt),
            checkpointing=CheckpointingConfiguration.from_json(ckpt),
            model_config=FbamModelConfiguration.from_json(model),
            validation_interval=vint, enable_validation=ev)

    @staticmethod
    def from_json_file(path: str) -> Optional["RunConfiguration"]:
        """Returns None when the file does not exist (reference: src/config.cpp:525-550)."""
        if not os.path.exists(path):
            return None
        with open(path, "r", encoding="utf-8") as f:
            return RunConfiguration.from_json(json.load(f))

    @property
    def grad_accum_steps(self) -> int:
        return self.total_batch_size // self.micro_batch_size

    def jsonstr(self) -> str:
        d = asdict(self)
        d["optimizer"] = d.pop("optimizer_config")
        return json.dumps(d, indent=4)


@dataclass
class ParallelEndpointConfiguration:
    ip: str
    port: int

    @staticmethod
    def from_json(o: Dict[str, Any], ctx: str) -> "ParallelEndpointConfiguration":
        ip = _str(o, "ip", ctx, non_empty=True)
        port = _uint(o, "port", ctx)
        if not 0 < port < 65536:
            raise ConfigError(f"'port' must be in 1..65535 in {ctx} JSON.")
        return ParallelEndpointConfiguration(ip, port)


@dataclass
class FrameHeadParallelConfiguration:
    use_frame_head_parallel: bool = False
    transport: str = "ccl"
    ccl_rendezvous: Optional[ParallelEndpointConfiguration] = None

    @staticmethod
    def from_json(o: Dict[str, Any]) -> "FrameHeadParallelConfiguration":
        ctx = "frame_head_parallel configuration"
        use = _bool(o, "use_frame_head_parallel", ctx)
        transport = _str(o, "transport", ctx)
        if transport != "ccl":
            raise ConfigError('frame_head_parallel.transport must be "ccl".')
        rdv = _obj(o, "ccl_rendezvous", ctx)
        if "ftccl_master" in o:
            raise ConfigError("'ftccl_master' is illegal in frame_head_parallel when transport is \"ccl\".")
        return FrameHeadParallelConfiguration(
            use, transport, ParallelEndpointConfiguration.from_json(rdv, "frame_head_parallel.ccl_rendezvous"))


@dataclass
class DdpParallelConfiguration:
    use_ddp_parallel: bool = False
    transport: str = ""
    ccl_rendezvous: Optional[ParallelEndpointConfiguration] = None
    ftccl_master: Optional[ParallelEndpointConfiguration] = None
    # additions: how gradients are reduced on the "ccl" transport
    #   "allreduce" = replicated optimizer (reference), "zero1" = NCCL reduce-scatter/all-gather,
    #   "fused" = peer-memory reduce-scatter + sharded AdamW + all-gather kernels
    grad_reduce: str = "allreduce"

    @staticmethod
    def from_json(o: Dict[str, Any]) -> "DdpParallelConfiguration":
        ctx = "ddp_parallel configuration"
        use = _bool(o, "use_ddp_parallel", ctx)
        if not use:
            for k in ("transport", "ccl_rendezvous", "ftccl_master"):
                if k in o:
                    raise ConfigError(f"'{k}' is illegal in ddp_parallel when use_ddp_parallel is false.")
            return DdpParallelConfiguration(False)
        transport = _str(o, "transport", ctx)
        if transport not in ("ccl", "ftccl"):
            raise ConfigError('ddp_parallel.transport must be "ccl" or "ftccl".')
        ccl = ft = None
        if transport == "ccl":
            rdv = _obj(o, "ccl_rendezvous", ctx)
            if "ftccl_master" in o:
                raise ConfigError("'ftccl_master' is illegal in ddp_parallel when transport is \"ccl\".")
            ccl = ParallelEndpointConfiguration.from_json(rdv, "ddp_parallel.ccl_rendezvous")
        else:
            m = _obj(o, "ftccl_master", ctx)
            if "ccl_rendezvous" in o:
                raise ConfigError("'ccl_rendezvous' is illegal in ddp_parallel when transport is \"ftccl\".")
            ft = ParallelEndpointConfiguration.from_json(m, "ddp_parallel.ftccl_master")
        mode = "allreduce"
        if "grad_reduce" in o:
            mode = _str(o, "grad_reduce", ctx)
            if mode not in ("allreduce", "zero1", "fused"):
                raise ConfigError('ddp_parallel.grad_reduce must be "allreduce", "zero1" or "fused".')
        return DdpParallelConfiguration(True, transport, ccl, ft, mode)


@dataclass
class ParallelConfiguration:
    frame_head_parallel: FrameHeadParallelConfiguration = field(default_factory=FrameHeadParallelConfiguration)
    ddp_parallel: DdpParallelConfiguration = field(default_factory=DdpParallelConfiguration)
    # additions: pipeline (frame head -> action model) and tensor parallel degrees
    pipeline_stages: int = 1
    tensor_parallel: int = 1

    @staticmethod
    def from_json(o: Dict[str, Any]) -> "ParallelConfiguration":
        ctx = "parallel configuration"
        fh = _obj(o, "frame_head_parallel", ctx)
        ddp = _obj(o, "ddp_parallel", ctx)
        cfg = ParallelConfiguration(FrameHeadParallelConfiguration.from_json(fh),
                                    DdpParallelConfiguration.from_json(ddp))
        cfg.pipeline_stages = _opt_uint(o, "pipeline_stages", ctx, 1)
        cfg.tensor_parallel = _opt_uint(o, "tensor_parallel", ctx, 1)
        if cfg.pipeline_stages not in (1, 2):
            raise ConfigError("'pipeline_stages' must be 1 or 2.")
        if cfg.tensor_parallel < 1:
            raise ConfigError("'tensor_parallel' must be at least 1.")
        return cfg

    @staticmethod
    def from_json_file(path: str) -> Optional["ParallelConfiguration"]:
        if not os.path.exists(path):
            return None
        with open(path, "r", encoding="utf-8") as f:
            return ParallelConfiguration.from_json(json.load(f))
