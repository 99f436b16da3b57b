"""``create_optimizer``: optimizer-configuration block → optimizer instance
(reference: ``include/optimizers.h:53-56``, ``src/optimizers.cpp:1516-1559``).  ``type: "muon"`` builds
Muon for matrices with an auxiliary AdamW for everything else."""
from __future__ import annotations

from typing import Callable, Iterable, Optional, Tuple

import torch

from ..config import OptimizerConfiguration
from .adamw import AdamwOptimizer
from .base import Optimizer
from .muon import MuonWithAuxAdam
from .sgd import SgdOptimizer


def create_optimizer(cfg: OptimizerConfiguration, named_params: Iterable[Tuple[str, torch.nn.Parameter]],
                     prefix: str, adam_names: Optional[Callable[[str], bool]] = None) -> Optimizer:
    if cfg.type == "sgd":
        return SgdOptimizer(named_params, prefix, cfg.learning_rate, cfg.momentum, cfg.nesterov, cfg.weight_decay)
    if cfg.type == "adamw":
        return AdamwOptimizer(named_params, prefix, cfg.learning_rate, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay)
    if cfg.type == "muon":
        return MuonWithAuxAdam(named_params, prefix, cfg.learning_rate, cfg.momentum, cfg.nesterov, cfg.weight_decay,
                               cfg.beta1, cfg.beta2, cfg.eps, adam_names)
    raise ValueError(f"Unsupported optimizer type '{cfg.type}'")
