"""Optimizers with fp32 master weights: SGD, AdamW, Muon and Muon with auxiliary AdamW."""
from .base import Optimizer
from .sgd import SgdOptimizer
from .adamw import AdamwOptimizer
from .muon import MuonOptimizer, MuonWithAuxAdam, newton_schulz, muon_update
from .factory import create_optimizer

__all__ = ["Optimizer", "SgdOptimizer", "AdamwOptimizer", "MuonOptimizer", "MuonWithAuxAdam", "newton_schulz",
           "muon_update", "create_optimizer"]
