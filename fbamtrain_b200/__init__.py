"""fbamtrain_b200 — a Blackwell-native training framework for frame-based action models."""
from .config import ParallelConfiguration, RunConfiguration
from .train import Trainer, run_training

__version__ = "0.1.0"
__all__ = ["ParallelConfiguration", "RunConfiguration", "Trainer", "run_training", "__version__"]
