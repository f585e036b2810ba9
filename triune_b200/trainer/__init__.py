"""Training: step engine, trainer, scheduler, checkpoints, evaluation."""

from ..parallel.dist import all_reduce_dict, all_reduce_tensor, cleanup_distributed, setup_distributed
from .checkpoint import load_checkpoint, save_best, save_checkpoint, save_latest
from .engine import TrainingEngine
from .evaluation import forward_causal_lm, run_eval, run_sample
from .scheduler import lr_schedule, set_optimizer_lr
from .trainer import ConsoleLogger, NullLogger, Trainer

__all__ = [
    "all_reduce_dict", "all_reduce_tensor", "cleanup_distributed", "setup_distributed", "load_checkpoint",
    "save_best", "save_checkpoint", "save_latest", "TrainingEngine", "forward_causal_lm", "run_eval", "run_sample",
    "lr_schedule", "set_optimizer_lr", "ConsoleLogger", "NullLogger", "Trainer",
]
