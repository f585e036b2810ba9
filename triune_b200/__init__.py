"""triune_b200: a Blackwell-native (sm_100a) training and serving framework for multi-exit MoE and dense
linear-attention language models."""

__version__ = "0.1.0"

from . import config, ops  # noqa: F401
from .config import ModelConfig, OptimConfig, ParallelConfig, ServeConfig, TrainConfig, build_config, get_model_config
from .models import MoE_FFN, TriuneTransformer


def build_model(cfg):
    """Build a model from a ModelConfig, a preset name, or a flat run-config dict."""
    from .models.factory import build_model as _b

    return _b(cfg)


__all__ = ["config", "ops", "ModelConfig", "OptimConfig", "ParallelConfig", "ServeConfig", "TrainConfig",
           "build_config", "get_model_config", "MoE_FFN", "TriuneTransformer", "build_model", "__version__"]
