"""Model construction from presets / configs (reference: ``triune/model/factory.py:11-39``)."""

from __future__ import annotations

from typing import Any, Dict, Union

from ..config import ModelConfig, get_model_config, model_config_from_flat


def build_model(cfg: Union[ModelConfig, str, Dict[str, Any]]):
    if isinstance(cfg, str):
        cfg = get_model_config(cfg)
    elif isinstance(cfg, dict):
        cfg = model_config_from_flat(cfg)
    if cfg.family == "universal":
        from .universal import UniversalTransformer

        return UniversalTransformer.from_config(cfg)
    from .transformer import TriuneTransformer

    return TriuneTransformer.from_config(cfg)
