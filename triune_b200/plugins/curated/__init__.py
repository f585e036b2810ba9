"""Modules that ship with the framework and install without a network: ``custom_loss_nodes`` (three graph nodes) and
``code_assistant_lora`` (a LoRA configuration preset in PEFT layout). ``CURATED`` is the catalogue the module manager
lists; ``builtin://<id>`` names an entry as an installation source (``triune/modules/curated`` of the reference)."""

from __future__ import annotations

from pathlib import Path
from typing import Any, Dict, List

ROOT = Path(__file__).resolve().parent
CURATED: List[Dict[str, Any]] = [
    {"id": "custom_loss_nodes", "name": "Custom loss nodes", "type": "plugin", "download_url": "builtin://custom_loss_nodes",
     "description": "Focal cross-entropy, an expert-load balance penalty and a router temperature annealer as graph nodes.",
     "nodes": ["FocalCrossEntropyLoss", "CentroidBalanceLoss", "TemperatureAnnealer"]},
    {"id": "code_assistant_lora", "name": "Code assistant LoRA preset", "type": "adapter", "download_url": "builtin://code_assistant_lora",
     "description": "Rank-16 LoRA on the query, value and output projections (PEFT adapter_config.json) for code fine-tuning."},
]


def curated_path(module_id: str) -> Path:
    """Directory of a curated module; ``-`` and ``_`` are interchangeable in the id. Raises ``KeyError`` when unknown."""
    for cand in (module_id, module_id.replace("-", "_")):
        if any(c["id"] == cand for c in CURATED) and (ROOT / cand).is_dir():
            return ROOT / cand
    raise KeyError(module_id)
