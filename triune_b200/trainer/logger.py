"""Experiment loggers (reference: ``triune/trainer/logger.py``): ``NullLogger``, ``WandbLogger`` and a JSON-lines
logger that needs no service, which is what a machine without network access can use."""

from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Optional


class NullLogger:
    run_id = None

    def log(self, values: dict, *, step: int) -> None:
        return None

    def finish(self) -> None:
        return None


class JsonlLogger:
    def __init__(self, path, run_id: Optional[str] = None, config: Optional[dict] = None):
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.run_id = run_id or time.strftime("run-%Y%m%d-%H%M%S")
        self._f = open(self.path, "a", encoding="utf-8")
        if config is not None:
            self._f.write(json.dumps({"run_id": self.run_id, "config": {k: v for k, v in config.items()
                                                                        if isinstance(v, (int, float, str, bool, type(None)))}}) + "\n")

    def log(self, values: dict, *, step: int) -> None:
        rec = {"step": int(step), "time": time.time()}
        rec.update({k: (float(v) if hasattr(v, "__float__") else v) for k, v in values.items()})
        self._f.write(json.dumps(rec) + "\n")
        self._f.flush()

    def finish(self) -> None:
        self._f.close()


class WandbLogger:
    def __init__(self, *, project: str, config: dict, run_id: Optional[str] = None):
        try:
            import wandb
        except ImportError as e:
            raise RuntimeError("wandb is not installed; pass --no-wandb to disable experiment logging") from e
        self._wandb = wandb
        self._run = wandb.init(project=project, config=config, id=run_id, resume="allow" if run_id else None)

    @property
    def run_id(self):
        return self._run.id

    def log(self, values: dict, *, step: int) -> None:
        self._wandb.log(values, step=step)

    def finish(self) -> None:
        self._wandb.finish()
