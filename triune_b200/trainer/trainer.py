"""Trainer: wires model, optimizer, data, checkpoints and the step engine.

Parity: ``Trainer`` (``triune/trainer/trainer.py:20-128``) plus the working data-parallel engine the reference
only sketches (``DistributedTrainingEngine``, ``triune/trainer/distributed.py:159-186``). ``train_step`` is the
call a user makes per optimizer step: it takes a HOST batch (pinned memory preferred), copies it to the device,
runs forward/backward/update and returns the loss as a Python float (device -> host read).
"""

from __future__ import annotations

import contextlib
import os
import signal
from typing import Any, Dict, Iterable, Optional

import torch

from ..data.dataloader import AsyncDevicePrefetcher, CyclingDataLoader
from ..optim.factory import build_optimizer
from . import checkpoint as ckpt
from .engine import TrainingEngine
from .scheduler import lr_schedule, set_optimizer_lr


class NullLogger:
    def log(self, metrics: Dict[str, Any]) -> None:
        pass


class ConsoleLogger(NullLogger):
    def log(self, metrics):
        print(" ".join(f"{k}={v:.5g}" if isinstance(v, float) else f"{k}={v}" for k, v in metrics.items()), flush=True)


class Trainer:
    def __init__(self, model: torch.nn.Module, config: Dict[str, Any], optimizer=None, train_loader: Optional[Iterable] = None,
                 eval_loader: Optional[Iterable] = None, tokenizer=None, device=None, logger=None, dp=None,
                 precision_context=None, sample_prompt: str = "The history of"):
        # ``precision_context`` / ``sample_prompt``: keywords of the reference's constructor. Weights here are kept in their
        # training dtype (bf16 on a GPU), so a context manager factory is only entered around evaluation passes.
        self.precision_context, self.sample_prompt = precision_context, sample_prompt
        self.config = dict(config)
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.model = model
        self.tokenizer = tokenizer
        self.dp = dp  # optional ShardedDataParallel wrapper (gradient reduce-scatter + sharded update)
        self.optimizer = optimizer if optimizer is not None else build_optimizer(model, self.config)
        if dp is not None:
            dp.attach(self.optimizer)
        self.logger = logger or NullLogger()
        self.grad_accum = int(self.config.get("grad_accum_steps", 1))
        self.z_loss_coef = float(self.config.get("z_loss_coef", 1e-3))
        self.vocab_size = int(self.config.get("vocab_size", getattr(model, "vocab_size", 0)))
        self.pad_token_id = getattr(tokenizer, "pad_token_id", None)
        self._loader = None
        if train_loader is not None:
            src = CyclingDataLoader(train_loader)
            self._loader = AsyncDevicePrefetcher(src, self.device) if self.device.type == "cuda" else src
        self.eval_loader = eval_loader
        self._pending = None
        self.engine = TrainingEngine(self)
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._h2d_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.graph_engine = None
        if self.config.get("cuda_graph") and self.device.type == "cuda":
            from ..runtime.cuda_graph import CUDAGraphEngine

            self.graph_engine = CUDAGraphEngine(self)

    # ---- protocol used by TrainingEngine ------------------------------------------------------
    def bf16_autocast(self):
        """Context manager for evaluation passes on models kept in fp32 (``precision_context`` given to the constructor
        wins)."""
        if self.precision_context is not None:
            return self.precision_context()
        from ..recipes import bf16_autocast

        return bf16_autocast(self.device.type)

    def next_batch(self):
        if self._pending is not None:
            b, self._pending = self._pending, None
            return b
        b = next(self._loader)
        return tuple(t.to(self.device) for t in b) if self.device.type != "cuda" or not b[0].is_cuda else b

    def model_autocast(self):
        return contextlib.nullcontext()

    lr_schedule = staticmethod(lr_schedule)
    set_optimizer_lr = staticmethod(set_optimizer_lr)

    def router_loss_fn(self, logits, labels):
        return torch.nn.functional.cross_entropy(logits.float(), labels)

    # ---- public per-step API ------------------------------------------------------------------
    def train_step(self, input_ids: torch.Tensor, labels: torch.Tensor, n_valid: Optional[int] = None) -> float:
        """One optimizer step on a host batch. Returns the loss (host float)."""
        if input_ids.device != self.device:
            nb = self.device.type == "cuda"
            self.h2d_bytes += input_ids.numel() * input_ids.element_size() + labels.numel() * labels.element_size()
            input_ids = input_ids.to(self.device, non_blocking=nb)
            labels = labels.to(self.device, non_blocking=nb)
        if n_valid is None:
            n_valid = int(labels.numel())  # callers with ignored labels pass the exact count
        loss = self.step_on_device(input_ids, labels, n_valid)
        self.d2h_bytes += 4
        return float(loss.item() if torch.is_tensor(loss) else loss)

    def step_on_device(self, input_ids: torch.Tensor, labels: torch.Tensor, n_valid: Optional[int] = None):
        """One optimizer step on device-resident tensors; returns the loss as a device tensor (no host sync)."""
        if n_valid is None:
            n_valid = int(labels.numel())
        if self.graph_engine is not None:
            return self.graph_engine.train_step(input_ids, labels, n_valid)
        self._pending = (input_ids, labels, n_valid)
        return self.engine.step_once()["loss"]

    def fit(self, total_steps: Optional[int] = None):
        self._install_signal_handlers()
        return self.engine.train(total_steps)

    def compile(self):  # API parity: there is no tracing compiler in this framework
        return self

    # ---- evaluation / checkpoints --------------------------------------------------------------
    @torch.no_grad()
    def run_eval(self) -> Optional[float]:
        if self.eval_loader is None:
            return None
        from .evaluation import run_eval

        return run_eval(self.model, self.eval_loader, self.device, int(self.config.get("eval_batches", 5)))

    def run_sample(self, prompt_ids=None, max_new_tokens: int = 16):
        from .evaluation import run_sample

        return run_sample(self.model, prompt_ids, self.device, max_new_tokens)

    def _ckpt_kwargs(self):
        return dict(model=self.model, optimizer=self.optimizer, step=self.engine.step, loss=0.0,
                    best_eval_loss=self.engine.best_eval_loss, config=self.config,
                    depth_usage_ema=self.engine.usage_ema.tolist())

    def save_latest(self):
        return ckpt.save_latest(self.config.get("checkpoint_dir", "checkpoints_full"), **self._ckpt_kwargs())

    def save_best(self):
        return ckpt.save_best(self.config.get("checkpoint_dir", "checkpoints_full"), **self._ckpt_kwargs())

    def resume(self, path: str):
        ck = ckpt.load_checkpoint(path, self.model, self.optimizer, self.config, map_location="cpu")
        self.engine.step = int(ck.get("step", 0))
        self.engine.best_eval_loss = float(ck.get("best_eval_loss", float("inf")))
        if ck.get("depth_usage_ema") is not None:
            self.engine.usage_ema = torch.tensor(ck["depth_usage_ema"], dtype=torch.float32)
        return ck

    def _install_signal_handlers(self):
        def handler(signum, frame):
            try:
                self.save_latest()
            finally:
                raise KeyboardInterrupt

        for sig in (signal.SIGINT, signal.SIGTERM):
            try:
                signal.signal(sig, handler)
            except (ValueError, OSError):
                pass
