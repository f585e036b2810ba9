"""CUDA-graph capture and replay of whole training steps and of inference calls.

Parity: ``CUDAGraphEngine`` (``triune/runtime/cuda_graph.py:19-216``): captures the full train step
(forward + backward + optimizer, in-place ``zero_grad``) or an inference function, replays it when the input
shapes match and falls back to eager execution otherwise.

A captured step is frozen control flow, so everything that changes between steps lives in device memory: the
batch (static input buffers), the learning rates and bias corrections (``optimizer.hyper``), the MoE step
counter. The CentroidSteer tier has three kinds of step (``optimizer.step_kind()``): ``refresh`` steps rebuild
the subspace bases with host-side decisions and always run eagerly; ``steer`` and ``plain`` steps each get
their own graph, captured the first time that kind occurs.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Tuple

import torch

from .. import ops
from ..profiling import nvtx_range


class CUDAGraphEngine:
    def __init__(self, trainer=None, warmup_steps: int = 2, device=None):
        if isinstance(trainer, (str, torch.device)):  # the reference's constructor takes the device first
            trainer, device = None, trainer
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        # state of the generic capture below (one training or inference step of any model / optimizer pair)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.static_input: Optional[torch.Tensor] = None
        self.static_target: Optional[torch.Tensor] = None
        self.static_loss: Optional[torch.Tensor] = None
        self.static_output: Any = None
        self.is_captured = False
        self.trainer = trainer
        self.graphs: Dict[Tuple, torch.cuda.CUDAGraph] = {}
        self.outputs: Dict[Tuple, Any] = {}
        self.launches: Dict[Tuple, int] = {}
        self.static_inputs: Dict[Tuple, Tuple[torch.Tensor, ...]] = {}
        self.pool = None
        self.warmup_steps = warmup_steps
        self.eager_steps = 0
        self.replays = 0
        self.captures = 0
        self.enabled = torch.cuda.is_available()
        # Eager steps and captures share ONE side stream: autograd nodes that outlive a step (gradient accumulators
        # kept alive by a retained graph) remember the stream they were created on, and a capture that has to wait
        # for work on any other, uncaptured stream is invalid.
        self.stream = torch.cuda.Stream() if self.enabled else None

    # ------------------------------------------------------------------ generic capture (any model / optimizer pair)
    # The method names and arguments of the reference's engine (``triune/runtime/cuda_graph.py:31-230``). Capture needs a
    # CUDA device; without one ``capture_*`` return False and ``step`` / ``inference_step`` run the fallback.
    def invalidate(self) -> None:
        self.graph = self.static_input = self.static_target = self.static_loss = self.static_output = None
        self.is_captured = False

    @staticmethod
    def _same(a: Optional[torch.Tensor], b: Optional[torch.Tensor]) -> bool:
        return a is not None and b is not None and a.shape == b.shape and a.dtype == b.dtype and a.device == b.device

    def can_replay(self, input_tokens: torch.Tensor, target_tokens: Optional[torch.Tensor] = None) -> bool:
        if not self.is_captured or self.graph is None or not self._same(input_tokens, self.static_input):
            return False
        return target_tokens is None or self.static_target is None or self._same(target_tokens, self.static_target)

    def _run_step(self, model, optimizer, loss_fn, step_fn):
        if step_fn is not None:
            return step_fn(model, optimizer, self.static_input, self.static_target)
        optimizer.zero_grad(set_to_none=False)  # gradients keep their storage: the graph replays in place
        out = model(self.static_input)
        if loss_fn is not None:
            loss = loss_fn(out, self.static_target)
        else:
            loss = (out[0] if isinstance(out, tuple) else out).sum()
        loss.backward()
        optimizer.step()
        return loss

    def capture_training_step(self, model, optimizer, sample_input: torch.Tensor, sample_target: torch.Tensor, loss_fn: Optional[Callable] = None,
                              step_fn: Optional[Callable] = None, warmup_steps: int = 3) -> bool:
        """Forward, backward and optimizer update of one batch shape in one graph; False (nothing captured) when that is
        not possible here."""
        if not torch.cuda.is_available() or self.device.type != "cuda":
            return False
        try:
            for group in getattr(optimizer, "param_groups", []):
                if "capturable" in group:
                    group["capturable"] = True
            self.static_input, self.static_target = sample_input.clone().to(self.device), sample_target.clone().to(self.device)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):  # warm-up on the capture stream: lazily created optimizer state exists afterwards
                for _ in range(max(1, int(warmup_steps))):
                    self._run_step(model, optimizer, loss_fn, step_fn)
            torch.cuda.current_stream(self.device).wait_stream(side)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self.static_loss = self._run_step(model, optimizer, loss_fn, step_fn)
            self.is_captured = True
            return True
        except Exception:
            self.invalidate()
            return False

    def step(self, input_tokens: torch.Tensor, target_tokens: Optional[torch.Tensor] = None, sync: bool = False, fallback_fn: Optional[Callable] = None):
        """Replay with a new batch; the loss stays on the device unless ``sync``. A batch of another shape goes to
        ``fallback_fn(input, target)``."""
        if not self.can_replay(input_tokens, target_tokens):
            if fallback_fn is None:
                raise RuntimeError("CUDA Graph cannot replay with mismatched tensor shapes without a fallback.")
            res = fallback_fn(input_tokens, target_tokens)
            if sync:
                return float(res.item()) if isinstance(res, torch.Tensor) else float(res)
            return res if isinstance(res, torch.Tensor) else torch.tensor(res, device=self.device)
        self.static_input.copy_(input_tokens, non_blocking=True)
        if self.static_target is not None and target_tokens is not None:
            self.static_target.copy_(target_tokens, non_blocking=True)
        self.graph.replay()
        if sync:
            return self.current_loss_item()
        return self.static_loss

    def current_loss_item(self) -> float:
        return float(self.static_loss.item()) if self.static_loss is not None else 0.0

    def capture_inference_step(self, model, sample_input: torch.Tensor, warmup_steps: int = 3) -> bool:
        if not torch.cuda.is_available() or self.device.type != "cuda":
            return False
        try:
            self.static_input = sample_input.clone().to(self.device)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side), torch.no_grad():
                for _ in range(max(1, int(warmup_steps))):
                    model(self.static_input)
            torch.cuda.current_stream(self.device).wait_stream(side)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side), torch.no_grad():
                self.static_output = model(self.static_input)
            self.is_captured = True
            return True
        except Exception:
            self.invalidate()
            return False

    def inference_step(self, input_tokens: torch.Tensor, fallback_fn: Optional[Callable] = None):
        if not self.can_replay(input_tokens):
            if fallback_fn is None:
                raise RuntimeError("CUDA Graph cannot replay with mismatched tensor shapes without a fallback.")
            return fallback_fn(input_tokens)
        self.static_input.copy_(input_tokens, non_blocking=True)
        self.graph.replay()
        return self.static_output

    # ------------------------------------------------------------------ training
    def _body(self, x, y, n_valid):
        tr = self.trainer
        eng = tr.engine
        eng.model.train()
        with nvtx_range("forward"):
            loss, _ = eng._micro_loss(x, y, n_valid)
        with nvtx_range("backward"):
            loss.backward()
        with nvtx_range("optimizer"):
            tr.optimizer.step()
            tr.optimizer.zero_grad(set_to_none=True)
        for m in eng._moe:
            m.step_bias()
        return loss.detach()

    def _prepare_host_state(self):
        """Everything the step reads from the host is pushed to the device before the launch."""
        tr = self.trainer
        eng = tr.engine
        lr = tr.lr_schedule(tr.config, eng.step)
        tr.set_optimizer_lr(tr.optimizer, lr)
        opt = tr.optimizer
        opt.grad_clip = tr.config.get("grad_clip", 1.0)
        opt.write_hyper()
        for m in eng._moe:
            m._global_step.fill_(eng.step)
        return lr

    def train_step(self, x: torch.Tensor, y: torch.Tensor, n_valid: Optional[int] = None):
        """One optimizer step on device tensors x, y. Returns the (device) loss tensor."""
        tr = self.trainer
        eng = tr.engine
        opt = tr.optimizer
        if n_valid is None:
            n_valid = int(y.numel())
        kind = opt.step_kind() if hasattr(opt, "step_kind") else "eager"
        capturable = (self.enabled and hasattr(opt, "write_hyper") and kind in ("plain", "steer")
                      and self.eager_steps >= self.warmup_steps and tr.config.get("depth_mode", "cortex") == "cortex"
                      and int(tr.config.get("grad_accum_steps", 1)) == 1 and eng.streaming_engine is None)
        if not capturable:
            if hasattr(opt, "capturable"):
                opt.capturable = False
            tr._pending = (x, y, n_valid)
            if self.stream is not None:
                cur = torch.cuda.current_stream()
                self.stream.wait_stream(cur)
                with torch.cuda.stream(self.stream):
                    out = eng.step_once()
                cur.wait_stream(self.stream)
            else:
                out = eng.step_once()
            self.eager_steps += 1
            return out["loss"]
        key = (kind, tuple(x.shape), int(n_valid))
        opt.capturable = True
        self._prepare_host_state()
        if key not in self.graphs:
            sx, sy = x.clone(), y.clone()
            self.static_inputs[key] = (sx, sy)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(g, pool=self.pool, stream=self.stream):
                loss = self._body(sx, sy, n_valid)
            if self.pool is None:
                self.pool = g.pool()
            self.graphs[key], self.outputs[key] = g, loss
            self.launches[key] = ops.launch_count() - before
            self.captures += 1
            g.replay()  # capture only records; this runs the step whose host bookkeeping just happened
            eng.step += 1
            self.replays += 1
            return self.outputs[key]
        sx, sy = self.static_inputs[key]
        sx.copy_(x, non_blocking=True)
        sy.copy_(y, non_blocking=True)
        self.graphs[key].replay()
        ops._tick(self.launches[key])
        opt.advance_counters(kind)
        eng.step += 1
        self.replays += 1
        return self.outputs[key]

    # ------------------------------------------------------------------ inference
    def capture_inference(self, fn: Callable, *example_inputs: torch.Tensor, name: str = "infer"):
        """Capture ``fn(*inputs)`` (no grad). Returns a callable that replays on same-shaped inputs and falls back
        to eager ``fn`` on any other shape."""
        if not self.enabled:
            return fn
        statics = tuple(t.clone() for t in example_inputs)
        with torch.no_grad():
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):
                    fn(*statics)
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self.pool):
                out = fn(*statics)
        if self.pool is None:
            self.pool = g.pool()
        shapes = tuple(tuple(t.shape) for t in statics)

        def run(*inputs):
            if tuple(tuple(t.shape) for t in inputs) != shapes:
                with torch.no_grad():
                    return fn(*inputs)
            for s_, t in zip(statics, inputs):
                s_.copy_(t, non_blocking=True)
            g.replay()
            self.replays += 1
            return out

        self.graphs[(name, shapes)] = g
        return run

    def stats(self) -> Dict[str, int]:
        return {"captures": self.captures, "replays": self.replays, "eager_steps": self.eager_steps,
                "graphs": len(self.graphs)}
