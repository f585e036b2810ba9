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
    def __init__(self, trainer=None, warmup_steps: int = 2):
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
