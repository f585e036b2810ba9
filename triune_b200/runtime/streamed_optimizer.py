"""Tiered optimizer (AdamW / Muon / CentroidSteer) for streamed layers.

Parity: the reference steps a streamed model layer by layer, moving one layer's optimizer state to the GPU, calling
``optimizer.step_parameters(layer_params, is_global_step_end)`` and moving the state back
(``triune/runtime/streaming.py:1080-1201``, ``_move_param_states_to_device`` / ``_move_param_states_to_cpu``).

Here the device holds ONE optimizer arena per *layer signature* (the names, shapes and dtypes of a layer's
parameters), built over a scratch copy of such a layer. Every streamed layer with that signature owns a *state set* in
pinned host memory: the fp32 master weights in arena order and the flat moment / momentum buffers, plus the
CentroidSteer tier's per-matrix dictionaries. Updating layer i is: copy its state set, weights and gradient into the
arena (a handful of large ``cudaMemcpyAsync`` calls, not one per tensor), run the same kernels a resident model would
run through ``step_parameters``, copy the results back. All layers of one global step share the step number, the
refresh schedule and the clip coefficient computed over the whole model beforehand.
"""

from __future__ import annotations

import copy
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

_FLAT_KEYS = ("exp_avg", "exp_avg_sq", "muon_mom")


def layer_signature(layer: nn.Module) -> Tuple:
    return tuple((n, tuple(p.shape), str(p.dtype)) for n, p in layer.named_parameters())


class _Group:
    """One device arena (optimizer over a scratch layer) shared by every layer of one signature."""

    def __init__(self, scratch: nn.Module, optimizer):
        self.scratch, self.opt = scratch, optimizer
        self.layers: List[int] = []
        # arena segment -> parameter name inside the layer
        self.seg_names = [s.name for s in optimizer.arena.segments]


class StreamedLayerOptimizer:
    def __init__(self, engine, make_optimizer: Optional[Callable[[nn.Module], torch.optim.Optimizer]] = None,
                 state_dtype: torch.dtype = torch.float32, **optimizer_kwargs):
        """``make_optimizer(scratch_layer)`` builds the device optimizer (default: ``CentroidSteerOptimizer`` with
        ``optimizer_kwargs`` and no clipping of its own: the engine clips over the whole model). ``state_dtype`` is the
        host format of the moment / momentum buffers (bf16 halves their PCIe traffic; master weights stay fp32)."""
        self.engine = engine
        self.state_dtype = state_dtype
        if make_optimizer is None:
            from ..optim import CentroidSteerOptimizer

            optimizer_kwargs.setdefault("grad_clip", None)
            make_optimizer = lambda m: CentroidSteerOptimizer(m, **optimizer_kwargs)
        self._make = make_optimizer
        self.groups: Dict[Tuple, _Group] = {}
        self.state: Dict[int, Dict] = {}
        self._layer_group: Dict[int, _Group] = {}
        for i in sorted(engine.stores):
            layer = engine.layers[i]
            sig = layer_signature(layer)
            grp = self.groups.get(sig)
            if grp is None:
                grp = self.groups[sig] = self._new_group(layer)
            grp.layers.append(i)
            self._layer_group[i] = grp

    def _new_group(self, layer: nn.Module) -> _Group:
        fwd = layer.__dict__.pop("forward", None)  # the engine's wrapper closes over the engine: not part of the copy
        try:
            scratch = copy.deepcopy(layer)
        finally:
            if fwd is not None:
                layer.__dict__["forward"] = fwd
        scratch.to(self.engine.device)
        for p in scratch.parameters():
            p.grad = None
        return _Group(scratch, self._make(scratch))

    # ------------------------------------------------------------------ host state sets
    def _pinned(self, n: int, dtype) -> torch.Tensor:
        t = torch.zeros(n, dtype=dtype)
        return t.pin_memory() if self.engine._pin else t

    def _new_state(self, i: int, grp: _Group) -> Dict:
        opt = grp.opt
        st = {k: self._pinned(getattr(opt, k).numel(), self.state_dtype) for k in _FLAT_KEYS}
        st["master"] = self._pinned(opt.arena.total, torch.float32)
        st["steer"] = {}
        st["fresh"] = True  # the master copy is taken from the layer's weights at the first update
        return st

    def state_bytes(self) -> int:
        return sum(sum(v.numel() * v.element_size() for v in st.values() if torch.is_tensor(v)) for st in self.state.values())

    # ------------------------------------------------------------------ one layer
    @torch.no_grad()
    def step_layer(self, i: int, grad_dev: torch.Tensor, coef, is_global_step_end: bool) -> None:
        """Update streamed layer ``i`` from its flat fp32 gradient on the device (layer-store layout)."""
        eng = self.engine
        store = eng.stores[i]
        grp = self._layer_group[i]
        opt, arena = grp.opt, grp.opt.arena
        st = self.state.get(i)
        if st is None:
            st = self.state[i] = self._new_state(i, grp)
        dev = eng.device
        nb = lambda t: t.numel() * t.element_size()
        by_name = {n: sl for (n, _), sl in zip(store.layer.named_parameters(), store.slices)}
        w_dev = store.host.to(dev, non_blocking=True)
        eng.telemetry["h2d_bytes"] += nb(store.host)
        # weights, gradient -> arena order
        for seg in arena.segments:
            off, n, _ = by_name[seg.name]
            arena.flat_param[seg.offset : seg.offset + n].copy_(w_dev[off : off + n])
            arena.flat_grad[seg.offset : seg.offset + n].copy_(grad_dev[off : off + n])
        # state set -> device
        if st["fresh"]:
            if arena.flat_master is not None:
                arena.flat_master.copy_(arena.flat_param)
            for k in _FLAT_KEYS:
                getattr(opt, k).zero_()
            opt.steer_state = {}
            st["fresh"] = False
        else:
            if arena.flat_master is not None:
                arena.flat_master.copy_(st["master"], non_blocking=True)
                eng.telemetry["h2d_bytes"] += nb(st["master"])
            else:
                arena.flat_param.copy_(st["master"], non_blocking=True)
                eng.telemetry["h2d_bytes"] += nb(st["master"])
            for k in _FLAT_KEYS:
                getattr(opt, k).copy_(st[k], non_blocking=True)
                eng.telemetry["h2d_bytes"] += nb(st[k])
            opt.steer_state = {k: {kk: (vv.to(dev, non_blocking=True) if torch.is_tensor(vv) else vv) for kk, vv in v.items()}
                               for k, v in st["steer"].items()}
        if hasattr(opt, "_q16"):
            opt._q16.clear()  # bf16 copies of another layer's bases
        # the steer tier reads routing statistics from the module it was built over
        for (_, b_real), (_, b_scr) in zip(store.layer.named_buffers(), grp.scratch.named_buffers()):
            b_scr.copy_(b_real.to(dev, non_blocking=True))
        opt.set_clip_coefficient(coef)
        opt.step_parameters([s.param for s in arena.segments], is_global_step_end=is_global_step_end)
        # results -> host
        master = arena.master()
        st["master"].copy_(master if master.dtype == torch.float32 else master.float(), non_blocking=True)
        eng.telemetry["d2h_bytes"] += nb(st["master"])
        for k in _FLAT_KEYS:
            st[k].copy_(getattr(opt, k), non_blocking=True)
            eng.telemetry["d2h_bytes"] += nb(st[k])
        st["steer"] = {k: {kk: (vv.to("cpu") if torch.is_tensor(vv) else vv) for kk, vv in v.items()}
                       for k, v in opt.steer_state.items()}
        out = torch.zeros_like(w_dev)
        for seg in arena.segments:
            off, n, _ = by_name[seg.name]
            out[off : off + n].copy_(arena.flat_param[seg.offset : seg.offset + n])
        store.host.copy_(out, non_blocking=True)
        eng.telemetry["d2h_bytes"] += nb(store.host)
        arena.flat_grad.zero_()

    # ------------------------------------------------------------------ whole pass
    def last_layer(self) -> Optional[int]:
        ids = [i for g in self.groups.values() for i in g.layers]
        return max(ids) if ids else None

    def group_of(self, i: int) -> _Group:
        return self._layer_group[i]

    def set_lr(self, lr: float) -> None:
        for g in self.groups.values():
            if hasattr(g.opt, "set_lr"):
                g.opt.set_lr(lr)
            else:
                for pg in g.opt.param_groups:
                    pg["lr"] = lr

    def state_dict(self) -> Dict:
        return {"layers": {i: {k: (v.clone() if torch.is_tensor(v) else copy.deepcopy(v)) for k, v in st.items()}
                           for i, st in self.state.items()},
                "step_counts": [g.opt.step_count for g in self.groups.values()]}

    def load_state_dict(self, sd: Dict) -> None:
        for i, st in sd["layers"].items():
            i = int(i)
            cur = self.state.get(i) or self._new_state(i, self._layer_group[i])
            for k, v in st.items():
                if torch.is_tensor(v):
                    cur[k].copy_(v)
                else:
                    cur[k] = copy.deepcopy(v)
            self.state[i] = cur
        for g, n in zip(self.groups.values(), sd["step_counts"]):
            g.opt.step_count = int(n)
