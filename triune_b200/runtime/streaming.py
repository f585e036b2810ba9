"""Layer streaming: train or run models whose layers do not all fit on the GPU.

Parity: ``LayerStreamingEngine`` / ``StreamingConfig`` / ``enable_layer_streaming``
(``triune/runtime/streaming.py:153-1308``) and ``ParameterStager`` (``triune/runtime/staging.py:19-621``).
Layers live in pinned host memory; the root (embedding, heads, norms, router) and ``resident_gpu_layers`` stay on
the GPU. A streamed layer is staged host->device with ``cudaMemcpyAsync`` from pinned memory on a SIDE stream
while the previous layer computes (prefetch of layer i+1 going forward, i-1 going backward), runs under
activation checkpointing (only its input is kept), and is evicted afterwards. Gradients leave device->host on a
third stream with their squared norm captured on the GPU; the optimizer then streams layer by layer: stage
weights + gradients + optimizer state, update, write back.

Design differences from the reference: instead of monkey-patching ``_forward_block`` and autograd hooks, each
streamed layer is wrapped in ONE ``torch.autograd.Function`` that owns stage / compute / evict for both
directions, so exception cleanup is a ``finally`` in one place; staging is per-layer flat buffers (one copy per
layer per direction, not one per tensor).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn


@dataclass
class StreamingConfig:
    enabled: bool = True
    chunk_size: int = 1
    pin_memory: Optional[bool] = None  # None: pin when CUDA is present
    async_prefetch: bool = True
    fp8_weights: bool = False
    grad_clip: float = 1.0
    instant_optimizer: bool = True
    resident_gpu_layers: int = 0
    activation_checkpointing: bool = True
    forward_snapshots: bool = True
    grad_dtype: str = "fp32"  # "bf16": gradients leave the device (and return for the update) in bf16: half the traffic
    layers_path: Optional[str] = None  # dotted path of the layer stack when discovery cannot decide
    fp4_weights: bool = False  # accepted for configuration files of the reference; weights stage as FP8 or in full precision
    capture_forward_snapshots: Optional[bool] = None  # the reference's name of ``forward_snapshots``

    def __post_init__(self):
        if self.capture_forward_snapshots is not None:
            self.forward_snapshots = bool(self.capture_forward_snapshots)
        self.capture_forward_snapshots = self.forward_snapshots


class LayerDiscoveryError(ValueError, AttributeError):
    """No single stack of layers could be named (a ``ValueError`` as in the reference; also an ``AttributeError``, which
    is what a missing dotted path is)."""


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class LayerStore:
    """Flat host storage of one layer: parameters (model dtype), fp32 gradient, and views for each tensor."""

    ALIGN = 64  # elements

    FP8_BLOCK = 128  # elements per scale of the FP8 staging copy

    def __init__(self, layer: nn.Module, pin: bool, grad_dtype: torch.dtype = torch.float32, fp8: bool = False):
        self.layer = layer
        self.params = [p for p in layer.parameters()]
        # Every tensor starts on a 128-byte boundary of the flat buffers (ALIGN elements covers 2- and 4-byte types):
        # the kernels read parameters in 16-byte vectors, and a tensor packed right behind a 3-element bias would
        # otherwise start on an odd address.
        self.numel = sum(_round_up(p.numel(), self.ALIGN) for p in self.params)
        dtype = self.params[0].dtype if self.params else torch.float32
        self.host = torch.zeros(self.numel, dtype=dtype)
        self.host_grad = torch.zeros(self.numel, dtype=grad_dtype)
        if pin:
            self.host, self.host_grad = self.host.pin_memory(), self.host_grad.pin_memory()
        self._pin = pin
        off = 0
        self.slices = []
        for p in self.params:
            n = p.numel()
            self.host[off : off + n].copy_(p.data.reshape(-1))
            p.data = self.host[off : off + n].view(p.shape)  # the host copy is the master
            self.slices.append((off, n, p.shape))
            off += _round_up(n, self.ALIGN)
        self.device_buf: Optional[torch.Tensor] = None
        self.ready: Optional[torch.cuda.Event] = None
        self.grad_sumsq = None
        # FP8 staging (``StreamingConfig.fp8_weights``): the forward and backward passes receive an E4M3 copy with one
        # fp32 scale per 128 elements (1.03 bytes per weight over PCIe instead of 2) and expand it on the device; tensors
        # with fewer than two dimensions (norm weights, biases) travel beside it unquantised. The master copy in
        # ``host`` is what the optimizer updates; ``refresh_fp8`` re-derives the staging copy afterwards.
        self.fp8 = bool(fp8)
        self.host_q = self.host_scale = self.host_small = None
        self.small_slices = [(off, n) for p, (off, n, _) in zip(self.params, self.slices) if p.dim() < 2]
        if self.fp8:
            self.refresh_fp8()

    def refresh_fp8(self, source: Optional[torch.Tensor] = None) -> None:
        """(Re)build the FP8 staging copy from ``source`` (a flat tensor in this store's layout, any device; default: the
        host master)."""
        B = self.FP8_BLOCK
        src = self.host if source is None else source
        padded = -(-self.numel // B) * B
        w = torch.zeros(padded, dtype=torch.float32, device=src.device)
        w[: self.numel] = src.float()
        blocks = w.view(-1, B)
        scale = (blocks.abs().amax(dim=1) / 448.0).clamp_min(1e-12)
        q = (blocks / scale[:, None]).to(torch.float8_e4m3fn).view(-1)
        small = torch.cat([src[o : o + n] for o, n in self.small_slices]) if self.small_slices else src[:0]
        if self.host_q is None:
            mk = (lambda t: t.pin_memory()) if self._pin else (lambda t: t)
            self.host_q = mk(torch.empty(padded, dtype=torch.float8_e4m3fn))
            self.host_scale = mk(torch.empty(padded // B, dtype=torch.float32))
            self.host_small = mk(torch.empty(small.numel(), dtype=self.host.dtype))
        self.host_q.copy_(q, non_blocking=True)
        self.host_scale.copy_(scale, non_blocking=True)
        self.host_small.copy_(small.to(self.host.dtype), non_blocking=True)

    def fp8_stage_bytes(self) -> int:
        return self.host_q.numel() + self.host_scale.numel() * 4 + self.host_small.numel() * self.host_small.element_size()

    def expand_fp8(self, device) -> torch.Tensor:
        """Copy the FP8 staging set to ``device`` and expand it to this store's flat layout in the model dtype."""
        nb = self.host_q.is_pinned()
        q = self.host_q.to(device, non_blocking=nb)
        sc = self.host_scale.to(device, non_blocking=nb)
        small = self.host_small.to(device, non_blocking=nb)
        buf = (q.float().view(-1, self.FP8_BLOCK) * sc[:, None]).view(-1)[: self.numel].to(self.host.dtype)
        pos = 0
        for o, n in self.small_slices:
            buf[o : o + n] = small[pos : pos + n]
            pos += n
        return buf

    def bind(self, buf: torch.Tensor):
        for p, (off, n, shape) in zip(self.params, self.slices):
            p.data = buf[off : off + n].view(shape)

    def bind_host(self):
        self.bind(self.host)


_LAYER_PATHS = ("layers", "model.layers", "model.decoder.layers", "transformer.h", "transformer.blocks", "gpt_neox.layers",
                "decoder.layers", "encoder.layer", "h", "blocks")


def find_layer_list(model: nn.Module, layers_attr: Optional[str] = None) -> nn.ModuleList:
    """The stack of repeated blocks to stream: ``layers_attr`` (dotted path) when given, else the usual places of this
    framework's models and of Hugging Face causal LMs, else the longest ``nn.ModuleList`` of same-typed modules
    (``triune/runtime/streaming.py:153-260`` of the reference probes the same way)."""
    def walk(path):
        obj = model
        for part in path.split("."):
            obj = getattr(obj, part, None)
            if obj is None:
                return None
        return obj if isinstance(obj, (nn.ModuleList, list, tuple)) and len(obj) > 0 else None

    if layers_attr:
        found = walk(layers_attr)
        if found is None:
            raise LayerDiscoveryError(f"Specified layers_path '{layers_attr}' does not name a non-empty layer list of the model")
        return found
    for path in _LAYER_PATHS:
        found = walk(path)
        if found is not None:
            return found
    stacks = [(n, m) for n, m in model.named_modules()
              if isinstance(m, nn.ModuleList) and len(m) > 1 and len({type(c) for c in m}) == 1]
    if not stacks:
        raise LayerDiscoveryError("no stack of repeated layers found; pass layers_path")
    longest = max(len(m) for _, m in stacks)
    top = [(n, m) for n, m in stacks if len(m) == longest]
    if len(top) > 1:
        raise LayerDiscoveryError(f"Ambiguous layer discovery: {[n for n, _ in top]} all hold {longest} layers; "
                                  "name the stack to stream with layers_path")
    return top[0][1]


class LayerStreamingEngine:
    def __init__(self, model: nn.Module, device, config: Optional[StreamingConfig] = None, layers_attr: Optional[str] = None,
                 optimizer=None, layers_path: Optional[str] = None):
        # ``optimizer`` / ``layers_path``: keywords of the reference's constructor (``triune/runtime/streaming.py``). A tiered
        # optimizer given here updates the streamed layers through ``step_parameters`` once the engine is attached.
        layers_attr = layers_attr or layers_path or (config.layers_path if config is not None else None)
        self._ctor_optimizer = optimizer
        self.model = model
        self.device = torch.device(device)
        self.cfg = config or StreamingConfig()
        self.cuda = self.device.type == "cuda"
        self.layers: List[nn.Module] = list(find_layer_list(model, layers_attr))
        pin = self.cuda if self.cfg.pin_memory is None else (self.cfg.pin_memory and self.cuda)
        self.resident = set(range(min(self.cfg.resident_gpu_layers, len(self.layers))))
        self.stores: Dict[int, LayerStore] = {}
        self.h2d_stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.d2h_stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.telemetry = {"h2d_bytes": 0, "d2h_bytes": 0, "h2d_copies": 0, "d2h_copies": 0, "peak_staged_layers": 0}
        self._staged: Dict[int, int] = {}
        self._attached = False
        self._orig_forward: Dict[int, Any] = {}
        self._pin = pin
        self.opt_state: Dict[int, Dict[str, torch.Tensor]] = {}
        self.step_count = 0
        self.layer_optimizer = None  # StreamedLayerOptimizer: tiered updates of the streamed layers

    def _chunk_for_layer_idx(self, idx: int):
        """(window number, first layer, last layer) of the staging window that holds layer ``idx``; windows are
        ``chunk_size`` layers wide (``triune/runtime/streaming.py:215-220`` of the reference)."""
        w = max(1, int(self.cfg.chunk_size))
        c = idx // w
        return c, c * w, min(len(self.layers), (c + 1) * w) - 1

    def _resolve_layers(self) -> List[nn.Module]:
        """The layer stack this engine streams (the reference's name of the discovery step)."""
        return list(self.layers)

    def enable_tiered_optimizer(self, make_optimizer=None, state_dtype: torch.dtype = torch.float32, **optimizer_kwargs):
        """Update streamed layers with the tiered optimizer (AdamW / Muon / CentroidSteer through
        ``step_parameters``, one layer's state on the device at a time) instead of the built-in AdamW."""
        from .streamed_optimizer import StreamedLayerOptimizer

        if not self._attached:
            self.attach()
        self.layer_optimizer = StreamedLayerOptimizer(self, make_optimizer, state_dtype, **optimizer_kwargs)
        return self.layer_optimizer

    def drop_prefetched(self):
        """Free device copies that were prefetched but are not in use (called when a layer raises: the prefetch of
        its neighbour would otherwise stay on the device until that layer next runs)."""
        for i, st in self.stores.items():
            if self._staged.get(i, 0) == 0 and st.device_buf is not None:
                if self.cuda:
                    self.h2d_stream.synchronize()
                st.bind_host()
                st.device_buf = None
                st.ready = None

    def cleanup(self):
        """Return every streamed layer to its host storage and drop staged device buffers and in-flight gradient
        bookkeeping (after an exception in forward, backward or the optimizer pass the engine is reusable)."""
        if self.cuda:
            for s_ in (self.h2d_stream, self.d2h_stream):
                s_.synchronize()
        for i, st in self.stores.items():
            st.bind_host()
            st.device_buf = None
            st.ready = None
            self._staged[i] = 0
            for p in st.params:
                p.grad = None

    # ------------------------------------------------------------------ the reference's method names
    # (``triune/runtime/streaming.py:442-450, 953-1078, 1209-1243``): the same operations under the names its callers use
    def set_optimizer(self, optimizer) -> None:
        """The optimizer that updates the root (non-streamed) parameters in ``step_optimizer``; a tiered optimizer also
        becomes the kind that updates the streamed layers."""
        self.optimizer = optimizer
        self._ctor_optimizer = optimizer
        if self._attached and optimizer is not None and hasattr(optimizer, "step_parameters") and self.layer_optimizer is None:
            kind = type(optimizer)
            kw = {k: getattr(optimizer, k) for k in ("lr", "weight_decay") if isinstance(getattr(optimizer, k, None), (int, float))}
            self.enable_tiered_optimizer(lambda module: kind(module, **kw))

    def get_root_parameters(self) -> List[nn.Parameter]:
        """Parameters outside the streamed block stack (embeddings, router, heads): resident on the device."""
        inside = {id(p) for layer in self.layers for p in layer.parameters()}
        return [p for p in self.model.parameters() if id(p) not in inside]

    def cleanup_resident_layers(self) -> None:
        self.cleanup()

    def flush_d2h_transfers(self) -> None:
        """Wait until every gradient that is on its way to host memory has arrived."""
        if self.cuda:
            self.d2h_stream.synchronize()

    def zero_grad(self) -> None:
        self.model.zero_grad(set_to_none=True)
        opt = getattr(self, "optimizer", None)
        if opt is not None:
            opt.zero_grad(set_to_none=True)
        for st in self.stores.values():  # gradients of streamed layers accumulate in their host buffers
            st.grad_sumsq = None
            if getattr(st, "_has_grad", False):
                st.host_grad.zero_()
                st._has_grad = False

    def step_optimizer(self, optimizer=None, **kw) -> float:
        """Clip, update the root parameters with ``optimizer`` and the streamed layers with their own optimizer; -> the
        global gradient norm."""
        return self.step_streaming_optimizer(optimizer if optimizer is not None else getattr(self, "optimizer", None), **kw)

    # ------------------------------------------------------------------ attach / detach
    def attach(self):
        if self._attached:
            return self
        layer_params = set()
        for i, layer in enumerate(self.layers):
            if i in self.resident:
                layer.to(self.device)
                continue
            layer.to("cpu")
            self.stores[i] = LayerStore(layer, self._pin, torch.bfloat16 if self.cfg.grad_dtype == "bf16" else torch.float32,
                                        fp8=self.cfg.fp8_weights)
            layer_params.update(id(p) for p in layer.parameters())
            self._wrap(i, layer)
        # root: everything that is not a streamed layer
        for p in self.model.parameters():
            if id(p) not in layer_params and p.device != self.device:
                p.data = p.data.to(self.device)
        for b in self.model.buffers():
            b.data = b.data.to(self.device)
        self._attached = True
        opt = self._ctor_optimizer
        if opt is not None and hasattr(opt, "step_parameters") and getattr(self, "layer_optimizer", None) is None:
            # the constructor was given a tiered optimizer: streamed layers are updated by the same kind, with its settings
            kind = type(opt)
            kw = {k: getattr(opt, k) for k in ("lr", "weight_decay") if isinstance(getattr(opt, k, None), (int, float))}
            self.enable_tiered_optimizer(lambda module: kind(module, **kw))
        return self

    def detach(self):
        for i, layer in enumerate(self.layers):
            if i in self._orig_forward:
                layer.forward = self._orig_forward.pop(i)
            if i in self.stores:
                self.stores[i].bind_host()
        self._attached = False

    def _wrap(self, i: int, layer: nn.Module):
        orig = layer.forward
        self._orig_forward[i] = orig
        engine = self

        def forward(x, *args, **kwargs):
            if torch.is_grad_enabled() and engine.cfg.activation_checkpointing and x.requires_grad:
                out = _StreamedLayerFn.apply(engine, i, orig, args, kwargs, x)
                return engine._unflatten(i, out)
            engine.stage(i, prefetch=i + 1)
            try:
                out = orig(x, *args, **kwargs)
            except BaseException:
                engine.release(i)
                engine.drop_prefetched()
                raise
            if not torch.is_grad_enabled():  # with a graph recorded and no recomputation, backward still reads these weights
                engine.release(i)
            return out

        layer.forward = forward

    # outputs of a block are (x, logits_or_None, cache_or_None); only tensors pass through autograd
    def _flatten(self, i, out):
        if torch.is_tensor(out):
            self._out_struct = None
            return out
        tensors = tuple(o for o in out if torch.is_tensor(o))
        self._out_struct = [torch.is_tensor(o) for o in out]
        self._out_consts = [None if torch.is_tensor(o) else o for o in out]
        return tensors if len(tensors) > 1 else tensors[0]

    def _unflatten(self, i, flat):
        if getattr(self, "_out_struct", None) is None:
            return flat
        it = iter(flat if isinstance(flat, tuple) else (flat,))
        return tuple(next(it) if is_t else c for is_t, c in zip(self._out_struct, self._out_consts))

    # ------------------------------------------------------------------ staging
    def _start_copy(self, i: int):
        st = self.stores[i]
        if st.device_buf is not None:
            return
        nbytes = st.fp8_stage_bytes() if st.fp8 else st.host.numel() * st.host.element_size()
        if not self.cuda:
            st.device_buf = st.expand_fp8(self.device) if st.fp8 else st.host
            self.telemetry["h2d_bytes"] += nbytes
            self.telemetry["h2d_copies"] += 1
            return
        with torch.cuda.stream(self.h2d_stream):
            st.device_buf = st.expand_fp8(self.device) if st.fp8 else st.host.to(self.device, non_blocking=True)
            st.ready = torch.cuda.Event()
            st.ready.record(self.h2d_stream)
        self.telemetry["h2d_bytes"] += nbytes
        self.telemetry["h2d_copies"] += 1

    def stage(self, i: int, prefetch: Optional[int] = None):
        if i not in self.stores:
            return
        self._start_copy(i)
        st = self.stores[i]
        if self.cuda and st.ready is not None:
            torch.cuda.current_stream(self.device).wait_event(st.ready)
        st.bind(st.device_buf)
        self._staged[i] = self._staged.get(i, 0) + 1
        self.telemetry["peak_staged_layers"] = max(self.telemetry["peak_staged_layers"],
                                                   sum(1 for s in self.stores.values() if s.device_buf is not None))
        c, lo, hi = self._chunk_for_layer_idx(i)
        ahead = range(i + 1, hi + 1) if prefetch is None or prefetch >= i else range(lo, i)
        for j in ahead:  # chunk_size > 1: the rest of this layer's window, in the direction of travel, comes with it
            if j in self.stores:
                self._start_copy(j)
        if self.cfg.async_prefetch and prefetch is not None and prefetch in self.stores:
            self._start_copy(prefetch)

    def release(self, i: int):
        if i not in self.stores:
            return
        st = self.stores[i]
        self._staged[i] = max(0, self._staged.get(i, 0) - 1)
        if self._staged[i] == 0:
            if self.cuda and st.device_buf is not None:
                st.device_buf.record_stream(torch.cuda.current_stream(self.device))
            st.bind_host()
            st.device_buf = None
            st.ready = None

    def collect_grads(self, i: int):
        """Move the gradients of layer i (on the device after its backward) into the pinned host buffer."""
        st = self.stores[i]
        flat = torch.zeros(st.numel, dtype=torch.float32, device=self.device)
        for p, (off, n, _) in zip(st.params, st.slices):
            if p.grad is not None:
                flat[off : off + n] = p.grad.reshape(-1).float()
                p.grad = None
        sumsq = flat.double().pow(2).sum()
        st.grad_sumsq = sumsq if st.grad_sumsq is None else st.grad_sumsq + sumsq
        if self.cuda:
            self.d2h_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.d2h_stream):
                acc = flat if self._first_micro(i) else flat + st.host_grad.to(self.device, non_blocking=True).float()
                st.host_grad.copy_(acc.to(st.host_grad.dtype), non_blocking=True)
                flat.record_stream(self.d2h_stream)
        else:
            acc = flat if self._first_micro(i) else flat + st.host_grad.float()
            st.host_grad.copy_(acc.to(st.host_grad.dtype))
        st._has_grad = True
        self.telemetry["d2h_bytes"] += st.numel * st.host_grad.element_size()
        self.telemetry["d2h_copies"] += 1

    def _first_micro(self, i: int) -> bool:
        return not getattr(self.stores[i], "_has_grad", False)

    # ------------------------------------------------------------------ optimizer
    @torch.no_grad()
    def step_streaming_optimizer(self, optimizer=None, grad_clip: Optional[float] = None, lr: float = 1e-4,
                                 betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.05):
        """Global-norm clip (fp64) then: root/resident parameters through ``optimizer`` (if given), streamed layers
        through a per-layer fused AdamW whose fp32 state lives in pinned host memory."""
        clip = self.cfg.grad_clip if grad_clip is None else grad_clip
        if self.cuda:
            self.d2h_stream.synchronize()
        total = torch.zeros((), dtype=torch.float64, device=self.device)
        streamed = set()
        for st in self.stores.values():
            streamed.update(id(p) for p in st.params)
            if st.grad_sumsq is not None:
                total += st.grad_sumsq.to(self.device)
        # root gradients: autograd's ``.grad``, or the fp32 arena view the kernels accumulate into (``main_grad``) when
        # the root optimizer is arena-based; ``.grad`` leftovers are folded into the arena first
        root_grads = []
        seen = set()
        for p in self.model.parameters():
            if id(p) in streamed or id(p) in seen:
                continue
            seen.add(id(p))
            mg = getattr(p, "main_grad", None)
            if mg is not None:
                if p.grad is not None:
                    mg.add_(p.grad.to(mg.dtype))
                    p.grad = None
                root_grads.append(mg)
            elif p.grad is not None:
                root_grads.append(p.grad)
        for g in root_grads:
            total += g.double().pow(2).sum()
        norm = total.sqrt()
        coef = torch.clamp(clip / (norm + 1e-6), max=1.0).float() if clip and clip > 0 else torch.ones((), device=self.device)
        for g in root_grads:
            g.mul_(coef.to(g.dtype))
        if optimizer is not None:
            optimizer.step()
            optimizer.zero_grad(set_to_none=True)
        self.step_count += 1
        t = self.step_count
        b1, b2 = betas
        try:
            if self.layer_optimizer is not None:
                self._step_layers_tiered(coef)
            else:
                self._step_layers_adamw(coef, t, lr, b1, b2, eps, weight_decay)
        except Exception:
            self.cleanup()
            raise
        if self.cuda:
            torch.cuda.current_stream(self.device).synchronize()
        return float(norm)

    def _step_layers_tiered(self, coef):
        pool = self.layer_optimizer
        ids = sorted(i for i, st in self.stores.items() if getattr(st, "_has_grad", False))
        last_of_group = {id(pool.group_of(i)): i for i in ids}
        for i in ids:
            st = self.stores[i]
            g = st.host_grad.to(self.device, non_blocking=True).float()
            self.telemetry["h2d_bytes"] += st.numel * st.host_grad.element_size()
            pool.step_layer(i, g, coef, is_global_step_end=(last_of_group[id(pool.group_of(i))] == i))
            if self.cuda:
                torch.cuda.current_stream(self.device).synchronize()  # host_grad / host are reused right away
            if st.fp8:
                st.refresh_fp8()
                self.telemetry["d2h_bytes"] += st.fp8_stage_bytes() if self.cuda else 0
            st.host_grad.zero_()
            st.grad_sumsq = None
            st._has_grad = False

    def _step_layers_adamw(self, coef, t, lr, b1, b2, eps, weight_decay):
        for i, st in self.stores.items():
            if not getattr(st, "_has_grad", False):
                continue
            if i not in self.opt_state:
                mk = lambda: (torch.zeros(st.numel, dtype=torch.float32).pin_memory() if self._pin
                              else torch.zeros(st.numel, dtype=torch.float32))
                self.opt_state[i] = {"m": mk(), "v": mk(), "master": mk()}
                self.opt_state[i]["master"].copy_(st.host.float())
            os_ = self.opt_state[i]
            dev = self.device
            g = st.host_grad.to(dev, non_blocking=True).float() * coef
            m, v, w = (os_[k].to(dev, non_blocking=True) for k in ("m", "v", "master"))
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            w.mul_(1 - lr * weight_decay).addcdiv_(m / (1 - b1**t), (v / (1 - b2**t)).sqrt() + eps, value=-lr)
            os_["m"].copy_(m, non_blocking=True)
            os_["v"].copy_(v, non_blocking=True)
            os_["master"].copy_(w, non_blocking=True)
            wq = w.to(st.host.dtype)
            st.host.copy_(wq, non_blocking=True)
            if st.fp8:  # the staging copy follows the update: quantised on the device, written back beside the master
                st.refresh_fp8(wq)
                self.telemetry["d2h_bytes"] += st.fp8_stage_bytes()
            st.host_grad.zero_()
            st.grad_sumsq = None
            st._has_grad = False
            self.telemetry["h2d_bytes"] += st.numel * (12 + st.host_grad.element_size())
            self.telemetry["d2h_bytes"] += st.numel * 14

    def get_telemetry(self) -> Dict[str, int]:
        return dict(self.telemetry)


class _StreamedLayerFn(torch.autograd.Function):
    """Checkpointed execution of one streamed layer: forward keeps only the input; backward re-stages the weights,
    recomputes, back-propagates and ships the weight gradients to the host."""

    @staticmethod
    def forward(ctx, engine: LayerStreamingEngine, i: int, fn, args, kwargs, x):
        ctx.engine, ctx.i, ctx.fn, ctx.args, ctx.kwargs = engine, i, fn, args, kwargs
        ctx.save_for_backward(x)
        engine.stage(i, prefetch=i + 1)
        try:
            with torch.no_grad():
                out = fn(x, *args, **kwargs)
        except BaseException:
            engine.release(i)
            engine.drop_prefetched()
            raise
        engine.release(i)
        return engine._flatten(i, out)

    @staticmethod
    def backward(ctx, *grads):
        engine, i = ctx.engine, ctx.i
        (x,) = ctx.saved_tensors
        engine.stage(i, prefetch=i - 1)
        try:
            xd = x.detach().requires_grad_(True)
            with torch.enable_grad():
                kw = dict(ctx.kwargs)
                if "update_stats" in kw:
                    kw["update_stats"] = False  # statistics were updated by the first pass
                out = ctx.fn(xd, *ctx.args, **kw)
            outs = [o for o in (out if isinstance(out, tuple) else (out,)) if torch.is_tensor(o)]
            pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and o.requires_grad]
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
            engine.collect_grads(i)
        except BaseException:
            engine.release(i)
            engine.drop_prefetched()
            for p in engine.stores[i].params:
                p.grad = None
            raise
        engine.release(i)
        return None, None, None, None, None, xd.grad


def enable_layer_streaming(model: nn.Module, device, config: Optional[StreamingConfig] = None, **kw) -> LayerStreamingEngine:
    cfg = config or StreamingConfig(**{k: v for k, v in kw.items() if k in StreamingConfig.__dataclass_fields__})
    eng = LayerStreamingEngine(model, device, cfg).attach()
    model._streaming_engine = eng
    return eng
