"""Per-parameter host <-> device staging with optional compressed transfer.

Parity (``triune/runtime/staging.py:19-621``): ``StagingBuffer`` (pinned host master, device execution tensor,
forward snapshot so the backward pass re-stages the weights the forward saw), ``FP8StagingBuffer`` (the host keeps an
E4M3 copy + scale so only one byte per weight crosses PCIe; the master is untouched), ``NVFP4StagingBuffer`` (packed
4-bit copy), ``ParameterStager`` (register a module, stage / apply / release / sync a layer, read-only buffer
detection, H2D / D2H telemetry).

On a B200 the host link is the bottleneck of a streamed step by an order of magnitude (PCIe / C2C versus 7.7 TB/s of
HBM), so the compressed buffers decode ON THE DEVICE after the copy: bytes moved shrink 2x / 3.5x while the decode is a
bandwidth-trivial kernel. ``LayerStreamingEngine`` stages whole layers as one flat copy; this class is the
finer-grained tool (foreign modules, mixed precision per tensor).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref


def _pin(t: torch.Tensor) -> torch.Tensor:
    if torch.cuda.is_available() and not t.is_pinned():
        try:
            return t.pin_memory()
        except RuntimeError:
            return t
    return t


@dataclass
class StagingBuffer:
    param: nn.Parameter
    cpu_master: torch.Tensor
    gpu_tensor: Optional[torch.Tensor] = None
    event: Optional[Any] = None
    forward_snapshot: Optional[torch.Tensor] = None
    capture_forward_snapshots: bool = True
    is_buffer: bool = False
    read_only: bool = False

    @property
    def cpu_master_bytes(self) -> int:
        return self.cpu_master.numel() * self.cpu_master.element_size()

    @property
    def snapshot_bytes(self) -> int:
        s = self.forward_snapshot
        return s.numel() * s.element_size() if s is not None else 0

    @property
    def gpu_bytes(self) -> int:
        g = self.gpu_tensor
        return g.numel() * g.element_size() if g is not None else 0

    def transfer_bytes(self) -> int:
        return self.cpu_master_bytes

    def _source(self, is_backward: bool) -> torch.Tensor:
        if not self.capture_forward_snapshots:
            return self.cpu_master
        if is_backward and self.forward_snapshot is not None:
            return self.forward_snapshot
        if self.forward_snapshot is None:
            self.forward_snapshot = _pin(self.cpu_master.detach().clone())
        return self.cpu_master

    def _upload(self, source: torch.Tensor, device, dtype) -> torch.Tensor:
        t = source.to(device, non_blocking=source.is_pinned())
        t = t.to(dtype) if t.dtype != dtype else t
        return t.clone() if t.data_ptr() == source.data_ptr() else t

    def stage_to_gpu(self, device, stream=None, target_dtype: Optional[torch.dtype] = None, non_blocking: bool = True,
                     is_backward: bool = False) -> torch.Tensor:
        device = torch.device(device)
        src = self._source(is_backward)
        dtype = target_dtype or src.dtype
        if stream is not None and device.type == "cuda":
            with torch.cuda.stream(stream):
                self.gpu_tensor = self._upload(src, device, dtype)
                self.event = torch.cuda.Event()
                self.event.record(stream)
        else:
            self.gpu_tensor, self.event = self._upload(src, device, dtype), None
        return self.gpu_tensor

    def wait(self) -> None:
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)  # device-side wait: the host does not block
            self.event = None

    def sync_to_cpu(self, non_blocking: bool = True) -> None:
        if self.gpu_tensor is not None:
            self.wait()
            self.cpu_master.copy_(self.gpu_tensor.to(self.cpu_master.dtype), non_blocking=non_blocking and self.cpu_master.is_pinned())
        self.forward_snapshot = None

    def release_gpu(self, clear_snapshot: bool = False, keep_snapshot_on_param: bool = False) -> None:
        if self.is_buffer and not self.read_only and self.gpu_tensor is not None:
            self.wait()
            self.cpu_master.copy_(self.gpu_tensor.to(self.cpu_master.dtype))  # running statistics etc. must survive
        self.gpu_tensor, self.event = None, None
        if clear_snapshot:
            self.forward_snapshot = None
        keep = keep_snapshot_on_param and self.forward_snapshot is not None and not self.is_buffer and not clear_snapshot
        self.param.data = self.forward_snapshot if keep else self.cpu_master


@dataclass
class FP8StagingBuffer(StagingBuffer):
    """Host keeps (E4M3 weights, fp32 128x128 block scales); staging moves 1 byte / weight and decodes on the device."""

    fp8_host: Optional[torch.Tensor] = None
    scale_host: Optional[torch.Tensor] = None
    _version: int = -1

    def _refresh(self):
        v = self.cpu_master._version
        if self.fp8_host is None or v != self._version:
            w = self.cpu_master.detach().float()
            w2 = w.reshape(w.shape[0], -1) if w.ndim >= 2 else w.reshape(1, -1)
            q, s = ref.fp8_block_quantize_weight(w2)
            self.fp8_host, self.scale_host, self._version = _pin(q), _pin(s), v

    @property
    def fp8_bytes(self) -> int:
        self._refresh()
        return self.fp8_host.numel() + self.scale_host.numel() * 4

    @property
    def saved_vram_bytes(self) -> int:
        return max(0, self.cpu_master_bytes - self.fp8_bytes)

    def transfer_bytes(self) -> int:
        return self.fp8_bytes

    def _upload(self, source, device, dtype):
        if source is not self.cpu_master:  # backward re-stage of a snapshot: exact bytes
            return super()._upload(source, device, dtype)
        self._refresh()
        q = self.fp8_host.to(device, non_blocking=self.fp8_host.is_pinned())
        s = self.scale_host.to(device, non_blocking=self.scale_host.is_pinned())
        R, C = q.shape
        w = q.float() * s.repeat_interleave(128, 0)[:R].repeat_interleave(128, 1)[:, :C]
        return w.to(dtype).reshape(self.cpu_master.shape)


@dataclass
class NVFP4StagingBuffer(StagingBuffer):
    """Host keeps packed NVFP4 (4.5 bits / weight); decoded on the device by the dequantise kernel."""

    packed_host: Optional[torch.Tensor] = None
    scales_host: Optional[torch.Tensor] = None
    tscale_host: Optional[torch.Tensor] = None
    _version: int = -1

    def eligible(self) -> bool:
        return self.cpu_master.ndim >= 2 and self.cpu_master.reshape(self.cpu_master.shape[0], -1).shape[1] % 16 == 0

    def _refresh(self):
        v = self.cpu_master._version
        if self.packed_host is None or v != self._version:
            w = self.cpu_master.detach().float()
            p, s, t = ref.nvfp4_quantize(w.reshape(w.shape[0], -1))
            self.packed_host, self.scales_host, self.tscale_host, self._version = _pin(p), _pin(s), t.reshape(1), v

    @property
    def nvfp4_bytes(self) -> int:
        self._refresh()
        return self.packed_host.numel() + self.scales_host.numel() + 4

    @property
    def saved_vram_bytes(self) -> int:
        return max(0, self.cpu_master_bytes - self.nvfp4_bytes)

    def transfer_bytes(self) -> int:
        return self.nvfp4_bytes if self.eligible() else self.cpu_master_bytes

    def _upload(self, source, device, dtype):
        if source is not self.cpu_master or not self.eligible():
            return super()._upload(source, device, dtype)
        self._refresh()
        p = self.packed_host.to(device, non_blocking=self.packed_host.is_pinned())
        s = self.scales_host.to(device, non_blocking=self.scales_host.is_pinned())
        t = self.tscale_host.to(device).reshape(())
        return ops.nvfp4_dequantize(p, s, t, dtype).reshape(self.cpu_master.shape)


class ParameterStager:
    def __init__(self, device, prefetch_stream=None, d2h_stream=None, use_fp8: bool = False, use_fp4: bool = False,
                 capture_forward_snapshots: bool = True, min_quant_numel: int = 65536):
        self.device = torch.device(device)
        self.prefetch_stream, self.d2h_stream = prefetch_stream, d2h_stream
        self.use_fp8, self.use_fp4 = use_fp8, use_fp4
        self.capture_forward_snapshots = capture_forward_snapshots
        self.min_quant_numel = min_quant_numel
        self.buffers: Dict[int, StagingBuffer] = {}
        self._by_module: Dict[int, List[StagingBuffer]] = {}
        self.telemetry: Dict[str, int] = {}
        self.reset_telemetry()

    # ------------------------------------------------------------------ registration
    def _make(self, t: nn.Parameter, is_buffer: bool, read_only: bool) -> StagingBuffer:
        master = _pin(t.data.detach().to("cpu"))
        quantisable = (not is_buffer and t.ndim >= 2 and t.numel() >= self.min_quant_numel and t.dtype.is_floating_point)
        kw = dict(param=t, cpu_master=master, capture_forward_snapshots=self.capture_forward_snapshots and not is_buffer,
                  is_buffer=is_buffer, read_only=read_only)
        if quantisable and self.use_fp4:
            b = NVFP4StagingBuffer(**kw)
            if b.eligible():
                return b
        if quantisable and self.use_fp8:
            return FP8StagingBuffer(**kw)
        return StagingBuffer(**kw)

    def register_module(self, module: nn.Module, register_backward_hooks: bool = False) -> None:
        """Move the module's tensors to (pinned) host masters and remember them. ``register_backward_hooks`` adds a full
        backward pre-hook that re-stages the forward-time weights before the module's backward runs."""
        bufs: List[StagingBuffer] = []
        for p in module.parameters(recurse=True):
            if id(p) not in self.buffers:
                self.buffers[id(p)] = self._make(p, False, not p.requires_grad)
                p.data = self.buffers[id(p)].cpu_master
            bufs.append(self.buffers[id(p)])
        persistent = {n for n, _ in module.named_buffers()} - {
            f"{mn + '.' if mn else ''}{bn}" for mn, m in module.named_modules() for bn in m._non_persistent_buffers_set}
        for name, b in module.named_buffers():
            if id(b) not in self.buffers:
                holder = nn.Parameter(b, requires_grad=False)  # uniform handling; the module keeps its own reference
                sb = self._make(holder, True, name not in persistent)
                sb._owner, sb._name = module, name
                self.buffers[id(b)] = sb
            bufs.append(self.buffers[id(b)])
        self._by_module[id(module)] = bufs
        if register_backward_hooks:
            module.register_full_backward_pre_hook(lambda m, g: self.stage_layer(m, is_backward=True, apply=True))

    def _layer_buffers(self, layer: nn.Module) -> List[StagingBuffer]:
        if id(layer) not in self._by_module:
            self.register_module(layer)
        return self._by_module[id(layer)]

    # ------------------------------------------------------------------ staging
    def stage_layer(self, layer: nn.Module, is_backward: bool = False, use_prefetch_stream: bool = False, apply: bool = True,
                    target_dtype: Optional[torch.dtype] = None) -> None:
        stream = self.prefetch_stream if use_prefetch_stream else None
        for b in self._layer_buffers(layer):
            if b.gpu_tensor is None:
                b.stage_to_gpu(self.device, stream, None if b.is_buffer else target_dtype, is_backward=is_backward)
                self.telemetry["h2d_async_transfers" if stream is not None else "h2d_sync_transfers"] += 1
                self.telemetry["h2d_bytes_transferred"] += b.transfer_bytes()
        if apply:
            self.apply_staged_tensors(layer)

    def apply_staged_tensors(self, layer: nn.Module) -> None:
        for b in self._layer_buffers(layer):
            if b.gpu_tensor is None:
                continue
            b.wait()
            if b.is_buffer:
                setattr_target = getattr(b, "_owner", None)
                if setattr_target is not None:
                    _set_buffer(setattr_target, b._name, b.gpu_tensor)
            else:
                b.param.data = b.gpu_tensor

    def release_layer(self, layer: nn.Module, clear_snapshot: bool = False) -> None:
        for b in self._layer_buffers(layer):
            gpu = b.gpu_tensor
            b.release_gpu(clear_snapshot=clear_snapshot)
            if b.is_buffer and getattr(b, "_owner", None) is not None and gpu is not None:
                _set_buffer(b._owner, b._name, b.cpu_master)

    def sync_layer_to_cpu(self, layer: nn.Module) -> None:
        """Write updated device weights back to the host masters (after an optimizer step on the device)."""
        ctx = torch.cuda.stream(self.d2h_stream) if self.d2h_stream is not None and self.device.type == "cuda" else None
        if ctx is not None:
            self.d2h_stream.wait_stream(torch.cuda.current_stream())
        for b in self._layer_buffers(layer):
            if b.gpu_tensor is None or b.read_only:
                continue
            if ctx is not None:
                with ctx:
                    b.sync_to_cpu()
                self.telemetry["d2h_async_transfers"] += 1
            else:
                b.sync_to_cpu(non_blocking=False)
                self.telemetry["d2h_sync_transfers"] += 1
            self.telemetry["d2h_bytes_transferred"] += b.cpu_master_bytes
        if ctx is not None:
            self.d2h_stream.synchronize()

    # ------------------------------------------------------------------ reporting / teardown
    def get_memory_summary(self) -> Dict[str, Any]:
        bufs = list(self.buffers.values())
        return {"num_buffers": len(bufs), "cpu_master_bytes": sum(b.cpu_master_bytes for b in bufs),
                "snapshot_bytes": sum(b.snapshot_bytes for b in bufs), "gpu_bytes": sum(b.gpu_bytes for b in bufs),
                "transfer_bytes_per_pass": sum(b.transfer_bytes() for b in bufs),
                "quantised_buffers": sum(isinstance(b, (FP8StagingBuffer, NVFP4StagingBuffer)) for b in bufs),
                "read_only_buffers": sum(b.read_only for b in bufs), **self.telemetry}

    def reset_telemetry(self) -> None:
        self.telemetry = {k: 0 for k in ("h2d_sync_transfers", "h2d_async_transfers", "h2d_bytes_transferred",
                                         "d2h_sync_transfers", "d2h_async_transfers", "d2h_bytes_transferred")}

    def cleanup_all(self) -> None:
        for b in self.buffers.values():
            gpu = b.gpu_tensor
            b.release_gpu(clear_snapshot=True)
            if b.is_buffer and getattr(b, "_owner", None) is not None and gpu is not None:
                _set_buffer(b._owner, b._name, b.cpu_master)

    def clear(self) -> None:
        self.cleanup_all()
        self.buffers.clear()
        self._by_module.clear()


def _set_buffer(owner: nn.Module, dotted: str, value: torch.Tensor) -> None:
    mod_path, _, name = dotted.rpartition(".")
    target = owner.get_submodule(mod_path) if mod_path else owner
    target._buffers[name] = value
