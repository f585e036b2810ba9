"""Session recurrent-state manager and the serving request queue.

Parity (``triune/api/srsm.py:11-144``): ``SessionRecurrentStateManager`` keeps the per-session recurrent cache (a list
of ``(state, offset)`` per layer) in an LRU with a TTL so a follow-up turn resumes without re-running the prefix;
``ServingRequestQueue`` bounds concurrency with a semaphore (16) and hands out cancel events.

Design for 180 GB parts: a GLA state is ``layers x heads x D x D`` fp32 (0.8 MB for the 90M model, ~10 MB for a
24-layer 1.5K-wide one), so thousands of sessions fit in HBM. Sessions therefore live in TWO tiers: a device tier with a
byte budget (resuming costs nothing) and a pinned-host tier that receives the least recently used sessions. Each
session is ONE flat tensor (all layers packed), so parking or restoring is a single asynchronous copy instead of one
per layer.
"""

from __future__ import annotations

import collections
import threading
import time
from typing import Any, Dict, List, Optional, Tuple

import torch


class _Entry:
    __slots__ = ("flat", "layout", "depth", "last_active", "on_device")

    def __init__(self, flat, layout, depth, on_device):
        self.flat, self.layout, self.depth, self.on_device = flat, layout, depth, on_device
        self.last_active = time.time()

    @property
    def nbytes(self) -> int:
        return self.flat.numel() * self.flat.element_size() if self.flat is not None else 0


def _pack(cache: List[Any]):
    """-> (flat tensor or None, layout). layout[i] = (shape or None, numel, offset value, dtype, passthrough item)."""
    tensors, layout = [], []
    for item in cache:
        state, off = (item if isinstance(item, tuple) else (None, 0)) if not torch.is_tensor(item) else (item, 0)
        if item is not None and not isinstance(item, tuple) and not torch.is_tensor(item):
            layout.append(("raw", item))
        elif torch.is_tensor(state):
            layout.append(("t", tuple(state.shape), state.numel(), off, state.dtype))
            tensors.append(state.detach().reshape(-1).float())
        else:
            layout.append(("none", off))
    flat = torch.cat(tensors) if tensors else None
    return flat, layout


def _unpack(flat: Optional[torch.Tensor], layout) -> List[Any]:
    out, pos = [], 0
    for rec in layout:
        if rec[0] == "raw":
            out.append(rec[1])
        elif rec[0] == "none":
            out.append((None, rec[1]))
        else:
            _, shape, n, off, dt = rec
            out.append((flat[pos : pos + n].view(shape).to(dt), off))
            pos += n
    return out


class SessionRecurrentStateManager:
    def __init__(self, max_active_sessions: int = 256, session_ttl_seconds: float = 3600.0, pin_memory: bool = True,
                 device_budget_bytes: int = 8 << 30):
        self.max_active_sessions, self.session_ttl_seconds = max_active_sessions, session_ttl_seconds
        self.pin_memory, self.device_budget_bytes = pin_memory, int(device_budget_bytes)
        self._lock = threading.Lock()
        self._sessions: "collections.OrderedDict[str, _Entry]" = collections.OrderedDict()
        self.hits = self.misses = self.spills = 0

    # ------------------------------------------------------------------ internals (lock held)
    def _purge_expired_locked(self) -> None:
        now = time.time()
        for sid in [s for s, e in self._sessions.items() if now - e.last_active > self.session_ttl_seconds]:
            del self._sessions[sid]

    def _device_bytes_locked(self) -> int:
        return sum(e.nbytes for e in self._sessions.values() if e.on_device)

    def _spill_locked(self) -> None:
        over = self._device_bytes_locked() - self.device_budget_bytes
        if over <= 0:
            return
        for e in self._sessions.values():  # oldest first
            if over <= 0:
                break
            if e.on_device and e.flat is not None:
                host = torch.empty(e.flat.shape, dtype=e.flat.dtype, pin_memory=self.pin_memory and torch.cuda.is_available())
                host.copy_(e.flat, non_blocking=True)
                over -= e.nbytes
                e.flat, e.on_device = host, False
                self.spills += 1
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()  # the host copies must be complete before the device blocks are reused

    # ------------------------------------------------------------------ API
    def get_session_cache(self, session_id: str, device) -> Optional[Tuple[List[Any], Optional[int]]]:
        if not session_id:
            return None
        device = torch.device(device)
        with self._lock:
            self._purge_expired_locked()
            e = self._sessions.get(session_id)
            if e is None:
                self.misses += 1
                return None
            self.hits += 1
            e.last_active = time.time()
            self._sessions.move_to_end(session_id)
            flat = e.flat
            if flat is not None and flat.device != device:
                flat = flat.to(device, non_blocking=True)
                if device.type == "cuda":
                    e.flat, e.on_device = flat, True
                    self._spill_locked()
            # the caller advances the state in place during generation: hand out a copy, keep ours intact until update
            return _unpack(flat.clone() if flat is not None else None, e.layout), e.depth

    def update_session_cache(self, session_id: str, cache: List[Any], depth: Optional[int] = None) -> None:
        if not session_id or not cache:
            return
        flat, layout = _pack(cache)
        on_dev = flat is not None and flat.is_cuda
        if flat is not None and not on_dev and self.pin_memory and torch.cuda.is_available():
            try:
                flat = flat.pin_memory()
            except RuntimeError:
                pass
        with self._lock:
            self._purge_expired_locked()
            self._sessions[session_id] = _Entry(flat, layout, depth, on_dev)
            self._sessions.move_to_end(session_id)
            while len(self._sessions) > self.max_active_sessions:
                self._sessions.popitem(last=False)
            self._spill_locked()

    def clear_session(self, session_id: str) -> bool:
        with self._lock:
            return self._sessions.pop(session_id, None) is not None

    def clear_all(self) -> None:
        with self._lock:
            self._sessions.clear()

    def stats(self) -> Dict[str, Any]:
        with self._lock:
            dev = self._device_bytes_locked()
            total = sum(e.nbytes for e in self._sessions.values())
            return {"active_sessions": len(self._sessions), "max_sessions": self.max_active_sessions,
                    "total_recurrent_memory_mb": round(total / 2**20, 2), "device_resident_mb": round(dev / 2**20, 2),
                    "host_parked_mb": round((total - dev) / 2**20, 2), "hits": self.hits, "misses": self.misses,
                    "spills": self.spills}


class ServingRequestQueue:
    def __init__(self, max_concurrency: int = 16):
        self.max_concurrency = max_concurrency
        self.active_requests: Dict[str, threading.Event] = {}
        self._lock = threading.Lock()
        self._semaphore = threading.Semaphore(max_concurrency)
        self.completed = self.rejected = 0

    def register_request(self, request_id: str) -> threading.Event:
        ev = threading.Event()
        with self._lock:
            self.active_requests[request_id] = ev
        return ev

    def unregister_request(self, request_id: str) -> None:
        with self._lock:
            if self.active_requests.pop(request_id, None) is not None:
                self.completed += 1

    def cancel_request(self, request_id: str) -> bool:
        with self._lock:
            ev = self.active_requests.get(request_id)
        if ev is None:
            return False
        ev.set()
        return True

    def cancel_all(self) -> int:
        with self._lock:
            evs = list(self.active_requests.values())
        for e in evs:
            e.set()
        return len(evs)

    def acquire(self, timeout: float = 30.0) -> bool:
        ok = self._semaphore.acquire(timeout=timeout)
        if not ok:
            self.rejected += 1
        return ok

    def release(self) -> None:
        self._semaphore.release()

    def stats(self) -> Dict[str, int]:
        with self._lock:
            return {"active": len(self.active_requests), "max_concurrency": self.max_concurrency, "completed": self.completed,
                    "rejected": self.rejected}
