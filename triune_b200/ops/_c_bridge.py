"""ctypes bridge to ``libtriune_core.so`` (reference: ``triune/ops/_c_bridge.py:16-378``).

Loads the C-ABI engine library built by ``triune_b200._build.build_core``, binds the exported signatures and
offers ``c_*`` wrappers over contiguous fp32 CPU tensors plus the ``NativeTriuneEngine`` and
``PinnedStageRing`` classes.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_uint16, c_uint32, c_uint64, c_void_p
from typing import Optional

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "libtriune_core.so")
_lib = None


class TriuneConfig(Structure):
    _fields_ = [("vocab_size", c_int), ("hidden_dim", c_int), ("num_layers", c_int), ("num_heads", c_int),
                ("head_dim", c_int), ("num_experts", c_int), ("top_k", c_int), ("max_seq_len", c_int),
                ("reflex_threshold", c_float)]


class TriuneStepStats(Structure):
    _fields_ = [("loss", c_float), ("lm_loss", c_float), ("router_loss", c_float), ("active_tier", c_int),
                ("tokens_processed", c_int), ("step_time_ms", c_float), ("vram_used_mb", c_float),
                ("cuda_runtime_bound", c_int)]


TriuneConfigStruct, TriuneStepStatsStruct = TriuneConfig, TriuneStepStats  # the reference's names of the two structures


def load_library(path: Optional[str] = None):
    global _lib
    if _lib is not None:
        return _lib
    p = path or _LIB_PATH
    if not os.path.exists(p):
        return None
    lib = ctypes.CDLL(p)
    fp, ip = POINTER(c_float), POINTER(c_int)
    lib.triune_engine_create.restype = c_void_p
    lib.triune_engine_create.argtypes = [POINTER(TriuneConfig), c_int]
    lib.triune_engine_destroy.argtypes = [c_void_p]
    lib.triune_engine_version.restype = c_char_p
    lib.triune_has_cuda_runtime.restype = c_int
    lib.triune_engine_step.restype = c_int
    lib.triune_engine_step.argtypes = [c_void_p, POINTER(c_uint16), POINTER(c_uint16), c_int, c_int, POINTER(TriuneStepStats)]
    lib.triune_cuda_graph_capture.restype = c_int
    lib.triune_cuda_graph_capture.argtypes = [c_void_p, c_int, c_int]
    lib.triune_cuda_graph_replay.restype = c_int
    lib.triune_cuda_graph_replay.argtypes = [c_void_p]
    lib.triune_centroid_steer_update_f32.argtypes = [fp, fp, c_int, c_int, c_float, c_float]
    lib.triune_route_tiers_f32.argtypes = [fp, fp, ip, c_int, c_float]
    lib.triune_compute_neuron_heatmap_f32.argtypes = [fp, fp, POINTER(c_uint32), c_int, c_int]
    lib.triune_gla_recurrent_step_f32.argtypes = [fp, fp, fp, fp, fp, fp, c_int, c_int]
    lib.triune_engine_set_losses.argtypes = [c_void_p, c_float, c_float, c_float, c_int]
    lib.triune_tier_colour_render_f32.argtypes = [fp, ip, POINTER(c_uint32), c_int, c_int]
    lib.triune_stage_ring_create.restype = c_void_p
    lib.triune_stage_ring_create.argtypes = [c_int, c_int, c_uint64]
    lib.triune_stage_ring_destroy.argtypes = [c_void_p]
    lib.triune_stage_ring_submit.restype = c_int
    lib.triune_stage_ring_submit.argtypes = [c_void_p, c_void_p, c_void_p, c_uint64]
    lib.triune_stage_ring_wait.restype = c_int
    lib.triune_stage_ring_wait.argtypes = [c_void_p, c_int]
    lib.triune_stage_ring_host_ptr.restype = c_void_p
    lib.triune_stage_ring_host_ptr.argtypes = [c_void_p, c_int]
    lib.triune_stage_ring_bytes_moved.restype = c_uint64
    lib.triune_stage_ring_bytes_moved.argtypes = [c_void_p]
    _lib = lib
    return lib


def is_available() -> bool:
    return load_library() is not None


def _fp(t: torch.Tensor):
    assert t.device.type == "cpu" and t.dtype == torch.float32 and t.is_contiguous()
    return ctypes.cast(t.data_ptr(), POINTER(c_float))


def c_centroid_steer_update(P: torch.Tensor, G: torch.Tensor, steer_scale: float, momentum: float) -> torch.Tensor:
    load_library().triune_centroid_steer_update_f32(_fp(P), _fp(G), P.shape[0], P.numel() // P.shape[0], steer_scale, momentum)
    return P


def c_route_tiers(logits: torch.Tensor, threshold: float = 0.5):
    n = logits.shape[0]
    probs = torch.empty(n, 3)
    tiers = torch.empty(n, dtype=torch.int32)
    load_library().triune_route_tiers_f32(_fp(logits), _fp(probs), ctypes.cast(tiers.data_ptr(), POINTER(c_int)), n, threshold)
    return probs, tiers


def c_neuron_heatmap(act: torch.Tensor, num_bins: int):
    bins = torch.empty(num_bins)
    rgba = torch.empty(num_bins, dtype=torch.int32)
    load_library().triune_compute_neuron_heatmap_f32(_fp(act), _fp(bins), ctypes.cast(rgba.data_ptr(), POINTER(c_uint32)),
                                                      act.numel(), num_bins)
    return bins, rgba.to(torch.int64) & 0xFFFFFFFF


def c_tier_colour_render(act: torch.Tensor, tiers: torch.Tensor) -> torch.Tensor:
    rows, width = act.shape
    rgba = torch.empty(rows, width, dtype=torch.int32)
    t32 = tiers.to(torch.int32).contiguous()
    load_library().triune_tier_colour_render_f32(_fp(act), ctypes.cast(t32.data_ptr(), POINTER(c_int)),
                                                  ctypes.cast(rgba.data_ptr(), POINTER(c_uint32)), rows, width)
    return rgba.view(torch.uint8).view(rows, width, 4)


def c_gla_recurrent_step(q, k, v, g, state):
    """q,k,v,g [BH, d] fp32; state [BH, d, d] fp32 updated in place; returns out [BH, d]."""
    out = torch.empty_like(q)
    load_library().triune_gla_recurrent_step_f32(_fp(q), _fp(k), _fp(v), _fp(g), _fp(state), _fp(out), q.shape[0], q.shape[1])
    return out


class NativeTriuneEngine:
    def __init__(self, vocab_size=32000, hidden_dim=384, num_layers=8, num_heads=6, head_dim=64, num_experts=8, top_k=2,
                 max_seq_len=2048, reflex_threshold=0.5, device_id=0):
        lib = load_library()
        if lib is None:
            raise RuntimeError("libtriune_core.so is not built; run python -m triune_b200._build")
        self._lib = lib
        self.cfg = TriuneConfig(vocab_size, hidden_dim, num_layers, num_heads, head_dim, num_experts, top_k, max_seq_len,
                                reflex_threshold)
        self._h = lib.triune_engine_create(ctypes.byref(self.cfg), device_id)
        if not self._h:
            raise RuntimeError("triune_engine_create failed")

    @property
    def is_ready(self) -> bool:
        return bool(self._lib is not None and self._h)

    @property
    def version(self) -> str:
        return self._lib.triune_engine_version().decode()

    def set_losses(self, loss, lm_loss, router_loss, tier=2):
        self._lib.triune_engine_set_losses(self._h, loss, lm_loss, router_loss, tier)

    def step(self, input_tokens: torch.Tensor, target_tokens: Optional[torch.Tensor] = None) -> dict:
        x = input_tokens.to(torch.int16).contiguous()
        y = target_tokens.to(torch.int16).contiguous() if target_tokens is not None else None
        st = TriuneStepStats()
        rc = self._lib.triune_engine_step(self._h, ctypes.cast(x.data_ptr(), POINTER(c_uint16)),
                                          ctypes.cast(y.data_ptr(), POINTER(c_uint16)) if y is not None else None,
                                          x.shape[0], x.shape[1], ctypes.byref(st))
        if rc != 0:
            raise RuntimeError(f"triune_engine_step failed with code {rc}")
        return {f[0]: getattr(st, f[0]) for f in TriuneStepStats._fields_}

    def capture_graph(self, batch, seq) -> int:
        return self._lib.triune_cuda_graph_capture(self._h, batch, seq)

    def replay_graph(self) -> int:
        return self._lib.triune_cuda_graph_replay(self._h)

    def close(self):
        if self._h:
            self._lib.triune_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PinnedStageRing:
    """Pinned host->device staging ring (cudaMemcpyAsync on a side stream, one event per slot)."""

    def __init__(self, device_id: int, num_slots: int, slot_bytes: int):
        self._lib = load_library()
        self._h = self._lib.triune_stage_ring_create(device_id, num_slots, slot_bytes)
        if not self._h:
            raise RuntimeError("stage ring creation failed")

    def submit(self, src: torch.Tensor, dst: torch.Tensor) -> int:
        nbytes = src.numel() * src.element_size()
        slot = self._lib.triune_stage_ring_submit(self._h, src.data_ptr(), dst.data_ptr(), nbytes)
        if slot < 0:
            raise RuntimeError(f"stage submit failed ({slot})")
        return slot

    def wait(self, slot: int) -> None:
        if self._lib.triune_stage_ring_wait(self._h, slot) != 0:
            raise RuntimeError("stage wait failed")

    @property
    def bytes_moved(self) -> int:
        return int(self._lib.triune_stage_ring_bytes_moved(self._h))

    def close(self):
        if self._h:
            self._lib.triune_stage_ring_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def get_native_c_info() -> dict:
    """Which native pieces are loaded: the C-ABI engine library and the CUDA extension."""
    from .. import _ext

    lib = None
    try:
        lib = load_library()
    except Exception:
        pass
    return {"c_engine_loaded": lib is not None, "c_engine_path": str(getattr(lib, "_name", "")) if lib is not None else None,
            "cuda_extension": _ext.ext_available(), "simd": "avx2+fma", "arch": "sm_100a"}
