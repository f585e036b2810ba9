"""Minimal safetensors reader / writer with no third-party dependency.

File layout: 8-byte little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}, "__metadata__":
{...}}``, then the raw little-endian tensor bytes. Parity: the reference ships a pure-Python fallback writer next to
the ``safetensors`` package path (``triune/export/exporter.py:28-146``); files written here load with the
``safetensors`` package and vice versa.
"""

from __future__ import annotations

import json
import mmap
import struct
from typing import Dict, Optional

import torch

_DT = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64", torch.int64: "I64",
       torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL",
       torch.float8_e4m3fn: "F8_E4M3", torch.float8_e5m2: "F8_E5M2"}
_RD = {v: k for k, v in _DT.items()}


def _raw(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    return t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    header, offset, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):
        t = tensors[name]
        if t.dtype not in _DT:
            raise TypeError(f"{name}: dtype {t.dtype} cannot be stored as safetensors")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _DT[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        blobs.append(t)
        offset += n
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for t in blobs:  # one tensor at a time: peak extra host memory is the largest tensor, not the model
            f.write(_raw(t))


def read_header(path: str) -> Dict[str, dict]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        return json.loads(f.read(n).decode("utf-8"))


def load_file(path: str, device: str = "cpu") -> Dict[str, torch.Tensor]:
    out = {}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        base = 8 + n
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            for name, info in header.items():
                if name == "__metadata__":
                    continue
                b, e = info["data_offsets"]
                dt = _RD[info["dtype"]]
                if e == b:
                    t = torch.empty(info["shape"], dtype=dt)
                else:
                    t = torch.frombuffer(bytearray(mm[base + b : base + e]), dtype=torch.uint8).view(dt).reshape(info["shape"])
                out[name] = t.to(device) if device != "cpu" else t
        finally:
            mm.close()
    return out
