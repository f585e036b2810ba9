"""Debugging aids for kernels that write through raw pointers: guard bands around output buffers and the index-error
word of the row-movement kernels.

The GPU pool has no memory checker, so stray writes are looked for the plain way: an output is carved out of a larger
buffer whose borders hold a known byte pattern, the kernel runs on the inner view, and the borders are compared
afterwards (``guarded_empty`` / ``check_guards``). An index that leaves its table is never followed by the kernels that
take index tables: it is skipped and recorded, and ``index_error()`` reads the record.
"""

from __future__ import annotations

from typing import Tuple

import torch

GUARD_BYTE = 0xA5


def guarded_empty(shape: Tuple[int, ...], dtype: torch.dtype, device, guard_rows: int = 4) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (inner view of ``shape``, the whole buffer). ``guard_rows`` rows of the trailing-dimension pitch in front of
    and behind the view are filled with ``GUARD_BYTE``; the view is contiguous and 256-byte aligned when the row size
    is a multiple of 256 bytes / ``guard_rows``."""
    cols = int(shape[-1])
    rows = 1
    for d in shape[:-1]:
        rows *= int(d)
    elem = torch.empty((), dtype=dtype).element_size()
    pad = guard_rows
    while (pad * cols * elem) % 256 != 0:  # keep the inner view aligned for TMA and vector access
        pad += 1
    whole = torch.empty((rows + 2 * pad, cols), dtype=dtype, device=device)
    whole.view(torch.uint8).fill_(GUARD_BYTE)
    inner = whole[pad : pad + rows].view(*shape)
    inner._guard_pad = pad  # type: ignore[attr-defined]
    return inner, whole


def check_guards(inner: torch.Tensor, whole: torch.Tensor) -> None:
    """Raise if a byte of either guard band changed."""
    pad = inner._guard_pad  # type: ignore[attr-defined]
    bytes_ = whole.view(torch.uint8)
    row = bytes_.shape[-1] if bytes_.dim() > 1 else 1
    flat = bytes_.reshape(-1)
    n = pad * row
    for name, band in (("front", flat[:n]), ("back", flat[-n:])):
        bad = (band != GUARD_BYTE).nonzero()
        if bad.numel():
            raise AssertionError(f"{name} guard band overwritten at byte {int(bad[0])} of {n} ({int(bad.numel())} bytes changed)")


def index_error(clear: bool = True):
    """None, or ``{"kernel", "row", "index", "limit"}`` of the first out-of-table index a row-movement kernel skipped
    since the last call. Synchronises the device."""
    from .. import _ext

    k, row, idx, lim = _ext.ext().index_error_word(bool(clear))
    if k == 0:
        return None
    return {"kernel": {1: "gather_rows", 2: "combine_rows"}.get(int(k), str(k)), "row": int(row), "index": int(idx), "limit": int(lim)}
