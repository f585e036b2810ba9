"""Symmetric NVLink memory: one buffer per rank, mapped by every peer, plus a signal pad of epoch flags.

Built on ``torch.distributed._symmetric_memory`` (CUDA VMM allocations exchanged through the process-group
store), which gives every kernel a device array of peer base pointers, a per-rank signal pad and, when the
fabric supports it, an NVLS multicast address for ``multimem`` reduce / broadcast instructions. NCCL is used only
for the rendezvous; all data movement on the fused paths is issued from inside our kernels.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist


def _align(n: int, a: int = 256) -> int:
    return -(-n // a) * a


@dataclass
class Region:
    offset: int  # bytes from the buffer base
    nbytes: int


class SymmetricBuffer:
    """A byte buffer in symmetric memory carved into named regions at identical offsets on every rank."""

    def __init__(self, regions: Dict[str, int], device: torch.device, group=None, use_multimem: Optional[bool] = None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.regions: Dict[str, Region] = {}
        off = 0
        for name, nbytes in regions.items():
            self.regions[name] = Region(off, int(nbytes))
            off = _align(off + int(nbytes))
        self.nbytes = off
        self.tensor = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.bufs_dev = int(self.handle.buffer_ptrs_dev)
        self.signals_dev = int(self.handle.signal_pad_ptrs_dev)
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.multicast = mc
        self.use_multimem = bool(mc) if use_multimem is None else (bool(use_multimem) and bool(mc))
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(self.group)

    def view(self, name: str, dtype: torch.dtype, numel: Optional[int] = None) -> torch.Tensor:
        r = self.regions[name]
        t = self.tensor[r.offset : r.offset + r.nbytes].view(dtype)
        return t if numel is None else t[:numel]

    def offset(self, name: str) -> int:
        return self.regions[name].offset

    def table(self) -> Tuple[int, int, int, int, int]:
        """(rank, world, peer buffer pointer array, peer signal pad array, multicast address)."""
        return self.rank, self.world, self.bufs_dev, self.signals_dev, self.multicast if self.use_multimem else 0

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    # ------------------------------------------------------------------ protocol audit
    def signal_slots(self, max_ranks: int = 16) -> torch.Tensor:
        """This rank's signal pad as int32 [channels, max_ranks] (slot = channel * max_ranks + source rank)."""
        pad = self.handle.get_signal_pad(self.rank, dtype=torch.int32)
        n = pad.numel() // max_ranks * max_ranks
        return pad.reshape(-1)[:n].view(-1, max_ranks)

    def audit_signals(self, expected: Dict[int, int], max_ranks: int = 16) -> Dict[int, bool]:
        """After a run: for each channel, did EVERY peer's last signal arrive with the epoch the protocol ended on?
        ``expected`` maps channel -> final epoch. A slot behind its epoch is a signal that was never sent (or a step one
        rank skipped); a slot ahead of it is a rank that ran an extra step. Synchronises."""
        torch.cuda.synchronize(self.tensor.device)
        slots = self.signal_slots(max_ranks).cpu()
        return {int(ch): bool((slots[int(ch), : self.world] == int(ep)).all()) for ch, ep in expected.items()}
