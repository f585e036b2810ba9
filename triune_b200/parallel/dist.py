"""Process-group setup and the scalar collectives of the trainer.

Parity: ``triune/trainer/distributed.py:57-186`` (``setup_distributed`` from ``WORLD_SIZE/RANK/LOCAL_RANK``,
NCCL on CUDA / gloo otherwise, ``all_reduce_tensor``, ``all_reduce_dict`` = one AVG all-reduce over a sorted
fp32 vector, ``cleanup_distributed``). One process per GPU; rendezvous on ``MASTER_ADDR`` (use 127.0.0.1).
"""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.distributed as dist


@dataclass
class DistributedContext:
    enabled: bool = False
    rank: int = 0
    local_rank: int = 0
    world_size: int = 1
    backend: Optional[str] = None
    device: torch.device = torch.device("cpu")

    @property
    def is_main(self) -> bool:
        return self.rank == 0


def setup_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> DistributedContext:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    if world <= 1:
        dev = torch.device("cuda", 0) if cuda else torch.device("cpu")
        if cuda:
            torch.cuda.set_device(0)
        return DistributedContext(False, 0, 0, 1, None, dev)
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if backend is None:
        backend = "nccl" if cuda else "gloo"
    dev = torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = dev
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return DistributedContext(True, rank, local, world, backend, dev)


def cleanup_distributed() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def all_reduce_tensor(t: torch.Tensor, ctx: Optional[DistributedContext] = None, op: str = "avg") -> torch.Tensor:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return t
    out = t.clone()
    dist.all_reduce(out, op=dist.ReduceOp.SUM)
    if op == "avg":
        out = out / dist.get_world_size()
    return out


def all_reduce_dict(d: Dict[str, float], ctx: Optional[DistributedContext] = None, device=None) -> Dict[str, float]:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return dict(d)
    keys = sorted(d)
    dev = device if device is not None else (torch.device("cuda", torch.cuda.current_device())
                                             if dist.get_backend() == "nccl" else torch.device("cpu"))
    v = torch.tensor([float(d[k]) for k in keys], dtype=torch.float32, device=dev)
    dist.all_reduce(v, op=dist.ReduceOp.SUM)
    v = v / dist.get_world_size()
    return {k: float(x) for k, x in zip(keys, v.tolist())}


def max_over_ranks(value: float, device=None) -> float:
    """Device-timed numbers are reported as the maximum over ranks."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    dev = device if device is not None else (torch.device("cuda", torch.cuda.current_device())
                                             if dist.get_backend() == "nccl" else torch.device("cpu"))
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
