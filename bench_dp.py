#!/usr/bin/env python
"""Data-parallel optimizer step alone: the fused NVLink kernels (reduce-scatter of the fp32 gradient arena into its
owners, AdamW on the owned shard, all-gather of the bf16 parameters) against one NCCL all-reduce plus a full update.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench_dp.py \\
        [--params 100e6] [--mode fused|nccl] [--multimem 0|1] [--matrix-frac 0.0] [--iters 10]

The arena is synthetic: ``--params`` parameters as 4M-element vectors (AdamW tier) and, with ``--matrix-frac``, that
share of them as 1024 x 1024 matrices (Muon tier: whole matrices per owner, Newton-Schulz on the owner, broadcast).
Gradients are random. Every phase is timed with CUDA events on the launching stream (max over ranks); bytes are what
ONE rank receives over NVLink in that phase; the bandwidth is set against the measured 770 GB/s per direction.
One JSON line per phase and one for the whole step."""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist
import torch.nn as nn

PEER_GBS = 770.0


class Synthetic(nn.Module):
    def __init__(self, n_params: int, matrix_frac: float):
        super().__init__()
        n_mat = int(n_params * matrix_frac) // (1024 * 1024)
        n_vec = max(1, (n_params - n_mat * 1024 * 1024) // (4 << 20))
        self.vecs = nn.ParameterList([nn.Parameter(torch.randn(4 << 20) * 0.02) for _ in range(n_vec)])
        self.mats = nn.ParameterList([nn.Parameter(torch.randn(1024, 1024) * 0.02) for _ in range(n_mat)])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=float, default=100e6)
    ap.add_argument("--mode", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--multimem", type=int, default=-1, help="-1 or 0: plain peer loads and stores (the default); 1: multimem through the switch where supported")
    ap.add_argument("--matrix-frac", type=float, default=0.0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    from triune_b200.optim import CentroidSteerOptimizer
    from triune_b200.parallel import setup_distributed
    from triune_b200.parallel.data_parallel import ShardedDataParallel

    ctx = setup_distributed(backend="nccl")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    world, rank = ctx.world_size, ctx.rank
    torch.manual_seed(0)
    model = Synthetic(int(a.params), a.matrix_frac).to(dev, torch.bfloat16)
    dp = ShardedDataParallel(ctx, mode=a.mode, use_multimem=None if a.multimem < 0 else bool(a.multimem))
    opt = CentroidSteerOptimizer(model, lr=1e-4, grad_clip=1.0, muon_ns_steps=5, storage_factory=dp.storage_factory)
    dp.attach(opt)
    arena = opt.arena
    n = arena.total
    phases = ["reduce_scatter", "adamw_allgather", "matrix_tiers", "broadcast_barrier"] if dp._fused is not None else []
    acc = {p: 0.0 for p in phases}
    total = 0.0
    for it in range(a.warmup + a.iters):
        arena.flat_grad.normal_()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        evs = [torch.cuda.Event(enable_timing=True)]
        evs[0].record()

        def mark(_name):
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            evs.append(e)

        if dp._fused is not None:
            dp._fused.step(mark)
        else:
            opt.step()
            mark("all")
        torch.cuda.synchronize()
        if it >= a.warmup:
            for i, p in enumerate(phases):
                acc[p] += evs[i].elapsed_time(evs[i + 1])
            total += evs[0].elapsed_time(evs[-1])
    t = torch.tensor([total / a.iters] + [acc[p] / a.iters for p in phases], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    status = dp._fused.check() if dp._fused is not None else 0
    if rank == 0:
        f = (world - 1) / world
        n_mat = sum(p.numel() for p in model.mats)
        n_vec = n - n_mat
        recv = {"reduce_scatter": n * 4 * f, "adamw_allgather": n_vec * 2 * f, "broadcast_barrier": n_mat * 2 * f, "matrix_tiers": 0.0}
        base = {"n_gpus": world, "arena_params": n, "mode": a.mode if world > 1 else "local",
                "multimem": bool(dp._fused.buf.use_multimem) if dp._fused is not None else None, "wait_status": status}
        for i, p in enumerate(phases):
            ms = float(t[i + 1])
            gbs = recv[p] / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
            print(json.dumps(dict(base, phase=p, ms=ms, recv_bytes_per_rank=recv[p], gbs=gbs, frac_of_peer_copy=gbs / PEER_GBS)), flush=True)
        ms = float(t[0])
        nv = n * 4 * f + n * 2 * f if a.mode == "fused" else 2 * n * 4 * f
        print(json.dumps(dict(base, phase="whole step", ms=ms, nvlink_bytes_per_rank=nv, gbs=nv / (ms * 1e-3) / 1e9,
                              ideal_ms=nv / (PEER_GBS * 1e9) * 1e3)), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
