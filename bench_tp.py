"""Tensor-parallel training throughput of the dense model family: one rank per GPU; `--tp N` makes tensor-parallel
groups of N consecutive ranks (default: the whole world) with data parallelism across them (sequence-parallel rows
between blocks, heads and FFN width split over a group; one batch of `--batch` sequences per replica).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29560 \
        bench_tp.py --steps 5 --warmup 3

Default model: the dense 1.5B-class configuration (d = 2048, 24 layers, 16 x 128 Gated DeltaNet heads, SwiGLU 5632),
4 x 2048 tokens per step for the group. `--tp-mode fused` (default) runs the all-gather and the reduce-scatter inside
the GEMM kernels over NVLink; `--tp-mode nccl` uses library collectives around plain GEMMs. With replicas, `--dp-mode
fused` (default) averages gradients and updates through the NVLink data-parallel kernels over each replica group and
`--dp-mode nccl` through one NCCL all-reduce. The reference has no tensor
parallelism, so there is no reference arm. Prints one JSON line on rank 0 (device-timed, maximum over the ranks).
"""

from __future__ import annotations

import argparse
import json
import time

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="bench-dense-1.5b")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (smoke runs)")
    ap.add_argument("--mixer", default="", help="override the sequence mixer: gla or gated_deltanet")
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel size (default: the whole world); the rest is data parallel")
    ap.add_argument("--tp-mode", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--dp-mode", default="fused", choices=["fused", "nccl"],
                    help="replica averaging: the fused NVLink reduce-scatter + update + all-gather kernels, or one NCCL all-reduce")
    a = ap.parse_args()

    from triune_b200.config import ModelConfig, get_model_config
    from triune_b200.models.universal import UniversalDenseTransformer
    from triune_b200.optim import CentroidSteerOptimizer
    from triune_b200.parallel import setup_distributed
    from triune_b200.parallel.tensor_parallel import TPContext
    from triune_b200.parallel.tp_model import TensorParallelDense, average_grads_over_replicas, make_tp_dp_groups

    ctx = setup_distributed()
    dev, rank, world = ctx.device, ctx.rank, ctx.world_size
    cfg = get_model_config(a.model).to_dict()
    if a.layers:
        cfg["num_layers"] = a.layers
    if a.mixer:
        cfg["mixer"] = a.mixer
    cfg = ModelConfig.from_dict(cfg)
    torch.manual_seed(0)  # every rank builds the same full model, then keeps its shards
    t0 = time.time()
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            full = UniversalDenseTransformer.from_config(cfg)
    finally:
        torch.set_default_dtype(prev)
    full_params = full.num_parameters()
    tp_size = a.tp if a.tp > 0 else world
    tp_group, dp_group = make_tp_dp_groups(tp_size)
    replicas, replica = world // tp_size, rank // tp_size
    tp = TPContext(group=tp_group, mode=a.tp_mode)
    model = TensorParallelDense(full, tp)
    del full
    torch.cuda.empty_cache()
    local_params = sum(p.numel() for p in model.parameters())
    # data parallelism across the replicas (ranks holding the same shard): the fused kernels own the optimizer step
    dp = None
    if replicas > 1:
        from triune_b200.parallel.data_parallel import ShardedDataParallel

        dp = ShardedDataParallel(ctx, mode=a.dp_mode, group=dp_group)
        opt = CentroidSteerOptimizer(model, lr=1e-4, grad_clip=1.0, storage_factory=dp.storage_factory)
        dp.attach(opt)
    else:
        opt = CentroidSteerOptimizer(model, lr=1e-4, grad_clip=1.0)
    build_s = time.time() - t0

    # one batch per replica; the ranks of a tensor-parallel group read the same one
    host = torch.randint(0, cfg.vocab_size, (a.batch, a.seq + 1),
                         generator=torch.Generator().manual_seed(1234 + replica)).pin_memory()
    n_valid = a.batch * a.seq

    def step():
        ids = host.to(dev, non_blocking=True)  # the same batch on every rank of the group
        loss = model.forward_loss(ids[:, :-1], ids[:, 1:], n_valid=n_valid)
        loss.backward()
        model.allreduce_replicated_grads()
        opt.step()  # with replicas: gradient reduce-scatter + sharded update + parameter all-gather over the dp group
        opt.zero_grad()
        return loss

    for _ in range(a.warmup):
        loss = step()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total = model.reduce_loss(loss)
    dp_status = int(dp._fused.check()) if (dp is not None and dp._fused is not None) else 0
    status = torch.tensor([max(tp.check(), dp_status)], device=dev)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    mem = torch.tensor([torch.cuda.max_memory_allocated() / 2**30], device=dev)
    dist.all_reduce(mem, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({
            "metric": "tensor-parallel train tok/s (device-timed, max over ranks)",
            "value": a.batch * a.seq * replicas / float(ms) * 1e3, "unit": "tok/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": float(ms), "higher_is_better": True, "scaling": "strong", "dtype": "bf16",
            "data": "synthetic uniform-random token ids from pinned host memory, random-init weights",
            "config": {"model": a.model, "layers": cfg.num_layers, "hidden_dim": cfg.hidden_dim, "mixer": cfg.mixer,
                       "params_total": full_params, "params_per_rank": local_params, "global_batch": a.batch * replicas,
                       "seq_len": a.seq, "parallelism": f"tp{tp_size} x dp{replicas}", "tp_mode": a.tp_mode,
                       "dp_mode": a.dp_mode if replicas > 1 else "none", "cuda_graph": False},
            "wait_status": int(status), "peak_mem_GB": round(float(mem), 1), "build_s": round(build_s, 1),
            "final_loss": float(total), "impl": "triune_b200",
        }), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
