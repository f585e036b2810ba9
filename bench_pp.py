"""Pipeline-parallel training throughput of the dense model family: one rank per GPU; `--pp N` makes pipelines of N
consecutive ranks (default: the whole world) with data parallelism across them. Each pipeline runs `--batch` sequences
per step as `--micro` micro-batches under the one-forward-one-backward schedule.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29570 \
        bench_pp.py --steps 5 --warmup 3

Default model: the dense 1.5B-class configuration with the GLA mixer, 16 x 2048 tokens per pipeline and step in 8
micro-batches. Boundary activations travel by NCCL send / recv. The reference has no pipeline parallelism, so there is
no reference arm. Prints one JSON line on rank 0 (device-timed on GPUs, wall clock on CPU; maximum over the ranks).
Without a GPU the same script runs on gloo (use a small `--model` / `--layers`), which is how the CPU tests drive it.
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
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--micro", type=int, default=8, help="micro-batches per step")
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (smoke runs)")
    ap.add_argument("--mixer", default="gla", help="sequence mixer: gla or gated_deltanet")
    ap.add_argument("--family", default="dense", choices=["dense", "triune"],
                    help="dense: UniversalDenseTransformer; triune: the multi-exit MoE model at full depth (tied embedding)")
    ap.add_argument("--pp", type=int, default=0, help="pipeline size (default: the whole world); the rest is data parallel")
    ap.add_argument("--head-weight", type=float, default=1.0,
                    help="relative cost of the last stage (> 1 gives it fewer blocks, because it also runs the vocabulary head)")
    a = ap.parse_args()

    from triune_b200.config import ModelConfig, get_model_config
    from triune_b200.models.universal import UniversalDenseTransformer
    from triune_b200.optim import CentroidSteerOptimizer
    from triune_b200.parallel import setup_distributed
    from triune_b200.models import TriuneTransformer
    from triune_b200.parallel.pipeline import PipelineEngine, PipelineStage, TriunePipelineStage, make_pp_dp_groups, split_layers
    from triune_b200.parallel.tp_model import average_grads_over_replicas

    ctx = setup_distributed()
    dev, rank, world = ctx.device, ctx.rank, ctx.world_size
    cuda = dev.type == "cuda"
    cfg = get_model_config(a.model).to_dict()
    if a.layers:
        cfg["num_layers"] = a.layers
    if a.family == "dense":
        cfg.update(mixer=a.mixer, tie_embeddings=False)
    elif a.layers:
        reflex = max(2, a.layers // 4)
        cfg.update(router_prefix_layers=1, reflex_exit_layer=reflex, limbic_exit_layer=max(reflex + 1, a.layers // 2))
    cfg = ModelConfig.from_dict(cfg)
    pp = a.pp if a.pp > 0 else world
    pp_group, dp_group = make_pp_dp_groups(pp)
    replicas, replica, stage_idx = world // pp, rank // pp, rank % pp
    weights = None if a.head_weight == 1.0 or pp == 1 else [1.0] * (pp - 1) + [a.head_weight]
    bounds = split_layers(cfg.num_layers, pp, weights)

    torch.manual_seed(0)  # every rank builds the same full model, then keeps its stage
    t0 = time.time()
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16 if cuda else torch.float32)
    try:
        with torch.device(dev):
            full = (UniversalDenseTransformer if a.family == "dense" else TriuneTransformer).from_config(cfg)
    finally:
        torch.set_default_dtype(prev)
    full_params = full.num_parameters()
    stage = (PipelineStage if a.family == "dense" else TriunePipelineStage)(full, stage_idx, pp, bounds)
    del full
    if cuda:
        torch.cuda.empty_cache()
    eng = PipelineEngine(stage, a.micro, pp_group)
    local_params = sum(p.numel() for p in stage.parameters())
    opt = CentroidSteerOptimizer(stage, lr=1e-4, grad_clip=0.0)  # clipping by the whole model's norm happens in the engine
    build_s = time.time() - t0

    host = torch.randint(0, cfg.vocab_size, (a.batch, a.seq + 1), generator=torch.Generator().manual_seed(1234 + replica))
    if cuda:
        host = host.pin_memory()

    def step():
        ids = host.to(dev, non_blocking=True)
        loss = eng.train_step(ids[:, :-1], ids[:, 1:], n_valid=(a.batch // a.micro) * a.seq)
        average_grads_over_replicas(stage, dp_group)
        eng.clip_grad_norm(1.0)
        opt.step()
        opt.zero_grad()
        return loss

    def sync():
        if cuda:
            torch.cuda.synchronize()
        dist.barrier()

    for _ in range(a.warmup):
        loss = step()
    sync()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    w0 = time.perf_counter()
    for _ in range(a.steps):
        loss = step()
    if cuda:
        e1.record()
    sync()
    per_step = (e0.elapsed_time(e1) if cuda else (time.perf_counter() - w0) * 1e3) / a.steps
    ms = torch.tensor([per_step], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    mem = torch.tensor([torch.cuda.max_memory_allocated() / 2**30 if cuda else 0.0], device=dev)
    dist.all_reduce(mem, op=dist.ReduceOp.MAX)
    if rank == 0:
        bubble = (pp - 1) / (a.micro + pp - 1)
        print(json.dumps({
            "metric": "pipeline-parallel train tok/s (max over ranks)",
            "value": a.batch * a.seq * replicas / float(ms) * 1e3, "unit": "tok/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": float(ms), "higher_is_better": True, "scaling": "strong",
            "dtype": "bf16" if cuda else "fp32", "timer": "cuda events" if cuda else "wall clock (cpu)",
            "data": "synthetic uniform-random token ids, random-init weights",
            "config": {"model": a.model, "layers": cfg.num_layers, "stage_layers": bounds, "hidden_dim": cfg.hidden_dim,
                       "family": a.family, "mixer": cfg.mixer if a.family == "dense" else "gla", "params_total": full_params, "params_rank0": local_params,
                       "global_batch": a.batch * replicas, "micro_batches": a.micro, "seq_len": a.seq,
                       "parallelism": f"pp{pp} x dp{replicas}", "schedule": "1F1B", "ideal_bubble_fraction": round(bubble, 3),
                       "cuda_graph": False},
            "peak_mem_GB": round(float(mem), 1), "build_s": round(build_s, 1), "final_loss": float(loss),
            "impl": "triune_b200",
        }), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
