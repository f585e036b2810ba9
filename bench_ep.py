"""Expert-parallel training throughput: one rank per GPU, experts sharded over the ranks (EP = world size), everything
else replicated with data-parallel gradient averaging.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29540 \
        bench_ep.py --steps 5 --warmup 3

The default shape is the large MoE benchmark configuration: d = 1536, 24 layers, 64 experts (top-2, hidden 4096),
16 x 2048 tokens per GPU. Token rows travel to the expert owners and back inside the dispatch / combine kernels
(peer stores over NVLink, `triune_b200/parallel/expert_parallel.py`); `--ep-mode nccl` runs the same model with
`all_to_all_single` instead. `--layers` / `--experts` / `--hidden` shrink the model for a smoke run.

The reference has no expert parallelism (its experts are replicated under DDP), so there is no reference arm.
Prints one JSON line on rank 0: tokens per second over all GPUs, device-timed, maximum over the ranks.
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
    ap.add_argument("--model", default="bench-ep-moe")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--experts", type=int, default=0)
    ap.add_argument("--hidden", type=int, default=0, help="expert hidden width")
    ap.add_argument("--ep-mode", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--capacity-factor", type=float, default=1.5)
    ap.add_argument("--profile", action="store_true", help="after the timed steps, print rank 0's kernel table of one more step")
    a = ap.parse_args()

    from triune_b200.config import ModelConfig, get_model_config
    from triune_b200.models import TriuneTransformer
    from triune_b200.optim import CentroidSteerOptimizer
    from triune_b200.parallel import setup_distributed
    from triune_b200.parallel.expert_parallel import EPContext, allreduce_replicated_grads, shard_experts

    ctx = setup_distributed()
    dev, rank, world = ctx.device, ctx.rank, ctx.world_size
    cfg = get_model_config(a.model).to_dict()
    if a.layers:
        L = a.layers
        reflex = max(2, L // 4)
        cfg.update(num_layers=L, router_prefix_layers=1, reflex_exit_layer=reflex, limbic_exit_layer=max(reflex + 1, L // 2))
    if a.experts:
        cfg["num_experts"] = a.experts
    if a.hidden:
        cfg["expert_hidden"] = a.hidden
    cfg = ModelConfig.from_dict(cfg)
    assert cfg.num_experts % world == 0, "the number of experts must be a multiple of the number of ranks"

    # Every rank builds the same full model straight on its GPU in bf16 (same seed), then keeps its slice of the experts.
    torch.manual_seed(0)
    t0 = time.time()
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = TriuneTransformer.from_config(cfg)
    finally:
        torch.set_default_dtype(prev)
    full_params = sum(p.numel() for p in model.parameters())
    ep = EPContext(cfg.num_experts, mode=a.ep_mode, capacity_factor=a.capacity_factor)
    n_moe = shard_experts(model, ep)
    torch.cuda.empty_cache()
    local_params = sum(p.numel() for p in model.parameters())
    opt = CentroidSteerOptimizer(model, lr=1e-4, grad_clip=1.0)
    build_s = time.time() - t0

    gen = torch.Generator().manual_seed(1234 + rank)
    host = torch.randint(0, cfg.vocab_size, (a.batch, a.seq + 1), generator=gen).pin_memory()

    def step():
        ids = host.to(dev, non_blocking=True)
        out = model.forward_loss(ids[:, :-1], ids[:, 1:], force_depth=2)
        loss = out[0] if isinstance(out, tuple) else out
        loss.backward()
        allreduce_replicated_grads(model)
        opt.step()
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
    status = torch.tensor([ep.check()], device=dev)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    mem = torch.tensor([torch.cuda.max_memory_allocated() / 2**30], device=dev)
    dist.all_reduce(mem, op=dist.ReduceOp.MAX)
    if rank == 0:
        tokens = a.batch * a.seq * world
        print(json.dumps({
            "metric": "expert-parallel train tok/s (device-timed, max over ranks)",
            "value": tokens / float(ms) * 1e3, "unit": "tok/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": float(ms), "higher_is_better": True, "scaling": "weak", "dtype": "bf16",
            "data": "synthetic uniform-random token ids from pinned host memory, random-init weights",
            "config": {"model": a.model, "layers": cfg.num_layers, "hidden_dim": cfg.hidden_dim, "experts": cfg.num_experts,
                       "top_k": cfg.top_k, "expert_hidden": cfg.expert_hidden, "moe_layers": n_moe,
                       "params_total": full_params, "params_per_rank": local_params,
                       "global_batch": a.batch * world, "seq_len": a.seq, "parallelism": f"ep{world} x dp{world} (replicated part)",
                       "ep_mode": a.ep_mode, "capacity_factor": a.capacity_factor, "cuda_graph": False},
            "wait_status": int(status), "peak_mem_GB": round(float(mem), 1), "build_s": round(build_s, 1),
            "final_loss": float(loss.detach()), "impl": "triune_b200",
        }), flush=True)
    if a.profile:
        from torch.profiler import ProfilerActivity, profile

        dist.barrier()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        if rank == 0:
            print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=30, max_name_column_width=90), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
