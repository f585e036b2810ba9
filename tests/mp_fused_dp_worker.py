"""Worker for the multi-GPU tests (launched by torchrun from test_multi_gpu.py): fused NVLink data-parallel step
vs the NCCL all-reduce baseline, the metric all-reduce, and a bounded wait that is made to expire."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triune_b200 import _ext  # noqa: E402
from triune_b200.config import ModelConfig  # noqa: E402
from triune_b200.models import TriuneTransformer  # noqa: E402
from triune_b200.optim import CentroidSteerOptimizer  # noqa: E402
from triune_b200.parallel import setup_distributed  # noqa: E402
from triune_b200.parallel.data_parallel import ShardedDataParallel  # noqa: E402
from triune_b200.utils import place_model  # noqa: E402


def build(ctx, mode, use_multimem):
    torch.manual_seed(0)
    cfg = ModelConfig(vocab_size=2048, hidden_dim=128, num_layers=5, num_heads=2, head_dim=64, num_experts=8, top_k=2,
                      router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3, expert_hidden=256, dense_hidden=256)
    model = place_model(TriuneTransformer.from_config(cfg), ctx.device, torch.bfloat16)
    dp = ShardedDataParallel(ctx, mode=mode, use_multimem=use_multimem)
    opt = CentroidSteerOptimizer(model, lr=1e-3, rank=16, grad_clip=1.0, storage_factory=dp.storage_factory)
    dp.attach(opt)
    return model, opt, dp


def run(model, opt, ctx, steps=3):
    g = torch.Generator().manual_seed(100 + ctx.rank)
    losses = []
    for _ in range(steps):
        ids = torch.randint(0, 2048, (2, 129), generator=g).to(ctx.device)
        loss = model.forward_loss(ids[:, :-1], ids[:, 1:], 2, n_valid=256)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss))
    torch.cuda.synchronize()
    return losses


def main():
    ctx = setup_distributed()
    use_mm = os.environ.get("TRIUNE_TEST_MULTIMEM", "0") == "1"
    out = {"rank": ctx.rank}
    m_ref, o_ref, _ = build(ctx, "nccl", None)
    l_ref = run(m_ref, o_ref, ctx)
    m_f, o_f, dp_f = build(ctx, "fused", use_mm)
    l_f = run(m_f, o_f, ctx)
    out["status"] = dp_f._fused.check()
    dist.barrier()  # every rank has finished its last step: no signal may be outstanding
    out["signals_consumed"] = bool(all(dp_f._fused.audit().values()))
    out["multimem"] = bool(dp_f._fused.buf.use_multimem)
    pa, pb = o_ref.arena.flat_param.float(), o_f.arena.flat_param.float()
    out["max_param_diff"] = float((pa - pb).abs().max())
    out["param_scale"] = float(pa.abs().max())
    # every rank must hold identical parameters after the fused step
    mine = pb.double().sum().reshape(1)
    allv = [torch.zeros_like(mine) for _ in range(ctx.world_size)]
    dist.all_gather(allv, mine)
    out["ranks_agree"] = bool(all(float(v) == float(allv[0]) for v in allv))
    out["loss_ref"], out["loss_fused"] = l_ref, l_f
    # the routing statistics behind the update rule (selection biases, centroids) are averaged over the ranks
    stats = [getattr(m, n).detach().double().sum().reshape(1) for m in m_f.modules() if hasattr(m, "expert_bias")
             for n in ("expert_bias", "last_centroids") if torch.is_tensor(getattr(m, n, None))]
    sm = torch.cat(stats).sum().reshape(1) if stats else torch.zeros(1, device=ctx.device, dtype=torch.double)
    alls = [torch.zeros_like(sm) for _ in range(ctx.world_size)]
    dist.all_gather(alls, sm)
    out["stats_agree"] = bool(all(abs(float(v) - float(alls[0])) <= 1e-9 * max(1.0, abs(float(alls[0]))) for v in alls))
    # metric all-reduce piggy-backed on the signal protocol
    buf = dp_f._fused.buf
    e = _ext.ext()
    local = torch.tensor([1.0 + ctx.rank, 2.0, 0.5 * ctx.rank], device=ctx.device)
    red = torch.zeros(3, device=ctx.device)
    st = torch.zeros(1, device=ctx.device, dtype=torch.int32)
    rank, world, bufs, sigs, _ = buf.table()
    e.metric_allreduce(rank, world, bufs, sigs, buf.offset("metric"), local, red, 3, buf.next_epoch(), st)
    torch.cuda.synchronize()
    w = ctx.world_size
    out["metric_ok"] = bool(torch.allclose(red.cpu(), torch.tensor([w + w * (w - 1) / 2, 2.0 * w, 0.5 * w * (w - 1) / 2])))
    # failure detection: a wait on a flag nobody raises expires after 0.2 s and reports status 4; the context survives
    dist.barrier()
    st2 = torch.zeros(1, device=ctx.device, dtype=torch.int32)
    e.comm_wait_only(rank, world, bufs, sigs, 6, 1 << 30, int(0.2e9), st2)
    torch.cuda.synchronize()
    out["timeout_status"] = int(st2.item())
    out["context_alive"] = float((torch.ones(4, device=ctx.device) * 2).sum()) == 8.0
    dist.barrier()
    print("RESULT " + json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
