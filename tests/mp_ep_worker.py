"""Worker of the expert-parallel GPU test: fused NVLink dispatch / combine against an fp32 PyTorch reference."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def reference(X, idx, wts, W1, B1, W2, B2):
    """All tokens of all ranks, every expert, fp32."""
    out = torch.zeros_like(X)
    for e in range(W1.shape[0]):
        sel = idx == e
        tok = sel.any(-1).nonzero(as_tuple=True)[0]
        if tok.numel() == 0:
            continue
        we = (wts * sel)[tok].sum(-1, keepdim=True)
        h = torch.nn.functional.gelu(X[tok] @ W1[e].t() + B1[e], approximate="tanh")
        out = out.index_add(0, tok, (h @ W2[e].t() + B2[e]) * we)
    return out


def main():
    from triune_b200.parallel import setup_distributed
    from triune_b200.parallel.expert_parallel import EPContext, ep_experts

    ctx = setup_distributed()
    dev, r, w = ctx.device, ctx.rank, ctx.world_size
    E, d, H, T, K = 8, 128, 256, 512, 2
    El = E // w
    g = torch.Generator(device=dev).manual_seed(0)
    W1 = torch.randn(E, H, d, device=dev, generator=g) * 0.05
    B1 = torch.randn(E, H, device=dev, generator=g) * 0.05
    W2 = torch.randn(E, d, H, device=dev, generator=g) * 0.05
    B2 = torch.randn(E, d, device=dev, generator=g) * 0.05
    Xall = torch.randn(w * T, d, device=dev, generator=g)
    logits = torch.randn(w * T, E, device=dev, generator=g)
    wall, iall = torch.softmax(logits, -1).topk(K, -1)
    wall = wall / wall.sum(-1, keepdim=True)
    Gall = torch.randn(w * T, d, device=dev, generator=g)
    out = {"rank": r}
    # fp32 reference over every token
    Xf = Xall.bfloat16().float().requires_grad_(True)
    wf = wall.clone().requires_grad_(True)
    ps = [p.bfloat16().float().requires_grad_(True) for p in (W1, B1, W2, B2)]
    yf = reference(Xf, iall, wf, *ps)
    yf.backward(Gall.bfloat16().float())
    sl = slice(r * T, (r + 1) * T)
    es = slice(r * El, (r + 1) * El)
    for mode in ("fused", "nccl"):
        ep = EPContext(E, mode=mode, capacity_factor=2.0)
        x = Xall[sl].bfloat16().clone().requires_grad_(True)
        wt = wall[sl].clone().requires_grad_(True)
        lw = [p[es].bfloat16().clone().requires_grad_(True) for p in (W1, B1, W2, B2)]
        for it in range(2):  # second pass reuses the workspaces and epochs
            for t in [x, wt] + lw:
                t.grad = None
            y = ep_experts(x, iall[sl].contiguous(), wt, lw[0], lw[1], lw[2], lw[3], ep)
            if mode == "fused":
                y.backward(Gall[sl].bfloat16())
        rel = lambda a, b: ((a.float() - b).abs().max() / b.abs().max().clamp_min(1e-9)).item()
        out[f"{mode}_fwd"] = rel(y, yf[sl])
        if mode == "fused":
            out["dx"] = rel(x.grad, Xf.grad[sl])
            out["dwts"] = rel(wt.grad, wf.grad[sl])
            for name, a, b in zip(("dw1", "db1", "dw2", "db2"), lw, ps):
                out[name] = rel(a.grad, b.grad[es])
        out[f"{mode}_status"] = ep.check()
    # capacity overflow: every token to expert 0 with a tight capacity must drop rows without faulting
    ep = EPContext(E, mode="fused", capacity_factor=0.25)
    idx0 = torch.zeros(T, K, dtype=torch.int64, device=dev)
    idx0[:, 1] = 1
    y = ep_experts(Xall[sl].bfloat16(), idx0, wall[sl].contiguous(), *[p[es].bfloat16() for p in (W1, B1, W2, B2)], ep)
    out["overflow_finite"] = bool(torch.isfinite(y.float()).all())
    out["overflow_dropped"] = int((y.float().abs().sum(-1) == 0).sum())
    out["overflow_status"] = ep.check()
    # model level: an expert-sharded TriuneTransformer computes what the unsharded model computes
    from triune_b200.config import ModelConfig
    from triune_b200.models import TriuneTransformer
    from triune_b200.parallel.expert_parallel import allreduce_replicated_grads, shard_experts
    from triune_b200.utils import place_model

    torch.manual_seed(3)
    cfg = ModelConfig(vocab_size=512, hidden_dim=128, num_layers=5, num_heads=2, head_dim=64, num_experts=8, top_k=2,
                      router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3, expert_hidden=256, dense_hidden=256)
    full = place_model(TriuneTransformer.from_config(cfg), dev, torch.bfloat16).eval()
    import copy

    sharded = copy.deepcopy(full)
    ep_m = EPContext(8, mode="fused", capacity_factor=4.0)
    out["model_layers_sharded"] = shard_experts(sharded, ep_m)
    tok = torch.randint(0, 512, (2, 128), device=dev, generator=torch.Generator(device=dev).manual_seed(10 + r))
    with torch.no_grad():
        a = full(tok, force_depth=2)[0].float()
        b = sharded(tok, force_depth=2)[0].float()
    out["model_fwd"] = ((a - b).abs().max() / a.abs().max()).item()
    out["model_fwd_mean"] = ((a - b).abs().mean() / a.abs().mean()).item()
    moe_full, moe_ep = full.layers[3].ffn, sharded.layers[3].ffn
    xin = torch.randn(2, 128, 128, device=dev, generator=torch.Generator(device=dev).manual_seed(20 + r)).bfloat16()
    with torch.no_grad():
        ya, yb = moe_full(xin).float(), moe_ep(xin).float()
    out["layer_fwd"] = ((ya - yb).abs().max() / ya.abs().max()).item()
    sharded.train()
    loss = sharded.forward_loss(tok, tok, force_depth=2)
    loss = loss[0] if isinstance(loss, tuple) else loss
    loss.backward()
    allreduce_replicated_grads(sharded)
    out["model_loss_finite"] = bool(torch.isfinite(loss))
    out["model_status"] = ep_m.check()
    sys.stdout.write("\nRESULT " + json.dumps(out) + "\n")
    sys.stdout.flush()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
