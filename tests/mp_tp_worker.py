"""Worker of the tensor-parallel GPU test: fused all-gather GEMM and GEMM reduce-scatter against fp32 PyTorch."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from triune_b200.parallel import setup_distributed
    from triune_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear, TPContext, ag_gemm, gemm_rs

    ctx = setup_distributed()
    dev, r, w = ctx.device, ctx.rank, ctx.world_size
    torch.manual_seed(0)  # identical "full" tensors on every rank
    M, K, N = 512 * w, 384, 768
    X = torch.randn(M, K, device=dev).bfloat16()
    W = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
    rows = M // w
    out = {"rank": r}
    for mode in ("fused", "nccl"):
        tp = TPContext(mode=mode, rs_fp32=False)
        # all-gather GEMM: column-parallel weight slice
        Wc = W[r * (N // w) : (r + 1) * (N // w)].contiguous()
        for it in range(3):  # repeated calls exercise the double-buffered workspace and the epochs
            y, gathered = ag_gemm(tp, X[r * rows : (r + 1) * rows].contiguous() * (it + 1), Wc)
            want = (X.float() * (it + 1)) @ Wc.float().t()
            err = ((y.float() - want).abs().max() / want.abs().max()).item()
            out[f"{mode}_ag_err"] = max(out.get(f"{mode}_ag_err", 0.0), err)
            out[f"{mode}_gather_ok"] = bool(torch.equal(gathered, X * (it + 1)))
        # GEMM reduce-scatter: row-parallel weight slice (reduction dimension split)
        Kp = K // w
        Wr = W[:, r * Kp : (r + 1) * Kp].contiguous()
        Xr = X[:, r * Kp : (r + 1) * Kp].contiguous()
        for it in range(3):
            y = gemm_rs(tp, Xr * (it + 1), Wr)
            want = ((X.float() * (it + 1)) @ W.float().t())[r * rows : (r + 1) * rows]
            err = ((y.float() - want).abs().max() / want.abs().max()).item()
            out[f"{mode}_rs_err"] = max(out.get(f"{mode}_rs_err", 0.0), err)
        # modules + autograd: column -> row block against the unsharded reference
        torch.manual_seed(1)
        W1 = (torch.randn(1024, K, device=dev) * 0.05).bfloat16()
        W2 = (torch.randn(K, 1024, device=dev) * 0.05).bfloat16()
        col, row = ColumnParallelLinear(K, 1024, tp), RowParallelLinear(1024, K, tp)
        with torch.no_grad():
            col.weight.copy_(W1[r * (1024 // w) : (r + 1) * (1024 // w)])
            row.weight.copy_(W2[:, r * (1024 // w) : (r + 1) * (1024 // w)])
        xs = X[r * rows : (r + 1) * rows].clone().requires_grad_(True)
        ys = row(torch.nn.functional.gelu(col(xs), approximate="tanh"))
        G = torch.randn(M, K, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).bfloat16()
        ys.backward(G[r * rows : (r + 1) * rows])
        Xf = X.float().requires_grad_(True)
        W1f, W2f = W1.float().requires_grad_(True), W2.float().requires_grad_(True)
        yf = torch.nn.functional.gelu(Xf @ W1f.t(), approximate="tanh") @ W2f.t()
        yf.backward(G.float())
        rel = lambda a, b: ((a.float() - b).abs().max() / b.abs().max().clamp_min(1e-9)).item()
        out[f"{mode}_mod_fwd"] = rel(ys, yf[r * rows : (r + 1) * rows])
        out[f"{mode}_mod_dx"] = rel(xs.grad, Xf.grad[r * rows : (r + 1) * rows])
        gw1 = col.weight.main_grad if hasattr(col.weight, "main_grad") else col.weight.grad
        gw2 = row.weight.main_grad if hasattr(row.weight, "main_grad") else row.weight.grad
        out[f"{mode}_mod_dw1"] = rel(gw1, W1f.grad[r * (1024 // w) : (r + 1) * (1024 // w)])
        out[f"{mode}_mod_dw2"] = rel(gw2, W2f.grad[:, r * (1024 // w) : (r + 1) * (1024 // w)])
        out[f"{mode}_status"] = tp.check()
        if mode == "fused":
            # device-timed comparison on a shape where the collective matters
            Mb, Kb, Nb = 8192 * w, 2048, 2560
            Xb = torch.randn(Mb // w, Kb, device=dev).bfloat16()
            Wb = (torch.randn(Nb, Kb, device=dev) * 0.02).bfloat16()
            tn = TPContext(mode="nccl")
            for name, c in (("fused", tp), ("nccl", tn)):
                for _ in range(3):
                    ag_gemm(c, Xb, Wb)
                torch.cuda.synchronize(); dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(10):
                    ag_gemm(c, Xb, Wb)
                e1.record(); torch.cuda.synchronize()
                out[f"ag_ms_{name}"] = e0.elapsed_time(e1) / 10
            Xp = torch.randn(Mb, Kb // w, device=dev).bfloat16()
            Wp = (torch.randn(Nb, Kb // w, device=dev) * 0.02).bfloat16()
            for name, c in (("fused", tp), ("nccl", tn)):
                for _ in range(3):
                    gemm_rs(c, Xp, Wp)
                torch.cuda.synchronize(); dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(10):
                    gemm_rs(c, Xp, Wp)
                e1.record(); torch.cuda.synchronize()
                out[f"rs_ms_{name}"] = e0.elapsed_time(e1) / 10
            out["fused_status_after_bench"] = tp.check()
    sys.stdout.write("\nRESULT " + json.dumps(out) + "\n")
    sys.stdout.flush()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
