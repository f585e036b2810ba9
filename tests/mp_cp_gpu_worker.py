"""Worker for the context-parallel GLA test on GPUs (NCCL, the sm_100a kernels): every rank holds one segment of the
sequence; outputs, the final state and all gradients must equal those of the whole-sequence kernel pass on one GPU and
of the fp32 oracle."""

import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triune_b200 import ops  # noqa: E402
from triune_b200.ops import reference as ref  # noqa: E402
from triune_b200.parallel.context_parallel import cp_gla  # noqa: E402


def nrel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-12))


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    r, w = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(11)  # the same full tensors on every rank
    B, Tl, H, D = 2, 256, 3, 64
    T = Tl * w
    q = F.normalize(torch.randn(B, T, H, D, device=dev).abs(), dim=-1).to(torch.bfloat16)
    k = F.normalize(torch.randn(B, T, H, D, device=dev).abs(), dim=-1).to(torch.bfloat16)
    v = torch.randn(B, T, H, D, device=dev).to(torch.bfloat16)
    gx = torch.randn(B, T, H, D, device=dev).to(torch.bfloat16)
    s0 = torch.randn(B, H, D, D, device=dev) * 0.1
    do = torch.randn(B, T, H, D, device=dev)
    # whole sequence on this GPU through the kernels, and the fp32 oracle
    full = [t.clone().requires_grad_(True) for t in (q, k, v, gx)]
    o_k, s_k = ops.gla(*full, initial_state=s0, scale=0.5, gate_logits=True)
    (o_k.float() * do).sum().backward()
    f32 = [t.float().requires_grad_(True) for t in (q, k, v, gx)]
    o_ref, s_ref = ref.gla_chunk(f32[0], f32[1], f32[2], torch.clamp(F.logsigmoid(f32[3]), min=-5.0), s0, 0.5)
    (o_ref * do).sum().backward()
    sl = slice(r * Tl, (r + 1) * Tl)
    seg = [t[:, sl].clone().requires_grad_(True) for t in (q, k, v, gx)]
    o, s_end = cp_gla(seg[0], seg[1], seg[2], seg[3], scale=0.5, gate_logits=True, initial_state=s0)
    (o.float() * do[:, sl]).sum().backward()
    torch.cuda.synchronize()
    out = {"rank": r, "world": w, "out_vs_kernel": nrel(o, o_k[:, sl]), "out_vs_oracle": nrel(o, o_ref[:, sl])}
    if r == w - 1:
        out["state_vs_oracle"] = nrel(s_end, s_ref)
    for name, a, b, c in zip(("dq", "dk", "dv", "dg"), seg, full, f32):
        out[name + "_vs_kernel"] = nrel(a.grad, b.grad[:, sl])
        out[name + "_vs_oracle"] = nrel(a.grad, c.grad[:, sl])
    with torch.no_grad():
        o2, _ = cp_gla(seg[0].detach(), seg[1].detach(), seg[2].detach(), seg[3].detach(), scale=0.5, gate_logits=True,
                       initial_state=s0)
    out["out_nograd"] = nrel(o2, o_ref[:, sl])
    # timing of the forward + backward of one segment against the whole sequence on one GPU (CUDA events)
    def timed(fn, iters=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    def cp_step():
        oo, _ = cp_gla(seg[0], seg[1], seg[2], seg[3], scale=0.5, gate_logits=True, initial_state=s0)
        (oo.float() * do[:, sl]).sum().backward()

    def full_step():
        oo, _ = ops.gla(*full, initial_state=s0, scale=0.5, gate_logits=True)
        (oo.float() * do).sum().backward()

    out["ms_cp_segment"] = timed(cp_step)
    out["ms_whole_sequence"] = timed(full_step)
    sys.stdout.write("\nRESULT " + json.dumps(out) + "\n")
    sys.stdout.flush()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
