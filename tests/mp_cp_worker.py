"""Worker for the context-parallel GLA test (gloo): every rank holds one segment of the sequence; outputs, the final
state and the gradients must equal those of the whole-sequence recurrence."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triune_b200.ops import reference as ref  # noqa: E402
from triune_b200.parallel.context_parallel import cp_gla  # noqa: E402


def emulate_kernel_path():
    """Make the CPU operators look like the CUDA kernels to cp_gla: the local pass returns a state WITHOUT a gradient
    and the kernel-path branch (decay clamp, analytic state gradient) is taken."""
    import triune_b200.parallel.context_parallel as cpm

    orig = cpm.ops.gla

    def detached_state(*a, **kw):
        o, s = orig(*a, **kw)
        return o, s.detach()

    cpm.ops.gla = detached_state
    cpm._kernel_path = lambda *a: True


def main():
    emulate = os.environ.get("CP_EMULATE_KERNEL_STATE") == "1"
    if emulate:
        emulate_kernel_path()
    dist.init_process_group("gloo")
    r, w = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(11)  # the same full tensors on every rank
    B, Tl, H, dk, dv = 2, 40, 3, 16, 24
    T = Tl * w
    dt = torch.float64
    q = torch.randn(B, T, H, dk, dtype=dt) * 0.5
    k = torch.randn(B, T, H, dk, dtype=dt) * 0.5
    v = torch.randn(B, T, H, dv, dtype=dt)
    x = torch.nn.functional.logsigmoid(torch.randn(B, T, H, dk, dtype=dt) * 2)  # per-dimension log decays
    if emulate:
        x = x.clamp(min=-4.5)  # stay above the kernels' clamp so that the unclamped oracle applies
    s0 = torch.randn(B, H, dk, dv, dtype=dt) * 0.1
    do = torch.randn(B, T, H, dv, dtype=dt)
    full = [t.clone().requires_grad_(True) for t in (q, k, v, x)]
    o_ref, s_ref = ref.gla_recurrent(full[0], full[1], full[2], full[3], s0, 0.5)
    (o_ref * do).sum().backward()
    sl = slice(r * Tl, (r + 1) * Tl)
    seg = [t[:, sl].clone().requires_grad_(True) for t in (q, k, v, x)]
    o, s_end = cp_gla(seg[0], seg[1], seg[2], seg[3], scale=0.5, gate_logits=False, initial_state=s0)
    (o * do[:, sl]).sum().backward()
    out = {"rank": r, "out": float((o - o_ref[:, sl]).abs().max())}
    if r == w - 1:
        out["state"] = float((s_end - s_ref).abs().max())
    for name, a, b in zip(("dq", "dk", "dv", "dg"), seg, full):
        out[name] = float((a.grad - b.grad[:, sl]).abs().max())
    with torch.no_grad():  # the inference form (plain collectives)
        o2, _ = cp_gla(seg[0].detach(), seg[1].detach(), seg[2].detach(), seg[3].detach(), scale=0.5, gate_logits=False,
                       initial_state=s0)
    out["out_nograd"] = float((o2 - o_ref[:, sl]).abs().max())
    sys.stdout.write("\nRESULT " + json.dumps(out) + "\n")
    sys.stdout.flush()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
