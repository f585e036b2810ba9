"""Device-timed micro-benchmarks of the sm_100a kernels with roofline fractions.

    python -m triune_b200.bench_kernels --case gemm --m 8192 --n 8192 --k 8192
    python -m triune_b200.bench_kernels --case all

Each case warms up, flushes L2 between timed iterations (writes a 256 MB buffer), times with CUDA events and
reports achieved FLOP/s or bytes/s against the measured peaks in ``MEASURED_PEAKS.json`` at the repository
root when present (copy bandwidth and cuBLAS bf16 throughput measured on this machine pool), otherwise against
6.65 TB/s and 1.59 PFLOP/s. The same entry point, with ``--iters`` small, is what the ncu captures under
``profiles/`` run.
"""

from __future__ import annotations

import argparse
import json
import os
from typing import Callable, Dict

import torch


def peaks() -> Dict[str, float]:
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops"]), "src": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "src": "fallback"}


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.fill_(1)


def timeit(fn: Callable, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def report(name, ms, flops=0.0, nbytes=0.0):
    pk = peaks()
    out = {"case": name, "ms": round(ms, 4)}
    if flops:
        tf = flops / ms / 1e9
        out.update(tflops=round(tf, 1), frac_of_peak=round(tf / pk["tflops"], 3))
    if nbytes:
        gbs = nbytes / ms / 1e6
        out.update(gbs=round(gbs, 1), frac_of_hbm=round(gbs / pk["hbm_gbs"], 3))
    out["peaks"] = pk["src"]
    print(json.dumps(out), flush=True)
    return out


def case_gemm(a):
    from . import ops

    M, N, K = a.m, a.n, a.k
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: ops.gemm(A, B, C), a.iters, a.warmup)
    report(f"tc_gemm {M}x{N}x{K}", ms, flops=2.0 * M * N * K, nbytes=2.0 * (M * K + N * K + M * N))


def case_wgrad(a):
    from . import ops

    M, N, K = a.m, a.n, a.k  # dW[M,N] += dY[K,M]^T X[K,N]
    dY = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    X = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    dW = torch.zeros(M, N, device="cuda", dtype=torch.float32)
    ms = timeit(lambda: ops.gemm(dY, X, dW, a_mn=True, b_mn=True, accumulate=True), a.iters, a.warmup)
    report(f"tc_gemm wgrad split-K {M}x{N}x{K}", ms, flops=2.0 * M * N * K, nbytes=2.0 * K * (M + N) + 4.0 * M * N)


def case_gla(a):
    from . import ops

    B, T, H, D = a.batch, a.seq, a.heads, 64
    q, k, v, g = (torch.randn(B, T, H, D, device="cuda").to(torch.bfloat16).requires_grad_(True) for _ in range(4))
    out = None

    def fwd():
        nonlocal out
        out, _ = ops.gla(q, k, v, g, gate_logits=True)

    ms = timeit(fwd, a.iters, a.warmup)
    report(f"gla fwd B{B} T{T} H{H}", ms, nbytes=2.0 * 5 * B * T * H * D)
    do = torch.randn_like(out)

    def fb():
        o, _ = ops.gla(q, k, v, g, gate_logits=True)
        o.backward(do)

    ms2 = timeit(fb, a.iters, a.warmup)
    report(f"gla fwd+bwd B{B} T{T} H{H}", ms2, nbytes=2.0 * 14 * B * T * H * D)


def case_gdn(a):
    """Gated DeltaNet: the recurrence kernel (no gradient) and forward + backward of the chunk-parallel training form."""
    from . import ops

    B, T, H, D = a.batch, a.seq, a.heads, a.head_dim
    q, k, v, g = (torch.randn(B, T, H, D, device="cuda").to(torch.bfloat16) for _ in range(4))
    k = torch.nn.functional.normalize(k.float(), dim=-1).to(torch.bfloat16)
    beta = torch.rand(B, T, H, device="cuda")

    def infer():
        with torch.no_grad():
            ops.gated_deltanet(q, k, v, g, beta=beta, gate_logits=True)

    ms = timeit(infer, a.iters, a.warmup)
    report(f"gdn recurrent kernel B{B} T{T} H{H} D{D}", ms, nbytes=2.0 * 5 * B * T * H * D)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, g)]
    do = torch.randn_like(q)

    def train():
        o, _ = ops.gated_deltanet(*leaves, beta=beta, gate_logits=True)
        o.backward(do)
        for t in leaves:
            t.grad = None

    torch.cuda.reset_peak_memory_stats()
    ms2 = timeit(train, max(1, a.iters // 2), min(a.warmup, 2))
    out = report(f"gdn chunk-parallel fwd+bwd B{B} T{T} H{H} D{D}", ms2)
    print(json.dumps({"case": out["case"], "peak_mem_GB": round(torch.cuda.max_memory_allocated() / 2**30, 2)}), flush=True)


def case_swiglu(a):
    """SwiGLU feed-forward, forward + backward: the activation inside the GEMM epilogues against the same three GEMMs
    with stand-alone activation kernels between them (M tokens, K model width, N hidden width)."""
    from . import _ext, ops

    M, K, H = a.m, a.k, a.n
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w13 = (torch.randn(2 * H, K, device="cuda") * K ** -0.5).to(torch.bfloat16).requires_grad_(True)
    w2 = (torch.randn(K, H, device="cuda") * H ** -0.5).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(M, K, device="cuda").to(torch.bfloat16)

    def clear():
        for t in (x, w13, w2):
            t.grad = None

    def fused():
        ops.swiglu_mlp(x, w13, w2).backward(dy)
        clear()

    def unfused():
        gu = ops.linear(x, w13)
        ops.linear(ops.swiglu(gu[:, :H], gu[:, H:]), w2).backward(dy)
        clear()

    flops = 18.0 * M * K * H  # 3 products forward (2 M K H each ... gate, up, down) and twice that backward
    ms = timeit(fused, a.iters, a.warmup)
    report(f"swiglu ffn fwd+bwd, activation in GEMM epilogues M{M} K{K} H{H}", ms, flops=flops)
    ms2 = timeit(unfused, a.iters, a.warmup)
    report(f"swiglu ffn fwd+bwd, stand-alone activation kernels M{M} K{K} H{H}", ms2, flops=flops)
    print(json.dumps({"case": "swiglu", "pair_kernel_launches": int(_ext.ext().tc_gemm_pair_launches())}), flush=True)


def case_rmsnorm(a):
    from . import ops

    x = torch.randn(a.m, a.n, device="cuda").to(torch.bfloat16)
    w = torch.ones(a.n, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: ops.rmsnorm(x, w), a.iters, a.warmup)
    report(f"rmsnorm {a.m}x{a.n}", ms, nbytes=4.0 * a.m * a.n)


def case_ce(a):
    from . import _ext

    lg = torch.randn(a.m, a.n, device="cuda").to(torch.bfloat16)
    t = torch.randint(0, a.n, (a.m,), device="cuda")
    ms = timeit(lambda: _ext.ext().ce_fwd_bwd(lg, t, -100, 1.0 / a.m), a.iters, a.warmup)
    report(f"cross_entropy fwd+grad {a.m}x{a.n}", ms, nbytes=6.0 * a.m * a.n)


def case_mlp(a):
    """Dense FFN forward + backward: the GELU-epilogue GEMM, the GELU'-epilogue data-gradient GEMM, two weight-gradient
    GEMMs and the plain GEMMs, at the benchmark model's shapes (tokens x d -> hidden -> d)."""
    from . import ops

    M, d, H = a.m, a.k, a.n
    x = torch.randn(M, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w1 = (torch.randn(H, d, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b1 = torch.zeros(H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w2 = (torch.randn(d, H, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b2 = torch.zeros(d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(M, d, device="cuda", dtype=torch.bfloat16)

    def fb():
        for t in (x, w1, b1, w2, b2):
            t.grad = None
        ops.mlp_gelu(x, w1, b1, w2, b2).backward(g)

    ms = timeit(fb, a.iters, a.warmup)
    report(f"mlp_gelu fwd+bwd {M}x{d}x{H}", ms, flops=6.0 * 2.0 * M * d * H, nbytes=2.0 * M * (4 * d + 3 * H))


def case_moe_route(a):
    from . import ops

    N, E = a.m, a.n
    logits = torch.randn(N, E, device="cuda")
    bias = torch.zeros(E, device="cuda")
    ms = timeit(lambda: ops.moe_route_plan(logits, bias, 2, 1.0, int(N / E * 1.5)), a.iters, a.warmup)
    report(f"moe_route_plan N={N} E={E} k=2 (route + sort + plan)", ms, nbytes=4.0 * N * E + 2 * N * (8 + 4 + 8 + 4 + 1))


def case_fp8(a):
    from .ops import quant_cuda, reference as ref

    M, N, K = a.m, a.n, a.k
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    wq, ws = ref.fp8_block_quantize_weight(torch.randn(N, K, device="cuda") * 0.05)
    xq, xs = quant_cuda.fp8_quantize_act(x)
    ms = timeit(lambda: quant_cuda.fp8_block_gemm(xq, xs, wq, ws), a.iters, a.warmup)
    report(f"fp8_block_gemm {M}x{N}x{K}", ms, flops=2.0 * M * N * K, nbytes=1.0 * (M * K + N * K) + 2.0 * M * N)
    ms = timeit(lambda: quant_cuda.fp8_quantize_act(x), a.iters, a.warmup)
    report(f"fp8_quantize_act {M}x{K}", ms, nbytes=3.0 * M * K)
    # MXFP8: 1x32 power-of-two scales applied by the tensor core (no promotion out of TMEM per K block)
    w16 = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    wq8, wsf = quant_cuda.mxfp8_quantize(w16)
    xq8, xsf = quant_cuda.mxfp8_quantize(x)
    for tile in (128, 256):
        ms = timeit(lambda: quant_cuda.mxfp8_gemm(xq8, xsf, wq8, wsf, 1.0, tile), a.iters, a.warmup)
        report(f"mxfp8_gemm (block-scaled tcgen05, 128x{tile} tiles) {M}x{N}x{K}", ms, flops=2.0 * M * N * K,
               nbytes=1.03 * (M * K + N * K) + 2.0 * M * N)
    ms = timeit(lambda: quant_cuda.mxfp8_quantize(x), a.iters, a.warmup)
    report(f"mxfp8_quantize {M}x{K}", ms, nbytes=3.03 * M * K)
    ms = timeit(lambda: quant_cuda.mxfp8_linear(x, wq8, wsf, torch.bfloat16), a.iters, a.warmup)
    report(f"mxfp8 linear (quantise + GEMM) {M}x{N}x{K}", ms, flops=2.0 * M * N * K)
    from .ops import gemm
    ms = timeit(lambda: gemm(x, w16), a.iters, a.warmup)
    report(f"bf16 tcgen05 GEMM {M}x{N}x{K}", ms, flops=2.0 * M * N * K)


def case_nvfp4(a):
    from .ops import quant_cuda

    N, K = a.n, a.k
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    p, s, t = quant_cuda.nvfp4_quantize(w)
    x = torch.randn(1, K, device="cuda", dtype=torch.bfloat16)
    e = quant_cuda._ext.ext()
    ms = timeit(lambda: e.nvfp4_gemv(x, p, s, t), a.iters, a.warmup)
    report(f"nvfp4_gemv M=1 {N}x{K}", ms, nbytes=N * K * 0.5625)
    ms = timeit(lambda: quant_cuda.nvfp4_dequant(p, s, t), a.iters, a.warmup)
    report(f"nvfp4_dequant {N}x{K}", ms, nbytes=N * K * 2.5625)
    ms = timeit(lambda: quant_cuda.nvfp4_quantize(w), a.iters, a.warmup)
    report(f"nvfp4_quantize {N}x{K}", ms, nbytes=N * K * 4.5625)
    # prefill: E2M1 x E2M1 with block scales on the tensor core, against decoding the weights in front of the bf16 GEMM
    M = a.m
    xm = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    sfb = quant_cuda.nvfp4_block_scales(s, K)
    a_p, a_sf = quant_cuda.nvfp4_quantize_act(xm)
    for tile in (128, 256):
        ms = timeit(lambda: e.nvfp4_gemm(a_p, a_sf, p, sfb, 1.0, tile), a.iters, a.warmup)
        report(f"nvfp4_gemm (block-scaled tcgen05, 128x{tile} tiles) {M}x{N}x{K}", ms, flops=2.0 * M * N * K,
               nbytes=0.5625 * (M * K + N * K) + 2.0 * M * N)
    ms = timeit(lambda: quant_cuda.nvfp4_quantize_act(xm), a.iters, a.warmup)
    report(f"nvfp4_quantize_act {M}x{K}", ms, nbytes=2.5625 * M * K)
    ms = timeit(lambda: quant_cuda.nvfp4_w4a4_linear(xm, p, sfb, 1.0, False, torch.bfloat16), a.iters, a.warmup)
    report(f"nvfp4 W4A4 linear (quantise + GEMM) {M}x{N}x{K}", ms, flops=2.0 * M * N * K)
    ms = timeit(lambda: quant_cuda.nvfp4_linear(xm, p, s, t, torch.bfloat16), a.iters, a.warmup)
    report(f"nvfp4 W4A16 linear (decode + bf16 GEMM) {M}x{N}x{K}", ms, flops=2.0 * M * N * K)


def case_dp(a):
    """The two data-parallel step kernels on a world of ONE rank (a loop-back peer table: the rank's own buffer is its
    only peer), so their instruction and memory counters can be profiled without a second GPU waiting on a flag. The
    NVLink figures come from ``bench_dp.py`` on 2 and 8 GPUs."""
    import os

    import torch.distributed as dist

    from . import _ext
    from .parallel.symm import SymmetricBuffer

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29591")
    dev = torch.device("cuda", 0)
    if not dist.is_initialized():
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    n = (a.m * a.k) // 1024 * 1024  # parameters of the synthetic arena (default 8192 * 8192 = 67 M)
    buf = SymmetricBuffer({"param": n * 2, "grad": n * 4, "norm": 2 * 4 + 64}, dev, use_multimem=False)
    buf.view("grad", torch.float32, n).normal_()
    master = torch.randn(n, device=dev) * 0.02
    m1, v1 = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    counter = torch.zeros(1, device=dev, dtype=torch.int32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    clip, norm = torch.zeros(1, device=dev), torch.zeros(1, device=dev)
    e = _ext.ext()
    rank, world, bufs, sigs, mc = buf.table()
    goff, noff, poff = buf.offset("grad"), buf.offset("norm"), buf.offset("param")
    state = {"ep": 0}

    def rs():
        state["ep"] += 1
        e.dp_reduce_scatter(rank, world, bufs, sigs, mc, goff, noff, [0, n], state["ep"], False, counter, status, None)

    def ag():
        # the reduce-scatter of the same epoch publishes the norm partial this kernel waits for
        rs()
        e.dp_adamw_allgather(rank, world, bufs, sigs, mc, goff, noff, poff, 0, n, 0, master, m1, v1, 1e-4, 0.9, 0.95, 1e-8, 0.05,
                             state["ep"], 1.0, clip, norm, state["ep"], False, status, None, None)

    ms_rs = timeit(rs, a.iters, a.warmup)
    report(f"dp_reduce_scatter, one rank, {n} parameters", ms_rs, nbytes=8.0 * n)
    ms_both = timeit(ag, a.iters, a.warmup)
    report(f"dp_adamw_allgather, one rank, {n} parameters (time of the pair minus the reduce-scatter)", max(ms_both - ms_rs, 1e-6),
           nbytes=30.0 * n)
    print(json.dumps({"case": "dp", "wait_status": int(status.item())}))
    dist.destroy_process_group()


def case_tp(a):
    """The fused tensor-parallel GEMMs (all-gather -> GEMM with in-kernel fetch warps and chunk flags; GEMM ->
    reduce-scatter with TMA reduce-add into the owner's buffer) on a world of ONE rank, for profiler counters: the
    whole kernel runs (flags, bounded waits, the reduce-add epilogue), only the remote rows are missing. The NVLink
    figures come from the 2- and 8-GPU runs of ``tests/mp_tp_worker.py`` and ``bench_tp.py``."""
    import os

    import torch.distributed as dist

    from .parallel import tensor_parallel as tpm

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29592")
    dev = torch.device("cuda", 0)
    if not dist.is_initialized():
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    ctx = tpm.TPContext(device=dev, mode="fused")
    ctx.mode = "fused"  # a one-rank context falls back to plain GEMMs by default; here the fused kernels are the point
    M, N, K = a.m, a.n, a.k
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05
    ms = timeit(lambda: tpm._ag_gemm_fused(ctx, x, w, False), a.iters, a.warmup)
    report(f"all-gather GEMM (fused kernel, one rank) {M}x{N}x{K}", ms, flops=2.0 * M * N * K)
    ms = timeit(lambda: tpm._gemm_rs_fused(ctx, x, w, False), a.iters, a.warmup)
    report(f"GEMM reduce-scatter (fused kernel, one rank, incl. zero fill, two signal rounds and the copy out) {M}x{N}x{K}", ms,
           flops=2.0 * M * N * K)
    from .ops import gemm

    ms = timeit(lambda: gemm(x, w), a.iters, a.warmup)
    report(f"plain tcgen05 GEMM {M}x{N}x{K}", ms, flops=2.0 * M * N * K)
    print(json.dumps({"case": "tp", "wait_status": int(ctx.check())}))
    dist.destroy_process_group()


def case_small(a):
    """The small bandwidth- or latency-bound kernels that have no case of their own: rotary embedding, add + RMSNorm,
    the GLA decode step, the tier router, the heat map and tier-colour render, the steer update, the triangular AdamW on
    the subspace cores, Newton-Schulz on a batch of square matrices, the LoRA linear, the small-M NVFP4 product and the
    GGML block decoder. Each runs on its own; a failure is printed and the next one runs."""
    from . import _ext, ops
    from .ops import reference as ref

    e = _ext.ext()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    bf = lambda *shape: torch.randn(*shape, device=dev, dtype=torch.bfloat16, generator=g)
    f32 = lambda *shape: torch.randn(*shape, device=dev, dtype=torch.float32, generator=g)
    it = max(2, min(a.iters, 5))

    def run(name, build):
        try:
            fn, nbytes, flops = build()
            with torch.no_grad():
                report(name, timeit(fn, it, 2), flops=flops, nbytes=nbytes)
        except Exception as ex:  # keep going: every line of this case is independent
            print(json.dumps({"case": name, "error": f"{type(ex).__name__}: {ex}"[:200]}), flush=True)

    def rope():
        x = bf(32, 2048, 6, 64)
        cos, sin = ops.rope_tables(2048, 64, device=dev)
        return (lambda: ops.apply_rope(x, cos, sin)), 2 * x.numel() * 2, 0.0

    def add_norm():
        x, r, w = bf(32768, 2048), bf(32768, 2048), torch.ones(2048, device=dev, dtype=torch.bfloat16)
        return (lambda: ops.add_rmsnorm(x, r, w)), 4 * x.numel() * 2, 0.0

    def decode():
        q, k, v = bf(4, 1, 6, 64), bf(4, 1, 6, 64), bf(4, 1, 6, 64)
        gd = -torch.rand(4, 1, 6, 64, device=dev, generator=g).to(torch.bfloat16) * 0.1
        st = f32(4, 6, 64, 64)
        return (lambda: ops.gla(q, k, v, gd, initial_state=st)), 2 * st.numel() * 4, 0.0

    def tiers():
        lg = f32(65536, 3)
        return (lambda: ops.route_tiers(lg, 0.5)), lg.numel() * 4 + 65536 * 4, 0.0

    def heat():
        act = f32(8192 * 384)
        return (lambda: ops.neuron_heatmap(act, 64)), act.numel() * 4, 0.0

    def render():
        act, t = f32(8192, 1536), torch.randint(0, 3, (8192,), device=dev, generator=g)
        return (lambda: ops.tier_colour_render(act, t)), act.numel() * 8, 0.0

    def steer():
        P, G = f32(80, 257, 257), f32(80, 257, 257)
        return (lambda: ops.triangular_steer_update(P, G, 0.9, 0.18)), 3 * P.numel() * 4, 0.0

    def tri_adamw():
        S, m, v = f32(80, 257, 257), torch.zeros(80, 257, 257, device=dev), torch.zeros(80, 257, 257, device=dev)
        return (lambda: e.triangular_adamw(S, m, v, 0.9, 0.999, 1e-8, 3, True, None)), 6 * S.numel() * 4, 0.0

    def ns():
        G = bf(40, 384, 384)
        return (lambda: ops.muon_ns(G, 5)), 0.0, 40 * 5 * 3 * 2.0 * 384**3

    def lora():
        x, w, A, B = bf(8192, 2048), bf(2048, 2048) * 0.02, bf(16, 2048) * 0.02, bf(2048, 16) * 0.02
        return (lambda: ops.lora_linear(x, w, None, A, B, 2.0)), 0.0, 2.0 * 8192 * 2048 * (2048 + 32)

    def gemv():
        w = bf(4096, 4096) * 0.02
        packed, scales, ts = ops.nvfp4_quantize(w)
        x = bf(4, 4096)
        return (lambda: e.nvfp4_gemv(x, packed, scales, ts)), packed.numel() + scales.numel(), 0.0

    def ggml():
        # Q8_0: blocks of 32 values = one fp16 scale + 32 int8; 64 Mi values decoded to bf16
        n = 64 << 20
        raw = torch.randint(0, 255, (n // 32 * 34,), device=dev, dtype=torch.uint8, generator=g)
        return (lambda: e.ggml_dequant(raw, 8, n)), raw.numel() + n * 2, 0.0

    for name, b in (("rotary embedding 32x2048x6x64", rope), ("add + RMSNorm 32768x2048", add_norm), ("GLA decode step B=4 H=6", decode),
                    ("tier router 65536 rows", tiers), ("neuron heat map 3.1 M activations, 64 bins", heat), ("tier-colour render 8192x1536", render),
                    ("steer update 80x257x257", steer), ("triangular AdamW 80x257x257", tri_adamw), ("Newton-Schulz 5 steps, 40x384x384", ns),
                    ("LoRA linear 8192x2048x2048 r=16", lora), ("NVFP4 small-M product 4x4096x4096", gemv), ("GGML Q8_0 decode, 64 Mi values", ggml)):
        run(name, b)


CASES = {"small": case_small, "tp": case_tp, "dp": case_dp, "mlp": case_mlp, "moe_route": case_moe_route, "fp8": case_fp8, "nvfp4": case_nvfp4, "gemm": case_gemm, "wgrad": case_wgrad, "gla": case_gla, "gdn": case_gdn, "swiglu": case_swiglu, "rmsnorm": case_rmsnorm, "ce": case_ce}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=6)
    ap.add_argument("--head-dim", type=int, default=64, help="head dimension of the gdn case (64 or 128)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    if a.case != "all":
        CASES[a.case](a)
        return
    for (m, n, k) in ((8192, 8192, 8192), (32768, 1536, 384), (32768, 384, 1536), (32768, 32000, 384)):
        a.m, a.n, a.k = m, n, k
        case_gemm(a)
    for (m, n, k) in ((1536, 384, 32768), (384, 384, 32768), (32000, 384, 8192)):
        a.m, a.n, a.k = m, n, k
        case_wgrad(a)
    case_gla(a)
    a.m, a.n = 32768, 384
    case_rmsnorm(a)
    a.m, a.n = 8192, 32000
    case_ce(a)


if __name__ == "__main__":
    main()
