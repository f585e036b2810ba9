"""The reference's published micro-benchmarks at their published shapes, both arms on the same GPU.

    python bench_micro.py                       # every case, both arms, one JSON line per measurement
    python bench_micro.py --only exits,moe      # a subset
    python bench_micro.py --impl ours           # one arm

The reference publishes laptop-GPU numbers for a list of small workloads (its ``benchmarks/*.md`` reports): the
forward latency of the three exits, prefill at several lengths, sequential decode, the sparse MoE layer against the
dense evaluation of all experts, the chunked linear + cross entropy, RMSNorm, SwiGLU, the NVFP4 linear layer, one GLA
layer against softmax attention at long context, and the optimizer step. This script times each of them at the shape
the report names, with this framework ("ours") and with the unmodified reference installed under ``baseline/_ref``
("reference") when it is there, so the two can be compared on one box instead of across hardware. Timing: CUDA
events around ``iters`` calls after 3 warm-up calls, a 256 MB write between timed calls to clear the L2 cache, median
reported. Every case stands alone: a failure is recorded as a line of its own and the run carries on.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
VOCAB = 32000
_FLUSH = None


def timed(fn, iters: int = 10, warmup: int = 3) -> float:
    """Median milliseconds of ``fn()`` over ``iters`` calls, L2 flushed before each."""
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _FLUSH.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def emit(**kw):
    print(json.dumps(kw), flush=True)


def guarded(case: str, impl: str):
    def deco(fn):
        def run(*a, **k):
            try:
                return fn(*a, **k)
            except Exception as e:  # one case must not end the run
                emit(case=case, impl=impl, error=f"{type(e).__name__}: {e}"[:300])
            finally:
                torch.cuda.empty_cache()
        return run
    return deco


# ---------------------------------------------------------------------------------------------------- the two model arms
def ours_model(vocab=VOCAB, **over):
    from triune_b200.config import get_model_config
    from triune_b200.models import TriuneTransformer
    from triune_b200.utils import place_model

    cfg = get_model_config("bench-90m")
    for k, v in dict(vocab_size=vocab, **over).items():
        setattr(cfg, k, v)
    torch.manual_seed(0)
    return place_model(TriuneTransformer.from_config(cfg), torch.device("cuda"), torch.bfloat16).eval()


_REF = {}


def ref_modules():
    """The reference's modules with the benchmark configuration (top-2 of 8 experts, expert hidden 4 d); None when absent."""
    if "mods" in _REF:
        return _REF["mods"]
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    mods = None
    if os.path.isdir(os.path.join(ref_dir, "triune")):
        try:
            sys.path.insert(0, ref_dir)
            import triune.model.config as rc

            rc.TOP_K_EXPERTS, rc.EXPERT_HIDDEN_MULTIPLIER = 2, 4
            import triune.model.moe as rmoe
            from triune.model.transformer import TriuneTransformer as RefModel

            rmoe.EXPERT_HIDDEN_MULTIPLIER, rmoe.TOP_K_EXPERTS = 4, 2
            mods = {"moe": rmoe, "Model": RefModel}
        except Exception as e:
            emit(impl="reference", unavailable=f"import failed: {type(e).__name__}: {e}"[:300])
    else:
        emit(impl="reference", unavailable="baseline/_ref is not installed")
    _REF["mods"] = mods
    return mods


def ref_model(vocab=VOCAB):
    m = ref_modules()
    torch.manual_seed(0)
    model = m["Model"](vocab_size=vocab, hidden_dim=384, num_layers=8, num_heads=6, head_dim=64, num_experts=8, router_prefix_layers=1,
                       reflex_exit_layer=2, limbic_exit_layer=5).to(device="cuda", dtype=torch.bfloat16).eval()
    for mod in model.modules():
        if isinstance(mod, m["moe"].MoE_FFN):
            mod.top_k = 2
    return model


def model_forward(model, impl):
    if impl == "ours":
        def fwd(ids, depth):
            with torch.no_grad():
                return model(ids, force_depth=depth, last_token_only=True)
    else:
        def fwd(ids, depth):
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                return model(ids, force_depth=depth, cache=model.init_cache(ids.shape[0]), last_token_only=True)
    return fwd


# ---------------------------------------------------------------------------------------------------- cases
def case_exits(impl, a):
    """Forward latency of the three exits, B=4 T=512 (published: 2.76 / 8.25 / 11.90 ms)."""
    model = ours_model() if impl == "ours" else ref_model()
    fwd = model_forward(model, impl)
    ids = torch.randint(0, VOCAB, (4, 512), device="cuda")
    for depth, name in enumerate(("reflex", "limbic", "cortex")):
        ms = timed(lambda: fwd(ids, depth), a.iters)
        emit(case="exit latency B=4 T=512", impl=impl, exit=name, ms=ms, tok_s=4 * 512 / ms * 1e3)


def case_prefill(impl, a):
    """Full-depth prefill at the published batch / length pairs."""
    model = ours_model() if impl == "ours" else ref_model()
    fwd = model_forward(model, impl)
    for B, T in ((1, 2048), (1, 8192), (1, 16384), (4, 16384), (32, 1024)):
        ids = torch.randint(0, VOCAB, (B, T), device="cuda")
        torch.cuda.reset_peak_memory_stats()
        ms = timed(lambda: fwd(ids, 2), max(3, a.iters // 2))
        emit(case=f"prefill B={B} T={T}", impl=impl, ms=ms, tok_s=B * T / ms * 1e3, peak_mb=torch.cuda.max_memory_allocated() / 2**20)


def case_decode(impl, a):
    """Sequential greedy decode, prompt 64, 64 new tokens (published: 157 tok/s)."""
    prompt = torch.randint(0, VOCAB, (1, 64), device="cuda")
    if impl == "ours":
        from triune_b200.inference import GraphedGreedyDecoder

        model = ours_model()

        def eager():
            with torch.no_grad():
                cache = model.init_cache(1)
                logits, cache = model(prompt, force_depth=2, cache=cache, last_token_only=True)
                for _ in range(64):
                    logits, cache = model(logits[:, -1].argmax(-1, keepdim=True), force_depth=2, cache=cache, last_token_only=True)

        ms = timed(eager, 3, 1)
        emit(case="decode prompt 64 + 64 new", impl=impl, variant="eager loop", ms=ms, tok_s=64 / ms * 1e3, ms_per_token=ms / 64)
        dec = GraphedGreedyDecoder(model, batch_size=1, decode_depth=2)

        def graphed():
            dec.prefill(prompt)
            return dec.decode(64)

        ms = timed(graphed, 3, 1)
        emit(case="decode prompt 64 + 64 new", impl=impl, variant="graph-replayed step", ms=ms, tok_s=64 / ms * 1e3, ms_per_token=ms / 64)
    else:
        model = ref_model()

        def loop():
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                cache = model.init_cache(1)
                logits, cache = model(prompt, force_depth=2, cache=cache, last_token_only=True)
                for _ in range(64):
                    logits, cache = model(logits[:, -1].argmax(-1, keepdim=True), force_depth=2, cache=cache, last_token_only=True)

        ms = timed(loop, 3, 1)
        emit(case="decode prompt 64 + 64 new", impl=impl, variant="eager loop", ms=ms, tok_s=64 / ms * 1e3, ms_per_token=ms / 64)


def case_moe(impl, a):
    """One MoE layer, d=384 E=8 k=2: routed (sparse) evaluation against all experts on all tokens (published at N=4096:
    1.99 ms against 14.957 ms; at N=1: 0.719 against 1.185 ms)."""
    torch.manual_seed(0)
    if impl == "ours":
        from triune_b200.models.moe import MoE_FFN

        layer = MoE_FFN(384, 8, 2, expert_hidden=1536).to("cuda", torch.bfloat16).eval()
    else:
        layer = ref_modules()["moe"].MoE_FFN(384, num_experts=8, top_k=2).to("cuda", torch.bfloat16).eval()
        layer.top_k = 2
    for N in (4096, 1):
        x = torch.randn(1, N, 384, device="cuda", dtype=torch.bfloat16)

        def sparse():
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16, enabled=impl != "ours"):
                return layer(x)

        ms = timed(sparse, a.iters)
        rec = dict(case=f"MoE layer d=384 E=8 k=2 N={N}", impl=impl, variant="routed (sparse)", ms=ms)
        if impl == "ours":
            def dense():  # every expert on every token, mixed by the full softmax: what routing saves
                with torch.no_grad():
                    h = x.reshape(-1, 384)
                    w1, b1, w2, b2 = layer.w1, layer.b1, layer.w2, layer.b2
                    hid = torch.nn.functional.gelu(torch.einsum("nd,ehd->enh", h, w1) + b1[:, None], approximate="tanh")
                    return torch.einsum("enh,edh->end", hid, w2) + b2[:, None]

            try:
                rec["dense_all_experts_ms"] = timed(dense, a.iters)
            except Exception as e:
                rec["dense_all_experts_error"] = f"{type(e).__name__}: {e}"[:120]
        emit(**rec)


def case_ce(impl, a):
    """Linear head + cross entropy without the full logits, V=32000 N=8192 d=384, forward and backward (published: 22.97 ms,
    60.7 MB; PyTorch 59.04 ms, 4000 MB)."""
    torch.manual_seed(0)
    h = torch.randn(8192, 384, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(VOCAB, 384, device="cuda", dtype=torch.bfloat16) * 0.02).requires_grad_(True)
    y = torch.randint(0, VOCAB, (8192,), device="cuda")
    if impl == "ours":
        from triune_b200 import ops

        def step():
            h.grad = w.grad = None
            ops.linear_cross_entropy(h, w, y).backward()
    else:
        ref_modules()
        from triune.kernels.fast_cross_entropy import chunked_cross_entropy_from_hidden

        def step():
            h.grad = w.grad = None
            chunked_cross_entropy_from_hidden(h, w, y, chunk_size=1024, force_chunked=True).backward()

    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    ms = timed(step, a.iters)
    emit(case="linear + CE fwd+bwd V=32000 N=8192 d=384", impl=impl, ms=ms, extra_peak_mb=(torch.cuda.max_memory_allocated() - base) / 2**20)

    def plain():
        h.grad = w.grad = None
        torch.nn.functional.cross_entropy((h @ w.t()).float(), y).backward()

    if impl == "ours":
        torch.cuda.reset_peak_memory_stats()
        ms = timed(plain, a.iters)
        emit(case="linear + CE fwd+bwd V=32000 N=8192 d=384", impl="pytorch", ms=ms, extra_peak_mb=(torch.cuda.max_memory_allocated() - base) / 2**20)


def case_rows(impl, a):
    """RMSNorm 4 x 1024 x 2048 and SwiGLU 4 x 1024 x 4096 forward (published: 0.349 ms; 1.123 ms)."""
    x = torch.randn(4, 1024, 2048, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(2048, device="cuda", dtype=torch.bfloat16)
    g, u = (torch.randn(4, 1024, 4096, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    if impl == "ours":
        from triune_b200 import ops

        norm, act = (lambda: ops.rmsnorm(x, w, 1e-6)), (lambda: ops.swiglu(g, u))
    else:
        ref_modules()
        from triune.kernels.fast_rmsnorm import fast_rmsnorm
        from triune.kernels.fast_swiglu import fast_swiglu

        norm, act = (lambda: fast_rmsnorm(x, w, 1e-6)), (lambda: fast_swiglu(g, u))
    with torch.no_grad():
        ms = timed(norm, a.iters * 2)
        emit(case="RMSNorm 4x1024x2048", impl=impl, ms=ms, gb_s=2 * x.numel() * 2 / ms / 1e6)
        ms = timed(act, a.iters * 2)
        emit(case="SwiGLU 4x1024x4096", impl=impl, ms=ms, gb_s=3 * g.numel() * 2 / ms / 1e6)
        if impl == "ours":
            emit(case="RMSNorm 4x1024x2048", impl="pytorch", ms=timed(lambda: torch.nn.functional.rms_norm(x, (2048,), w, 1e-6), a.iters * 2))
            emit(case="SwiGLU 4x1024x4096", impl="pytorch", ms=timed(lambda: torch.nn.functional.silu(g) * u, a.iters * 2))


def case_nvfp4(impl, a):
    """NVFP4 linear layer 4096 x 4096 on 4096 rows (published: 0.99 ms, 10.0 MB, cosine 0.99503 to the bf16 layer)."""
    torch.manual_seed(0)
    lin = torch.nn.Linear(4096, 4096, bias=False).to("cuda", torch.bfloat16)
    x = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
    if impl == "ours":
        from triune_b200.models.quant_linear import NVFP4Linear

        q = NVFP4Linear.from_linear(lin, hadamard=True).eval()
    else:
        ref_modules()
        from triune.kernels.fast_nvfp4 import NVFP4Linear as RefQ

        q = RefQ.from_linear(lin) if hasattr(RefQ, "from_linear") else RefQ(4096, 4096, bias=False).to("cuda")
    with torch.no_grad():
        ms = timed(lambda: q(x), a.iters)
        y, y0 = q(x).float(), lin(x).float()
        cos = float(torch.nn.functional.cosine_similarity(y.flatten(), y0.flatten(), dim=0))
        size = sum(t.numel() * t.element_size() for t in list(q.buffers()) + list(q.parameters()))
        emit(case="NVFP4 linear 4096x4096, 4096 rows", impl=impl, ms=ms, tflops=2 * 4096**3 / ms / 1e9, weight_mb=size / 2**20, cosine_to_bf16=cos)
        if impl == "ours":
            emit(case="NVFP4 linear 4096x4096, 4096 rows", impl="bf16 layer", ms=timed(lambda: lin(x), a.iters))


def case_gla(impl, a):
    """One linear-attention layer against softmax attention at long context: prefill T=8192 (H=6, dk=64; published 0.60 ms
    against 6.07 ms), prefill L=16384 (H=8; 3.72 against 14.97 ms), and one decode step after 16384 tokens."""
    torch.manual_seed(0)
    for H, T in ((6, 8192), (8, 16384)):
        q, k, v = (torch.randn(1, T, H, 64, device="cuda", dtype=torch.bfloat16) * 0.3 for _ in range(3))
        g = -torch.rand(1, T, H, 64, device="cuda", dtype=torch.bfloat16) * 0.1
        if impl == "ours":
            from triune_b200 import ops

            fn = lambda: ops.gla(q, k, v, g)
        else:
            ref_modules()
            from triune.kernels.fast_gla import fast_chunk_gla

            fn = lambda: fast_chunk_gla(q, k, v, g)
        with torch.no_grad():
            ms = timed(fn, a.iters)
            emit(case=f"GLA layer prefill T={T} H={H} dk=64", impl=impl, ms=ms, tok_s=T / ms * 1e3)
            if impl == "ours":
                qs, ks, vs = (t.transpose(1, 2) for t in (q, k, v))
                ms = timed(lambda: torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True), a.iters)
                emit(case=f"GLA layer prefill T={T} H={H} dk=64", impl="softmax attention (library)", ms=ms, tok_s=T / ms * 1e3)
    if impl == "ours":
        from triune_b200 import ops

        H = 8
        state = torch.randn(1, H, 64, 64, device="cuda", dtype=torch.float32)
        q1, k1, v1 = (torch.randn(1, 1, H, 64, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        g1 = -torch.rand(1, 1, H, 64, device="cuda", dtype=torch.bfloat16) * 0.1
        with torch.no_grad():
            ms = timed(lambda: ops.gla(q1, k1, v1, g1, initial_state=state), a.iters * 3)
            emit(case="GLA decode step after 16384 tokens, H=8", impl=impl, ms=ms, state_kb=state.numel() * 4 / 1024)
            kc, vc = (torch.randn(1, H, 16384, 64, device="cuda", dtype=torch.bfloat16) for _ in range(2))
            qd = torch.randn(1, H, 1, 64, device="cuda", dtype=torch.bfloat16)
            ms = timed(lambda: torch.nn.functional.scaled_dot_product_attention(qd, kc, vc), a.iters * 3)
            emit(case="GLA decode step after 16384 tokens, H=8", impl="softmax attention (library), KV cache", ms=ms, cache_kb=2 * kc.numel() * 2 / 1024)


def case_optim(impl, a):
    """One optimizer step on a small model with gradients in place (published medians on 17 M parameters: AdamW 1.54,
    CentroidSteer 4.76, Muon 6.27 ms)."""
    torch.manual_seed(0)
    if impl == "ours":
        from triune_b200.optim import build_optimizer

        # the bench model at vocabulary 4096 with 2 experts per layer: the same architecture in both arms
        model = ours_model(vocab=4096, num_experts=2).train()
        mk = lambda kind: build_optimizer(model, {"optimizer": kind, "lr": 1e-4, "ns_steps": 5})
    else:
        m = ref_modules()
        from triune.optim.centroid import CentroidSteerOptimizer as RefOpt

        model = m["Model"](vocab_size=4096, hidden_dim=384, num_layers=8, num_heads=6, head_dim=64, num_experts=2, router_prefix_layers=1,
                           reflex_exit_layer=2, limbic_exit_layer=5).to(device="cuda", dtype=torch.bfloat16).train()
        mk = lambda kind: (RefOpt(model, lr=1e-4, muon_ns_steps=5) if kind == "centroid_steer"
                           else RefOpt(model, lr=1e-4, use_triangular_core=False, steer_scale=0.0, muon_ns_steps=5) if kind == "muon"
                           else torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True))
    n = sum(p.numel() for p in model.parameters())
    ids = torch.randint(0, 4096, (4, 256), device="cuda")
    for kind in ("adamw", "centroid_steer", "muon"):
        opt = mk(kind)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=impl != "ours"):
            out = model(ids, force_depth=2)
            logits = out[0] if isinstance(out, tuple) else out
            torch.nn.functional.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), ids.reshape(-1)).backward()
        ms = timed(lambda: opt.step(), a.iters, 3)  # the same gradients every call: only the update is timed
        state = sum(t.numel() * t.element_size() for st in opt.state.values() if isinstance(st, dict) for t in st.values() if torch.is_tensor(t))
        emit(case=f"optimizer step, {n / 1e6:.2f} M parameters", impl=impl, optimizer=kind, ms=ms, state_mb=state / 2**20)
        opt.zero_grad(set_to_none=True)
        del opt


CASES = {"exits": case_exits, "prefill": case_prefill, "decode": case_decode, "moe": case_moe, "ce": case_ce, "rows": case_rows,
         "nvfp4": case_nvfp4, "gla": case_gla, "optim": case_optim}


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--only", default="", help="comma-separated case names: " + ", ".join(CASES))
    ap.add_argument("--impl", default="both", choices=["both", "ours", "reference"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--budget", type=float, default=0.0, help="seconds after which the remaining cases are skipped (0: no limit)")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        emit(error="bench_micro.py needs a GPU")
        return 1
    names = [n for n in (a.only.split(",") if a.only else CASES) if n]
    impls = ["ours", "reference"] if a.impl == "both" else [a.impl]
    t_start = time.time()
    pr = torch.cuda.get_device_properties(0)
    emit(device=pr.name, sms=pr.multi_processor_count, torch=torch.__version__, timing="CUDA events, median, L2 flushed between calls",
         iters=a.iters, started=time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()))
    for impl in impls:
        if impl == "reference" and ref_modules() is None:
            continue
        for n in names:
            if n not in CASES:
                emit(error=f"unknown case {n!r}")
                continue
            if a.budget and time.time() - t_start > a.budget:
                emit(case=n, impl=impl, skipped=f"the time budget of {a.budget:.0f} s was used up")
                continue
            guarded(CASES[n].__doc__.split("\n")[0] if CASES[n].__doc__ else n, impl)(CASES[n])(impl, a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
