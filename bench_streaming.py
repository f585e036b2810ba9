"""Layer-streamed training on ONE GPU: the model's layers live in pinned host memory and pass through the GPU a few at
a time (forward, then backward in reverse, each layer's optimizer update applied as its gradients arrive).

    python bench_streaming.py                                   # dense 1.5B-class preset, 4 x 2048 tokens, 2 resident layers
    python bench_streaming.py --shape 1536 13 --vocab 4096 --batch 2 --seq 512   # the reference's 1.52 B streaming shape

`--shape D L` builds a model of width D with L layers instead of a preset (the reference's streaming table uses
(512, 8), (768, 10), (1024, 14), (1536, 13) at vocabulary 4096, batch 2, sequence 512:
`scripts/benchmark_layer_streaming.py:44-100`). Prints one JSON line: seconds per step (device-timed), tokens per second,
host-to-device traffic per step and peak GPU memory, next to the same model trained fully resident when `--resident-too`
is given and it fits.
"""

from __future__ import annotations

import argparse
import json
import time

import torch


def build(a):
    from triune_b200.config import ModelConfig, get_model_config
    from triune_b200.models import TriuneTransformer

    if a.shape:
        d, L = a.shape
        heads = max(1, d // 64)
        reflex = max(2, L // 4)
        cfg = ModelConfig(vocab_size=a.vocab, hidden_dim=d, num_layers=L, num_heads=heads, head_dim=64, num_experts=a.experts,
                          router_prefix_layers=1, reflex_exit_layer=reflex, limbic_exit_layer=max(reflex + 1, L // 2))
    else:
        cfg = get_model_config(a.model)
    torch.manual_seed(0)
    return TriuneTransformer.from_config(cfg).to(torch.bfloat16), cfg


def timed_steps(step, steps: int, warmup: int) -> float:
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps / 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="bench-dense-1.5b")
    ap.add_argument("--shape", type=int, nargs=2, default=None, metavar=("D", "L"))
    ap.add_argument("--vocab", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--resident-layers", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--resident-too", action="store_true", help="also time the same model fully resident on the GPU")
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "tiered"],
                    help="streamed layers: the engine's built-in AdamW, or the tiered optimizer (AdamW / Muon / CentroidSteer "
                         "through step_parameters, one layer's state on the device at a time)")
    ap.add_argument("--state-dtype", default="fp32", choices=["fp32", "bf16"], help="host format of the tiered optimizer's moments")
    ap.add_argument("--fp8-weights", action="store_true", help="stage the forward / backward weights as E4M3 + block scales")
    ap.add_argument("--grad-dtype", default="fp32", choices=["fp32", "bf16"], help="format of the gradients between device and host")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_streaming.py needs a CUDA device")

    from triune_b200.runtime.streaming import StreamingConfig, enable_layer_streaming

    t0 = time.time()
    model, cfg = build(a)
    params = sum(p.numel() for p in model.parameters())
    build_s = time.time() - t0
    host = torch.randint(0, cfg.vocab_size, (a.batch, a.seq + 1), generator=torch.Generator().manual_seed(1)).pin_memory()
    eng = enable_layer_streaming(model, "cuda", config=StreamingConfig(resident_gpu_layers=a.resident_layers, fp8_weights=a.fp8_weights,
                                                                       grad_dtype=a.grad_dtype))
    last = {}
    root_opt = None
    if a.optimizer == "tiered":
        from triune_b200.optim import CentroidSteerOptimizer

        streamed = {id(p) for st in eng.stores.values() for p in st.params}
        inner = CentroidSteerOptimizer(model, lr=1e-4, grad_clip=None, only=lambda n, p: id(p) not in streamed)
        eng.enable_tiered_optimizer(lr=1e-4, state_dtype=torch.bfloat16 if a.state_dtype == "bf16" else torch.float32)

        class _Root:  # the engine clips the root gradients itself, then calls step / zero_grad
            def step(self):
                inner.set_clip_coefficient(1.0)
                inner.step_parameters([s_.param for s_ in inner.arena.segments], is_global_step_end=True)

            def zero_grad(self, set_to_none=True):
                inner.zero_grad()

        root_opt = _Root()

    def step():
        ids = host.to("cuda", non_blocking=True)
        out = model.forward_loss(ids[:, :-1], ids[:, 1:], force_depth=2)
        loss = out[0] if isinstance(out, tuple) else out
        loss.backward()
        eng.step_streaming_optimizer(root_opt, lr=1e-4)
        last["loss"] = loss

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    tel0 = dict(eng.get_telemetry())
    sec = timed_steps(step, a.steps, 0)
    tel = eng.get_telemetry()
    rec = {"metric": "layer-streamed train tok/s (one GPU, device-timed)", "value": a.batch * a.seq / sec, "unit": "tok/s",
           "s_per_step": round(sec, 4), "steps": a.steps, "warmup": a.warmup, "dtype": "bf16",
           "config": {"model": a.model if not a.shape else f"d{a.shape[0]}-L{a.shape[1]}-V{a.vocab}", "params": params,
                      "layers": cfg.num_layers, "hidden_dim": cfg.hidden_dim, "batch": a.batch, "seq_len": a.seq,
                      "resident_layers": a.resident_layers, "streamed_optimizer": a.optimizer, "state_dtype": a.state_dtype,
                      "fp8_weights": a.fp8_weights, "grad_dtype": a.grad_dtype},
           "h2d_GB_per_step": round((tel.get("h2d_bytes", 0) - tel0.get("h2d_bytes", 0)) / a.steps / 2**30, 2),
           "peak_gpu_GB": round(torch.cuda.max_memory_allocated() / 2**30, 2), "build_s": round(build_s, 1),
           "final_loss": float(last["loss"]), "impl": "triune_b200"}
    if a.resident_too:
        from triune_b200.optim import CentroidSteerOptimizer

        del eng, model
        torch.cuda.empty_cache()
        model, _ = build(a)
        model.cuda()
        opt = CentroidSteerOptimizer(model, lr=1e-4)
        torch.cuda.reset_peak_memory_stats()

        def rstep():
            ids = host.to("cuda", non_blocking=True)
            out = model.forward_loss(ids[:, :-1], ids[:, 1:], force_depth=2)
            (out[0] if isinstance(out, tuple) else out).backward()
            opt.step()
            opt.zero_grad()

        rsec = timed_steps(rstep, a.steps, a.warmup)
        rec["resident"] = {"s_per_step": round(rsec, 4), "tok_s": a.batch * a.seq / rsec,
                           "peak_gpu_GB": round(torch.cuda.max_memory_allocated() / 2**30, 2)}
    print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
