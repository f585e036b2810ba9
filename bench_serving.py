#!/usr/bin/env python
"""Serving benchmark of the 90.8M-class MoE-GLA model: long-context prefill and greedy decode, on one GPU or on all GPUs
of a node.

    python bench_serving.py [--impl ours|reference] [--batch 4] [--seq 16384] [--new-tokens 256] [--iters 5]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench_serving.py --layout replicas
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench_serving.py --layout ep

Under a multi-process launch every rank serves its own ``batch x seq`` prompt batch. ``--layout replicas``: one full
model per GPU, no communication. ``--layout ep``: the routed experts are sharded over all ranks (fused NVLink dispatch /
combine kernels), everything else replicated. Times are device-timed per rank; the reported value is the whole-node
aggregate, world x tokens / max-over-ranks time. Decode is measured on rank 0 of a one-GPU run only.

Prefill: one forward over ``batch x seq`` uniform-random token ids into the recurrent cache, logits of the last
position only; timed with CUDA events after warm-up iterations, L2 irrelevant (inputs and activations are far larger
than it). Variants: bf16 weights, block-scaled FP8 (E4M3), NVFP4 (E2M1 + E4M3/16 scales). Decode: greedy, ``new-tokens``
tokens for one sequence, plain Cortex decoding versus self-speculative decoding (Reflex exit drafts, Cortex verifies);
wall-clock with a device synchronise on both sides because the loop is host-driven. One JSON line per measurement.
``--impl reference`` runs the unmodified reference (``baseline/_ref``) through its own forward for the same shapes.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
VOCAB = 32000


def timed(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def emit(**kw):
    print(json.dumps(kw), flush=True)


def run_ours(a):
    from triune_b200 import ops
    from triune_b200.config import get_model_config
    from triune_b200.models import TriuneTransformer
    from triune_b200.models.quant_linear import convert_to_fp8, convert_to_nvfp4
    from triune_b200.models.speculative import SelfSpeculativeGenerator
    from triune_b200.utils import place_model

    rank, world, local = _dist_env()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    ep = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    ids = torch.randint(0, VOCAB, (a.batch, a.seq), device=dev, generator=torch.Generator(device=dev).manual_seed(rank))
    for variant in a.variants.split(","):
        torch.manual_seed(0)
        model = place_model(TriuneTransformer.from_config(get_model_config(a.model)), dev, torch.bfloat16).eval()
        if world > 1 and a.layout == "ep":
            from triune_b200.parallel.expert_parallel import EPContext, shard_experts

            ep = EPContext(model.num_experts, device=dev, mode="fused")
            shard_experts(model, ep)
        converted = 0
        if variant == "fp8":
            converted = convert_to_fp8(model)
        elif variant == "nvfp4":
            converted = convert_to_nvfp4(model)

        @torch.no_grad()
        def prefill():
            return model(ids, force_depth=2, cache=model.init_cache(a.batch), last_token_only=True)

        ops.reset_launch_count()
        prefill()
        launches = ops.launch_count()
        ms = _max_over_ranks(timed(prefill, a.iters), dev, world)
        status = int(ep.check()) if ep is not None else 0
        if rank == 0:
            emit(metric="prefill tok/s", impl="triune_b200", variant=variant, value=world * a.batch * a.seq / ms * 1e3, unit="tok/s",
                 ms=ms, batch=a.batch, seq_len=a.seq, n_gpus=world, layout=(a.layout if world > 1 else "one GPU"), model=a.model,
                 converted_linears=converted, gpu_launches=launches, dtype="bf16 activations", wait_status=status)
        if variant == "bf16" and a.new_tokens > 0 and world == 1:
            from triune_b200.inference import GraphedGreedyDecoder

            prompt = ids[:1, :128]
            gen = SelfSpeculativeGenerator(model, k_draft=a.k_draft)
            graphed = GraphedGreedyDecoder(model, batch_size=1, decode_depth=2)
            for name, fn in (("decode (Cortex, greedy, one CUDA graph per token)", lambda: graphed.generate(prompt, a.new_tokens)),
                             ("decode (Cortex, greedy)", lambda: gen.generate_autoregressive(prompt, a.new_tokens)),
                             ("decode (self-speculative, greedy)", lambda: gen.generate(prompt, a.new_tokens, temperature=0.0))):
                fn()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                out = fn()
                torch.cuda.synchronize()
                dt = time.perf_counter() - t0
                emit(metric=name + " tok/s", impl="triune_b200", value=(out.shape[1] - prompt.shape[1]) / dt, unit="tok/s",
                     new_tokens=int(out.shape[1] - prompt.shape[1]), acceptance_rate=round(gen.acceptance_rate, 3) if "spec" in name else None)
            # the same scheme with a whole round (k drafts, one batched verification, commit) replayed as ONE CUDA graph
            from triune_b200.inference import GraphedSpeculativeDecoder

            def spec_run(tag):
                dec = GraphedSpeculativeDecoder(model, k_draft=a.k_draft)
                dec.generate(prompt, a.new_tokens)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                out = dec.generate(prompt, a.new_tokens)
                torch.cuda.synchronize()
                dt = time.perf_counter() - t0
                ref_out = graphed.generate(prompt, a.new_tokens)
                same = (out == ref_out)[0].long()
                agree = int(torch.cumprod(same, 0).sum().item()) - prompt.shape[1]
                # bf16: the batched verification (rows of 4 tokens) and the one-token step round differently, so with
                # random-init weights (near-uniform logits) an arg-max can flip; the scheme itself is exact (CPU test)
                emit(metric=f"decode (self-speculative, greedy, one CUDA graph per round{tag}) tok/s", impl="triune_b200",
                     value=(out.shape[1] - prompt.shape[1]) / dt, unit="tok/s", new_tokens=int(out.shape[1] - prompt.shape[1]),
                     acceptance_rate=round(dec.acceptance_rate, 3), k_draft=a.k_draft,
                     tokens_equal_to_greedy_before_first_difference=agree)

            spec_run("")
            # random-init exits never agree with the full depth; a short KL distillation of the exit heads toward the
            # full-depth predictions (the model's own `distill_exit_heads`) gives the drafts something to agree on
            calib = torch.randint(0, VOCAB, (32, 128), device=dev, generator=torch.Generator(device=dev).manual_seed(7))
            calib[0] = prompt[0]
            rep = model.distill_exit_heads(calib, steps=200, lr=3e-3, batch_size=8)
            model.eval()
            spec_run(f", exit heads distilled {rep['steps']} steps")
        del model
        torch.cuda.empty_cache()


def _dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))


def _max_over_ranks(ms: float, dev, world: int) -> float:
    if world == 1:
        return ms
    import torch.distributed as dist

    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_reference(a):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "triune")):
        emit(impl="reference", unavailable="baseline/_ref is not installed")
        return
    try:
        sys.path.insert(0, ref_dir)
        import triune.model.config as rc

        rc.TOP_K_EXPERTS, rc.EXPERT_HIDDEN_MULTIPLIER = 2, 4
        import triune.model.moe as rmoe
        from triune.model.transformer import TriuneTransformer as RefModel

        rmoe.EXPERT_HIDDEN_MULTIPLIER, rmoe.TOP_K_EXPERTS = 4, 2
    except Exception as e:
        emit(impl="reference", unavailable=f"import failed: {type(e).__name__}: {e}"[:300])
        return
    rank, world, local = _dist_env()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:  # independent replicas of the reference, one per GPU (it has no expert-parallel serving path)
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    model = RefModel(vocab_size=VOCAB, hidden_dim=384, num_layers=8, num_heads=6, head_dim=64, num_experts=8, router_prefix_layers=1,
                     reflex_exit_layer=2, limbic_exit_layer=5).to(device=dev, dtype=torch.bfloat16).eval()
    for m in model.modules():
        if isinstance(m, rmoe.MoE_FFN):
            m.top_k = 2
    ids = torch.randint(0, VOCAB, (a.batch, a.seq), device=dev, generator=torch.Generator(device=dev).manual_seed(0))

    @torch.no_grad()
    def prefill():
        cache = model.init_cache(a.batch)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            return model(ids, force_depth=2, cache=cache, last_token_only=True)

    try:
        ms = _max_over_ranks(timed(prefill, a.iters), dev, world)
        if rank == 0:
            emit(metric="prefill tok/s", impl="reference", variant="bf16", value=world * a.batch * a.seq / ms * 1e3, unit="tok/s",
                 ms=ms, batch=a.batch, seq_len=a.seq, n_gpus=world, layout="replicas" if world > 1 else "one GPU")
        if a.new_tokens > 0 and world == 1:
            prompt = ids[:1, :128]

            @torch.no_grad()
            def decode():
                cache = model.init_cache(1)
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    logits, cache = model(prompt, force_depth=2, cache=cache, last_token_only=True)
                    for _ in range(a.new_tokens):
                        tok = logits[:, -1].argmax(-1, keepdim=True)
                        logits, cache = model(tok, force_depth=2, cache=cache, last_token_only=True)

            decode()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            decode()
            torch.cuda.synchronize()
            emit(metric="decode (Cortex, greedy) tok/s", impl="reference", value=a.new_tokens / (time.perf_counter() - t0), unit="tok/s",
                 new_tokens=a.new_tokens)
    except Exception as e:
        emit(impl="reference", unavailable=f"run failed: {type(e).__name__}: {e}"[:300])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=16384)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--k-draft", type=int, default=3)
    ap.add_argument("--variants", default="bf16,fp8,nvfp4")
    ap.add_argument("--layout", default="replicas", choices=["replicas", "ep"], help="multi-GPU layout (under torchrun)")
    ap.add_argument("--model", default="bench-90m", help="model preset of the native arm")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        emit(impl=a.impl, unavailable="no CUDA device")
        return
    (run_ours if a.impl == "ours" else run_reference)(a)


if __name__ == "__main__":
    main()
