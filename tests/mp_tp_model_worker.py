"""Worker for the tensor-parallel dense model test (gloo on CPU, or NCCL / fused kernels on GPUs): the sharded model
must reproduce the loss and the gradients of the unsharded one."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triune_b200.config import ModelConfig  # noqa: E402
from triune_b200.models.universal import UniversalDenseTransformer  # noqa: E402
from triune_b200.parallel.tensor_parallel import TPContext  # noqa: E402
from triune_b200.parallel.tp_model import TensorParallelDense  # noqa: E402


def rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-9))


def main():
    use_cuda = os.environ.get("TRIUNE_TP_DEVICE", "cpu") == "cuda"
    dist.init_process_group("nccl" if use_cuda else "gloo")
    r, w = dist.get_rank(), dist.get_world_size()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", r)))
    dev = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    dtype = torch.bfloat16 if use_cuda else torch.float32
    out = {"rank": r}
    for mixer, ffn in (("gla", "swiglu"), ("gated_deltanet", "gelu")):
        torch.manual_seed(7)
        D = 64 if use_cuda else 16
        cfg = ModelConfig(family="universal", vocab_size=256, hidden_dim=4 * D, num_layers=2, num_heads=4, head_dim=D,
                          mixer=mixer, ffn=ffn, dense_hidden=8 * D, num_experts=1, top_k=1, tie_embeddings=False)
        full = UniversalDenseTransformer.from_config(cfg).to(dev, dtype)
        B, T = 2, (256 if use_cuda else 32)
        ids = torch.randint(0, 256, (B, T + 1), generator=torch.Generator().manual_seed(3)).to(dev)
        x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
        loss_full = full.forward_loss(x, y)
        loss_full = loss_full[0] if isinstance(loss_full, tuple) else loss_full
        loss_full.backward()
        ref_grads = {n: (getattr(p, "main_grad", None) if getattr(p, "main_grad", None) is not None else p.grad).detach().clone()
                     for n, p in full.named_parameters()}
        full.zero_grad(set_to_none=True)

        tp = TPContext(device=dev, mode=os.environ.get("TRIUNE_TP_MODE", "nccl"))
        model = TensorParallelDense(full, tp)
        part = model.forward_loss(x, y)
        part.backward()
        model.allreduce_replicated_grads()
        total = model.reduce_loss(part)
        key = f"{mixer}_{ffn}"
        out[key + "_loss"] = abs(float(total) - float(loss_full)) / max(1e-9, abs(float(loss_full)))
        # replicated parameters: summed partial gradients equal the full gradients
        out[key + "_embed"] = rel(model.embed_tokens.weight.grad, ref_grads["embed_tokens.weight"])
        out[key + "_head"] = rel(model.lm_head.weight.grad, ref_grads["lm_head.weight"])
        out[key + "_norm"] = rel(model.layers[1].input_norm.weight.grad, ref_grads["layers.1.input_norm.weight"])
        # sharded parameters: slices of the full gradients
        blk = model.layers[0]
        H, Hl, d = cfg.num_heads, blk.heads_local, cfg.hidden_dim
        g_qkvg = ref_grads["layers.0.attn.qkvg_weight"].view(4, H, D, d)[:, r * Hl:(r + 1) * Hl].reshape(4 * Hl * D, d)
        out[key + "_qkvg"] = rel(blk.qkvg_weight.grad[: 4 * Hl * D], g_qkvg)
        g_out = ref_grads["layers.0.attn.out_proj.weight"].view(d, H, D)[:, r * Hl:(r + 1) * Hl].reshape(d, Hl * D)
        out[key + "_out"] = rel(blk.out_weight.grad, g_out)
        hl = blk.hidden_local
        if ffn == "swiglu":
            hid = cfg.resolved_dense_hidden()
            g_up = ref_grads["layers.0.mlp.gate_up"].view(2, hid, d)[:, r * hl:(r + 1) * hl].reshape(2 * hl, d)
            g_down = ref_grads["layers.0.mlp.down.weight"][:, r * hl:(r + 1) * hl]
        else:
            g_up = ref_grads["layers.0.mlp.0.weight"][r * hl:(r + 1) * hl]
            g_down = ref_grads["layers.0.mlp.2.weight"][:, r * hl:(r + 1) * hl]
            out[key + "_down_bias"] = rel(blk.down_bias.grad, ref_grads["layers.0.mlp.2.bias"])
        out[key + "_up"] = rel(blk.up_weight.grad, g_up)
        out[key + "_down"] = rel(blk.down_weight.grad, g_down)
        if blk.has_beta:
            g_beta = ref_grads["layers.0.attn.beta_proj.weight"][r * Hl:(r + 1) * Hl]
            out[key + "_beta"] = rel(blk.qkvg_weight.grad[4 * Hl * D: 4 * Hl * D + Hl], g_beta)
        out[key + "_status"] = tp.check() if use_cuda else 0
    sys.stdout.write("\nRESULT " + json.dumps(out) + "\n")
    sys.stdout.flush()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
