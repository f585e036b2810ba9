"""Worker for tensor parallel 2 x data parallel 2 on four gloo ranks: gradients after the two reductions equal those of
the unsharded model on the whole batch."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triune_b200.config import ModelConfig  # noqa: E402
from triune_b200.models.universal import UniversalDenseTransformer  # noqa: E402
from triune_b200.parallel.tensor_parallel import TPContext  # noqa: E402
from triune_b200.parallel.tp_model import TensorParallelDense, average_grads_over_replicas, make_tp_dp_groups  # noqa: E402


def rel(a, b):
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-12))


def main():
    dist.init_process_group("gloo")
    r = dist.get_rank()
    tp_group, dp_group = make_tp_dp_groups(2)
    tp_rank, replica = r % 2, r // 2
    torch.manual_seed(5)
    D = 16
    cfg = ModelConfig(family="universal", vocab_size=128, hidden_dim=4 * D, num_layers=2, num_heads=4, head_dim=D,
                      mixer="gla", ffn="swiglu", dense_hidden=8 * D, num_experts=1, top_k=1, tie_embeddings=False)
    full = UniversalDenseTransformer.from_config(cfg)
    ids = torch.randint(0, 128, (4, 33), generator=torch.Generator().manual_seed(9))
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    loss_full = full.forward_loss(x, y)
    loss_full = loss_full[0] if isinstance(loss_full, tuple) else loss_full
    loss_full.backward()
    ref = {n: p.grad.detach().clone() for n, p in full.named_parameters()}
    full.zero_grad(set_to_none=True)

    tp = TPContext(group=tp_group, device="cpu", mode="nccl")
    model = TensorParallelDense(full, tp)
    xb, yb = x[replica * 2:(replica + 1) * 2], y[replica * 2:(replica + 1) * 2]   # this replica's half of the batch
    part = model.forward_loss(xb, yb)
    part.backward()
    model.allreduce_replicated_grads()
    average_grads_over_replicas(model, dp_group)
    total = model.reduce_loss(part)                     # mean loss of this replica's half
    both = total.clone()
    dist.all_reduce(both, group=dp_group)
    out = {"rank": r, "loss": abs(float(both) / 2 - float(loss_full)) / abs(float(loss_full))}
    out["embed"] = rel(model.embed_tokens.weight.grad, ref["embed_tokens.weight"])
    out["head"] = rel(model.lm_head.weight.grad, ref["lm_head.weight"])
    blk = model.layers[0]
    H, Hl, d = cfg.num_heads, blk.heads_local, cfg.hidden_dim
    g_qkvg = ref["layers.0.attn.qkvg_weight"].view(4, H, D, d)[:, tp_rank * Hl:(tp_rank + 1) * Hl].reshape(4 * Hl * D, d)
    out["qkvg"] = rel(blk.qkvg_weight.grad[: 4 * Hl * D], g_qkvg)
    hl, hid = blk.hidden_local, cfg.resolved_dense_hidden()
    out["down"] = rel(blk.down_weight.grad, ref["layers.0.mlp.down.weight"][:, tp_rank * hl:(tp_rank + 1) * hl])
    sys.stdout.write("\nRESULT " + json.dumps(out) + "\n")
    sys.stdout.flush()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
