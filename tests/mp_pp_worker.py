"""Worker of the pipeline-parallel test: every rank builds the same small dense model, keeps its stage, runs two 1F1B
steps and compares loss and gradients with the whole model on the whole batch (computed locally in the same process)."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    micro = int(os.environ.get("PP_MICRO", "4"))
    from triune_b200.config import ModelConfig
    from triune_b200.models.universal import UniversalDenseTransformer
    from triune_b200.parallel.pipeline import PipelineEngine, PipelineStage, peak_live_micro_batches

    from triune_b200.parallel.pipeline import make_pp_dp_groups
    from triune_b200.parallel.tp_model import average_grads_over_replicas

    pp = int(os.environ.get("PP_SIZE", "0")) or world
    pp_group, dp_group = make_pp_dp_groups(pp)
    stage_idx, replica, replicas = rank % pp, rank // pp, world // pp
    tol = 1e-9 if replicas == 1 else 1e-6  # the average over replicas travels as one flat fp32 buffer
    if os.environ.get("PP_FAMILY", "dense") == "triune":
        tol = 1e-6  # the expert router computes its logits in fp32 whatever the model's dtype
        # the multi-exit MoE family: tied embedding / head across first and last stage, capacity wide enough that the
        # micro-batches drop no token the whole batch would keep
        from triune_b200.models import TriuneTransformer
        from triune_b200.parallel.pipeline import TriunePipelineStage

        cfg = ModelConfig(vocab_size=96, hidden_dim=32, num_layers=6, num_heads=2, head_dim=16, num_experts=4, top_k=2,
                          reflex_exit_layer=2, limbic_exit_layer=3, router_prefix_layers=1, capacity_multiplier=8.0)
        torch.manual_seed(0)
        oracle = TriuneTransformer.from_config(cfg).double()
        torch.manual_seed(0)
        full = TriuneTransformer.from_config(cfg).double()
        stage = TriunePipelineStage(full, stage_idx, pp, update_stats=False)
        oracle_loss = lambda a, b: oracle.forward_loss(a, b, force_depth=2)  # noqa: E731
    else:
        cfg = ModelConfig(family="universal", vocab_size=96, hidden_dim=32, num_layers=5, num_heads=2, head_dim=16,
                          mixer="gla", ffn="swiglu", tie_embeddings=False)
        torch.manual_seed(0)
        oracle = UniversalDenseTransformer.from_config(cfg).double()
        torch.manual_seed(0)
        full = UniversalDenseTransformer.from_config(cfg).double()
        stage = PipelineStage(full, stage_idx, pp)
        oracle_loss = oracle.forward_loss
    del full
    eng = PipelineEngine(stage, micro, pp_group)

    gen = torch.Generator().manual_seed(7)
    ids = torch.randint(0, cfg.vocab_size, (8 * replicas, 17), generator=gen)
    x_all, y_all = ids[:, :-1], ids[:, 1:]                 # the oracle sees every replica's batch
    x, y = x_all[8 * replica: 8 * replica + 8], y_all[8 * replica: 8 * replica + 8]
    for step in range(2):  # the second step checks that nothing of the first is left in flight
        for p in stage.parameters():
            p.grad = None
        loss = eng.train_step(x, y)
        average_grads_over_replicas(stage, dp_group)
        if replicas > 1:
            dist.all_reduce(loss, group=dp_group)
            loss = loss / replicas
        oracle.zero_grad()
        ref = oracle_loss(x_all, y_all)
        ref.backward()
        assert abs(float(loss) - float(ref.detach())) < 1e-6, (rank, step, float(loss), float(ref.detach()))
        want = dict(oracle.named_parameters())
        n = 0
        for name, p in stage.full_names():
            if want[name].grad is None:  # early-exit heads take no gradient from the full-depth loss
                assert p.grad is None or float(p.grad.abs().max()) == 0.0, name
                continue
            assert p.grad is not None, name
            err = (p.grad - want[name].grad).abs().max().item()
            assert err < tol, (rank, name, err)
            n += 1
        assert n > 0
        assert eng.peak_live == peak_live_micro_batches(stage_idx, pp, micro), (eng.peak_live, rank)
    with torch.no_grad():  # forward-only pass through the pipeline against the oracle in eval mode
        oracle.eval()
        want_eval = oracle_loss(x, y)
        oracle.train()
    got_eval = eng.eval_loss(x, y)
    assert abs(float(got_eval) - float(want_eval)) < 1e-5, (rank, float(got_eval), float(want_eval))
    assert stage.training
    total = eng.clip_grad_norm(1e9)
    ref_norm = torch.sqrt(sum(p.grad.pow(2).sum() for p in oracle.parameters() if p.grad is not None))
    assert abs(float(total) - float(ref_norm)) < 1e-6 * max(1.0, float(ref_norm)), (float(total), float(ref_norm))
    dist.barrier()
    if rank == 0:
        print("PP_OK", world, micro, f"pp{pp}xdp{replicas}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
