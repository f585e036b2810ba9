"""Parallelism: process groups, sharded data parallelism, tensor / expert / context parallel layers, symmetric memory.

The heavier modules are imported lazily (they pull in the CUDA extension and symmetric memory):

    from triune_b200.parallel import TensorParallelDense, TPContext, cp_gla, EPContext, shard_experts
"""

from .dist import (DistributedContext, all_reduce_dict, all_reduce_tensor, cleanup_distributed, max_over_ranks,
                   setup_distributed)

_LAZY = {
    "ShardedDataParallel": "data_parallel",
    "TPContext": "tensor_parallel",
    "ColumnParallelLinear": "tensor_parallel",
    "RowParallelLinear": "tensor_parallel",
    "ag_gemm": "tensor_parallel",
    "gemm_rs": "tensor_parallel",
    "TensorParallelDense": "tp_model",
    "tensor_parallelize": "tp_model",
    "EPContext": "expert_parallel",
    "ExpertParallelMoE": "expert_parallel",
    "shard_experts": "expert_parallel",
    "allreduce_replicated_grads": "expert_parallel",
    "cp_gla": "context_parallel",
    "ElasticGroup": "elastic",
    "run_elastic": "elastic",
    "RankFailure": "elastic",
    "CollectiveTimeout": "elastic",
    "FailureDetector": "elastic",
    "Heartbeat": "elastic",
    "PipelineStage": "pipeline",
    "TriunePipelineStage": "pipeline",
    "PipelineEngine": "pipeline",
    "pipeline_parallelize": "pipeline",
    "make_pp_dp_groups": "pipeline",
    "make_tp_dp_groups": "tp_model",
    "average_grads_over_replicas": "tp_model",
}

__all__ = ["DistributedContext", "all_reduce_dict", "all_reduce_tensor", "cleanup_distributed", "max_over_ranks",
           "setup_distributed"] + sorted(_LAZY)


def __getattr__(name):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    import importlib

    return getattr(importlib.import_module(f"{__name__}.{mod}"), name)
