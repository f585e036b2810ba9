"""Parallelism: process groups, sharded data parallelism, tensor / expert parallel layers, symmetric memory."""

from .dist import (DistributedContext, all_reduce_dict, all_reduce_tensor, cleanup_distributed, max_over_ranks,
                   setup_distributed)

__all__ = ["DistributedContext", "all_reduce_dict", "all_reduce_tensor", "cleanup_distributed", "max_over_ranks",
           "setup_distributed"]
