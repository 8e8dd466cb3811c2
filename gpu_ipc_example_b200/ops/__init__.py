from .functional import (all_gather_into_tensor, all_reduce, allgather_linear, allreduce_residual_rmsnorm, default_communicator,
                         init, linear_allreduce, reduce_scatter_tensor, shutdown)

__all__ = ["init", "shutdown", "default_communicator", "all_reduce", "all_gather_into_tensor", "reduce_scatter_tensor",
           "allreduce_residual_rmsnorm", "linear_allreduce", "allgather_linear"]
