"""Functional face of the collectives, shaped like `torch.distributed`: a module-level default
communicator plus `all_reduce(tensor)`, `all_gather_into_tensor(out, x)`, `reduce_scatter_tensor(out, x)`.

The reference's smoke script does exactly this with a oneCCL process group
(script/gpu_inference_test.py:21-45); `init()` + `all_reduce()` below is that flow on this library.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel.communicator import Communicator

_default: Optional[Communicator] = None


def init(comm: Optional[Communicator] = None, **kw) -> Communicator:
    """Installs the default communicator: `comm`, or one built from an initialised `torch.distributed`
    group (keyword arguments go to `Communicator.from_torch_distributed`)."""
    global _default
    if comm is None:
        import torch.distributed as dist

        comm = Communicator.from_torch_distributed(**kw) if dist.is_initialized() else Communicator.create(**kw)
    _default = comm
    return comm


def default_communicator() -> Communicator:
    if _default is None:
        raise RuntimeError("no default communicator: call gpu_ipc_example_b200.ops.init() first")
    return _default


def shutdown() -> None:
    global _default
    if _default is not None:
        _default.close()
        _default = None


def all_reduce(tensor, algo: str = "auto", comm: Optional[Communicator] = None):
    """In-place sum over ranks (like `dist.all_reduce`).  On an emulated world (all ranks on one GPU) every
    function of this module takes one tensor per rank, as a list."""
    c = comm or default_communicator()
    if isinstance(tensor, (list, tuple)):
        return c.all_reduce(list(tensor), None, algo)
    if tensor.is_contiguous() and tensor.data_ptr() % 16 == 0 and c.nlocal == 1:
        return c.all_reduce_(tensor, algo)
    return c.all_reduce(tensor, None, algo)


def all_gather_into_tensor(output: torch.Tensor, tensor: torch.Tensor, algo: str = "allgather_auto",
                           comm: Optional[Communicator] = None) -> torch.Tensor:
    c = comm or default_communicator()
    return c.all_gather(tensor, output, algo)


def reduce_scatter_tensor(output: torch.Tensor, tensor: torch.Tensor, algo: str = "auto",
                          comm: Optional[Communicator] = None) -> torch.Tensor:
    c = comm or default_communicator()
    return c.reduce_scatter(tensor, output, algo)


def allreduce_residual_rmsnorm(x, residual, gamma, eps: float = 1e-5, comm: Optional[Communicator] = None):
    return (comm or default_communicator()).allreduce_residual_rmsnorm(x, residual, gamma, eps)


def linear_allreduce(x, weight, residual=None, gamma=None, eps: float = 1e-5, comm: Optional[Communicator] = None):
    return (comm or default_communicator()).linear_allreduce(x, weight, residual, gamma, eps)


def allgather_linear(x_shard, weight, comm: Optional[Communicator] = None):
    return (comm or default_communicator()).allgather_linear(x_shard, weight)
