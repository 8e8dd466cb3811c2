"""Tensor-parallel linear layers on top of the fused kernels (inference; no autograd).

`RowParallelLinear` holds a K-slice of the weight and returns the all-reduced product, optionally with
the residual add and RMSNorm that follow it in a decoder block, from one kernel.  `ColumnParallelLinear`
holds an N-slice; with `gather_input=True` its input is row-sharded and the all-gather is fused into
the GEMM.  Both work on one rank per process or on all ranks of an emulated world (lists of tensors).
"""
from __future__ import annotations

from typing import Optional

import torch

from .communicator import Communicator


class RowParallelLinear:
    def __init__(self, comm: Communicator, weight, fused: str = "gemm"):
        """weight: [N, K_local] (nn.Linear layout) or a list with one such tensor per local rank.
        fused: "gemm" = tcgen05 GEMM + reduce-scatter epilogue kernel; "allreduce" = library GEMM followed by
        the one-shot all-reduce (+ residual + RMSNorm) kernel."""
        assert fused in ("gemm", "allreduce")
        self.comm, self.weight, self.fused = comm, weight, fused

    def __call__(self, x, residual=None, gamma=None, eps: float = 1e-5):
        c = self.comm
        if self.fused == "gemm":
            return c.linear_allreduce(x, self.weight, residual, gamma, eps)
        many = isinstance(x, (list, tuple))
        parts = [xi @ wi.t() for xi, wi in zip(x, self.weight)] if many else x @ self.weight.t()
        if gamma is not None:
            return c.allreduce_residual_rmsnorm(parts, residual, gamma, eps)
        out = c.all_reduce(parts)
        if residual is not None:
            out = [o + r for o, r in zip(out, residual)] if many else out + residual
        return out


class ColumnParallelLinear:
    def __init__(self, comm: Communicator, weight, gather_input: bool = False):
        """weight: [N_local, K] or a list of those.  gather_input: the input arrives row-sharded
        ([M / world, K] per rank) and is all-gathered inside the GEMM kernel."""
        self.comm, self.weight, self.gather_input = comm, weight, gather_input

    def __call__(self, x):
        if self.gather_input:
            return self.comm.allgather_linear(x, self.weight)
        if isinstance(x, (list, tuple)):
            return [xi @ wi.t() for xi, wi in zip(x, self.weight)]
        return x @ self.weight.t()
