"""The user-facing layers and the torch.distributed-shaped functions, on an emulated world."""
import pytest
import torch

from gpu_ipc_example_b200 import Communicator, ops
from gpu_ipc_example_b200.parallel import ColumnParallelLinear, RowParallelLinear

pytestmark = pytest.mark.gpu


def test_row_and_column_parallel_layers():
    world, M, K, N = 4, 64, 512, 512
    with Communicator.virtual(world, 0, staging_bytes=64 << 20) as comm:
        g = torch.Generator(device="cuda").manual_seed(0)
        x = torch.randn(M, K, device="cuda", generator=g).half()
        w = (torch.randn(N, K, device="cuda", generator=g) * 0.03).half()
        res = torch.randn(M, N, device="cuda", generator=g).half()
        gam = (torch.rand(N, device="cuda", generator=g) + 0.5).half()
        want = x.float() @ w.float().t()
        # row parallel: K is split
        xs = [c.contiguous() for c in x.chunk(world, dim=1)]
        ws = [c.contiguous() for c in w.chunk(world, dim=1)]
        for fused in ("gemm", "allreduce"):
            layer = RowParallelLinear(comm, ws, fused=fused)
            out = layer(xs)
            torch.cuda.synchronize()
            comm.check()
            torch.testing.assert_close(out[1].float(), want, atol=4e-2, rtol=2e-2)
            out, new_res = layer(xs, [res] * world, [gam] * world)
            torch.cuda.synchronize()
            comm.check()
            s = want + res.float()
            torch.testing.assert_close(new_res[2].float(), s, atol=5e-2, rtol=2e-2)
            torch.testing.assert_close(out[2].float(), s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * gam.float(),
                                       atol=5e-2, rtol=3e-2)
        # column parallel with the all-gather inside the GEMM: M is split on input, N on the weight
        col = ColumnParallelLinear(comm, [c.contiguous() for c in w.chunk(world, dim=0)], gather_input=True)
        outs = col([c.contiguous() for c in x.chunk(world, dim=0)])
        torch.cuda.synchronize()
        comm.check()
        torch.testing.assert_close(torch.cat([o.float() for o in outs], dim=1), want, atol=4e-2, rtol=2e-2)


def test_functional_api_with_a_world_of_one():
    comm = Communicator.virtual(1, 0, staging_bytes=8 << 20)
    ops.init(comm)
    try:
        x = torch.randn(4, 1, 14336, device="cuda").half()   # the reference smoke script's tensor shape
        y = x.clone()
        ops.all_reduce(y)
        torch.cuda.synchronize()
        assert torch.equal(x, y)
        out = torch.empty(4, 1, 14336, device="cuda", dtype=torch.float16)
        ops.all_gather_into_tensor(out, x)
        torch.cuda.synchronize()
        assert torch.equal(out, x)
    finally:
        ops.shutdown()
