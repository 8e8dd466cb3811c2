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


def test_functional_api_on_an_emulated_world_of_four():
    """The torch.distributed-shaped functions with real exchanges behind them: every argument is a list with
    one tensor per emulated rank."""
    world = 4
    comm = Communicator.virtual(world, 0, staging_bytes=32 << 20)
    ops.init(comm)
    try:
        g = torch.Generator(device="cuda").manual_seed(4)
        xs = [torch.randn(4, 1, 14336, device="cuda", generator=g).half() for _ in range(world)]  # the smoke script's shape
        want = torch.stack([x.float() for x in xs]).sum(0)
        ys = [x.clone() for x in xs]
        ops.all_reduce(ys)
        torch.cuda.synchronize()
        comm.check()
        for y in ys:
            torch.testing.assert_close(y.float(), want, atol=2e-2, rtol=4e-3)
            assert torch.equal(y, ys[0])
        outs = [torch.empty(world * 4, 1, 14336, device="cuda", dtype=torch.float16) for _ in range(world)]
        ops.all_gather_into_tensor(outs, xs)
        torch.cuda.synchronize()
        comm.check()
        for o in outs:
            assert torch.equal(o, torch.cat(xs))
        big = [torch.randn(world * 4096, device="cuda", generator=g).half() for _ in range(world)]
        shards = [torch.empty(4096, device="cuda", dtype=torch.float16) for _ in range(world)]
        ops.reduce_scatter_tensor(shards, big)
        torch.cuda.synchronize()
        comm.check()
        total = torch.stack([b.float() for b in big]).sum(0)
        for r, sh in enumerate(shards):
            torch.testing.assert_close(sh.float(), total[r * 4096:(r + 1) * 4096], atol=2e-2, rtol=4e-3)
        part = [torch.randn(8, 1024, device="cuda", generator=g).half() for _ in range(world)]
        res = [torch.randn(8, 1024, device="cuda", generator=torch.Generator(device="cuda").manual_seed(9)).half()] * world
        gam = [torch.ones(1024, device="cuda").half()] * world
        out, new_res = ops.allreduce_residual_rmsnorm(part, res, gam)
        torch.cuda.synchronize()
        comm.check()
        s = (torch.stack([p.float() for p in part]).sum(0) + res[0].float()).half().float()
        torch.testing.assert_close(new_res[3].float(), s, atol=2e-2, rtol=4e-3)
        torch.testing.assert_close(out[3].float(), s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5), atol=3e-2, rtol=1e-2)
    finally:
        ops.shutdown()


def test_soak_and_self_test_on_an_emulated_world():
    with Communicator.virtual(8, 0, staging_bytes=32 << 20) as comm:
        rep = comm.soak(("simple_pcie_p", "simple", "small_pcie_p", "small"), min_transactions=20000, nelems=1 << 18)
        assert all(v["mismatches"] == 0 and v["transactions"] >= 20000 for v in rep.values()), rep
        assert comm.self_test(5000) is True and comm.safe_protocols is False
        # a failed self-test makes `auto` avoid the 64-byte-segment formats
        comm._C.set_safe_protos(comm._h, True)
        xs = [torch.ones(4096, device="cuda", dtype=torch.float16) for _ in range(8)]
        comm.all_reduce(xs, None, "auto")
        torch.cuda.synchronize()
        comm.check()
        assert comm.last_info.proto == "LL16" and float(xs[0][0]) == 8.0
