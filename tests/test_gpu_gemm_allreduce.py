"""The tcgen05/TMA row-parallel GEMM fused with its all-reduce (and residual + RMSNorm), against a
plain PyTorch fp32 reference.  World sizes above one are emulated on the single GPU (one cooperative
launch, block rows are ranks), which exercises the peer stores, flags and the delivery counter."""
import pytest
import torch

from gpu_ipc_example_b200 import Communicator

pytestmark = pytest.mark.gpu


def _mk(world, M, K, N, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    xs = [torch.randn(M, K, device="cuda", generator=g).to(dtype) for _ in range(world)]
    ws = [(torch.randn(N, K, device="cuda", generator=g) * 0.02).to(dtype) for _ in range(world)]
    res = torch.randn(M, N, device="cuda", generator=g).to(dtype)
    gam = (torch.rand(N, device="cuda", generator=g) + 0.5).to(dtype)
    return xs, ws, res, gam


def _ref(xs, ws):
    dtype = xs[0].dtype
    # every rank's partial product is rounded to the element type before the sum, as the kernel does
    return torch.stack([(x.float() @ w.float().t()).to(dtype).float() for x, w in zip(xs, ws)]).sum(0)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_gemm_allreduce_plain(world):
    with Communicator.virtual(world, 0, staging_bytes=96 << 20) as comm:
        for (M, K, N) in ((128, 256, 256), (1, 512, 1024), (16, 448, 512), (300, 512, 1024), (2048, 448, 1024)):
            xs, ws, _, _ = _mk(world, M, K, N, torch.float16, seed=M)
            outs = comm.linear_allreduce(xs, ws)
            torch.cuda.synchronize()
            comm.check()
            want = _ref(xs, ws)
            for o in outs:
                torch.testing.assert_close(o.float(), want, atol=3e-2, rtol=1e-2)


@pytest.mark.parametrize("world", [1, 2, 8])
def test_local_linear_on_the_weight_streaming_kernel(world):
    """`Communicator.linear`: the decode-sized kernel as a plain GEMM (no exchange); every emulated rank gets
    its own product.  Called twice per shape: the fp32 scratch must be left clean for the next launch."""
    with Communicator.virtual(world, 0, staging_bytes=96 << 20) as comm:
        for dtype in (torch.float16, torch.bfloat16):
            for (M, K, N) in ((1, 512, 256), (32, 1024, 1280), (7, 448, 128), (16, 8192, 1024)):
                for rep in range(2):
                    xs, ws, _, _ = _mk(world, M, K, N, dtype, seed=M + rep)
                    outs = comm.linear(xs, ws)
                    torch.cuda.synchronize()
                    comm.check()
                    assert comm.last_info.launches == 1
                    for x, w, o in zip(xs, ws, outs):
                        torch.testing.assert_close(o.float(), x.float() @ w.float().t(), atol=3e-2 if dtype == torch.float16 else 1.5e-1,
                                                   rtol=2e-2)
        # shapes the kernel does not take go to the framework's matmul
        xs, ws, _, _ = _mk(world, 40, 256, 192, torch.float16)
        outs = comm.linear(xs, ws)
        for x, w, o in zip(xs, ws, outs):
            torch.testing.assert_close(o.float(), x.float() @ w.float().t(), atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("world", [1, 8])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemm_allreduce_residual_rmsnorm(world, dtype):
    with Communicator.virtual(world, 0, staging_bytes=96 << 20) as comm:
        for (M, K, N) in ((1, 448, 8192), (16, 448, 8192), (128, 448, 8192), (200, 256, 1024)):
            xs, ws, res, gam = _mk(world, M, K, N, dtype, seed=7 + M)
            out, new_res = comm.linear_allreduce(xs, ws, [res] * world, [gam] * world, 1e-5)
            torch.cuda.synchronize()
            comm.check()
            s = (_ref(xs, ws) + res.float()).to(dtype).float()
            want = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * gam.float()
            tol = dict(atol=4e-2, rtol=2e-2) if dtype == torch.float16 else dict(atol=2.5e-1, rtol=5e-2)
            for o, r in zip(out, new_res):
                torch.testing.assert_close(r.float(), s, **tol)
                torch.testing.assert_close(o.float(), want, **tol)


def test_repeated_calls_reuse_the_workspace():
    with Communicator.virtual(4, 0, staging_bytes=64 << 20) as comm:
        for it in range(6):
            xs, ws, res, gam = _mk(4, 64, 256, 512, torch.float16, seed=it)
            out, new_res = comm.linear_allreduce(xs, ws, [res] * 4, [gam] * 4)
            torch.cuda.synchronize()
            comm.check()
            s = (_ref(xs, ws) + res.float()).half().float()
            torch.testing.assert_close(new_res[3].float(), s, atol=4e-2, rtol=2e-2)


def test_result_of_one_call_is_the_residual_of_the_next():
    """Calls of one shape alternate between two sets of output buffers: a decoder chains them without copies."""
    with Communicator.virtual(2, 0, staging_bytes=64 << 20) as comm:
        xs, ws, res, gam = _mk(2, 16, 256, 512, torch.float16, seed=11)
        _, r1 = comm.linear_allreduce(xs, ws, [res] * 2, [gam] * 2)
        _, r2 = comm.linear_allreduce(xs, ws, r1, [gam] * 2)
        out3, r3 = comm.linear_allreduce(xs, ws, r2, [gam] * 2)
        torch.cuda.synchronize()
        comm.check()
        assert r1[0].data_ptr() != r2[0].data_ptr() and r1[0].data_ptr() == r3[0].data_ptr()
        y = _ref(xs, ws)
        s1 = (y + res.float()).half().float()
        s2 = (y + s1).half().float()
        s3 = (y + s2).half().float()
        torch.testing.assert_close(r2[1].float(), s2, atol=4e-2, rtol=2e-2)
        torch.testing.assert_close(r3[0].float(), s3, atol=6e-2, rtol=2e-2)
        want = s3 * torch.rsqrt(s3.pow(2).mean(-1, keepdim=True) + 1e-5) * gam.float()
        torch.testing.assert_close(out3[0].float(), want, atol=6e-2, rtol=2e-2)


def test_graph_replay_with_device_side_counters():
    with Communicator.virtual(4, 0, staging_bytes=64 << 20, device_seq=True) as comm:
        xs, ws, res, gam = _mk(4, 32, 256, 512, torch.float16, seed=3)
        s = (_ref(xs, ws) + res.float()).half().float()
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            comm.linear_allreduce(xs, ws, [res] * 4, [gam] * 4)  # allocates the workspace outside the capture
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                out, new_res = comm.linear_allreduce(xs, ws, [res] * 4, [gam] * 4)
                out, new_res = comm.linear_allreduce(xs, ws, [res] * 4, [gam] * 4)
            for _ in range(3):
                for t in new_res:
                    t.zero_()
                g.replay()
                stream.synchronize()
                comm.check()
                torch.testing.assert_close(new_res[2].float(), s, atol=4e-2, rtol=2e-2)


@pytest.mark.parametrize("world", [1, 2, 8])
def test_allgather_linear(world):
    """All-gather fused into the GEMM: row-sharded X, column-parallel W, against fp32 matmul."""
    with Communicator.virtual(world, 0, staging_bytes=96 << 20) as comm:
        for (M, K, N) in ((128, 256, 256), (8 * 40, 448, 512), (2048, 512, 1024), (16, 512, 192)):
            g = torch.Generator(device="cuda").manual_seed(M + world)
            x = torch.randn(M, K, device="cuda", generator=g).half()
            ws = [(torch.randn(N, K, device="cuda", generator=g) * 0.05).half() for _ in range(world)]
            shards = list(x.chunk(world, dim=0))
            for rep in range(3):  # the gathered-input buffer alternates between two halves
                outs = comm.allgather_linear([s.contiguous() for s in shards], ws, fused=True if rep < 2 else None)
                torch.cuda.synchronize()
                comm.check()
                for o, w in zip(outs, ws):
                    torch.testing.assert_close(o.float(), x.float() @ w.float().t(), atol=3e-2, rtol=1e-2)
