"""One rank of the multi-GPU checks; started by tests/test_multi_gpu.py under torch.distributed.run.

Usage: multi_gpu_worker.py <mode>   with mode in {collectives, nvls, faults, hostmem}
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gpu_ipc_example_b200 import CollectiveError, Communicator  # noqa: E402


FAILURES = []


def soft(fn):
    """Record a failed check instead of raising: every rank keeps issuing the same sequence of
    collectives and reaches the common teardown, so no rank exits while others still wait on it."""
    def wrapped(*a, **k):
        try:
            return fn(*a, **k)
        except Exception as e:  # noqa: BLE001
            FAILURES.append(f"{fn.__name__}{a[1:3]}: {str(e)[:400]}")
    return wrapped


def gather_inputs(x):
    world = dist.get_world_size()
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x)
    return parts


@soft
def check_allreduce(comm, algo, n, dtype=torch.float16, symmetric=False, **kw):
    rank = dist.get_rank()
    g = torch.Generator(device="cuda").manual_seed(1000 + rank)
    x = torch.randn(n, device="cuda", generator=g).to(dtype)
    want = torch.stack([p.float() for p in gather_inputs(x)]).sum(0)
    if symmetric:
        buf = comm.empty([n], dtype)
        buf.copy_(x)
        comm.all_reduce(buf, None, algo, **kw)
        y = buf
    else:
        y = x.clone()
        comm.all_reduce(y, None, algo, **kw)
    torch.cuda.synchronize()
    comm.check()
    tol = dict(atol=2e-2, rtol=4e-3) if dtype == torch.float16 else dict(atol=1.5e-1, rtol=3e-2)
    torch.testing.assert_close(y.float(), want, **tol)
    # bit-identical on every rank
    ys = gather_inputs(y)
    for other in ys:
        assert torch.equal(other, ys[0]), f"{algo} n={n}: ranks differ"


@soft
def mode_collectives(comm, nvls):
    world = comm.world
    algos = ["small", "simple", "small_pcie_p", "simple_pcie_p", "small_ring", "simple_ring", "small_pcie", "simple_pcie",
             "oneshot", "oneshot:ll512", "bulk", "auto", "bisect"]
    if nvls:
        algos.append("nvls")
    for algo in algos:
        for n in (128, 1920, 14336, 65536 + 24, 1 << 20):
            check_allreduce(comm, algo, n)
        check_allreduce(comm, algo, 100003, torch.bfloat16)
    for algo in (["bulk", "nvls"] if nvls else ["bulk"]):
        check_allreduce(comm, algo, 8 * world * 4096, symmetric=True)
        assert comm.last_info.staged is False
        comm.free_symmetric()
    # stress: the same rings reused by different schedules thousands of times
    for it in range(300):
        check_allreduce(comm, ["simple_pcie_p", "oneshot", "simple", "small"][it % 4], [4096, 65536, 1920][it % 3])
    rank = dist.get_rank()
    for algo in ["allgather_small", "allgather_simple", "allgather_direct", "allgather_bulk"] + (["allgather_nvls"] if nvls else []):
        for n in (128, 14336, 1 << 18):
            x = (torch.rand(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rank)) * 2 - 1).half()
            want = torch.cat(gather_inputs(x))
            out = comm.all_gather(x, None, algo)
            torch.cuda.synchronize()
            comm.check()
            assert torch.equal(out, want), f"{algo} n={n}"
    for algo in (["bulk", "nvls"] if nvls else ["bulk"]):
        n = world * 40000
        x = torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rank)).half()
        want = torch.stack([p.float() for p in gather_inputs(x)]).sum(0)
        out = comm.reduce_scatter(x, None, algo)
        torch.cuda.synchronize()
        comm.check()
        shard = n // world
        torch.testing.assert_close(out.float(), want[rank * shard:(rank + 1) * shard], atol=2e-2, rtol=4e-3)
    # flag-in-data reduce-scatter: launches back to back (they alternate between the halves of the ring)
    for algo in ("parallel:ll512", "parallel:ll16", "parallel:ll128", "auto"):
        cases = []
        for it in range(40):
            n = world * (8 if it % 3 == 0 else (4096 if it % 3 == 1 else 2 * 777))
            x = torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1000 * it + rank)).half()
            cases.append((x, comm.reduce_scatter(x, None, algo)))
        torch.cuda.synchronize()
        comm.check()
        for x, out in cases[-6:]:
            want = torch.stack([p.float() for p in gather_inputs(x)]).sum(0)
            shard = x.numel() // world
            torch.testing.assert_close(out.float(), want[rank * shard:(rank + 1) * shard], atol=2e-2, rtol=4e-3)
    # fused all-reduce + residual + RMSNorm at decode shapes, and at a prefill shape (all-reduce + one local kernel)
    for rows, hidden in ((1, 8192), (32, 8192), (16, 3584), (512, 4096)):
        x = torch.randn(rows, hidden, device="cuda", generator=torch.Generator(device="cuda").manual_seed(50 + rank)).half()
        res = torch.randn(rows, hidden, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7)).half()
        gam = torch.rand(hidden, device="cuda", generator=torch.Generator(device="cuda").manual_seed(8)).half() + 0.5
        out, new_res = comm.allreduce_residual_rmsnorm(x, res, gam, 1e-5)
        torch.cuda.synchronize()
        comm.check()
        s = torch.stack([p.float() for p in gather_inputs(x)]).sum(0) + res.float()
        s16 = s.half().float()
        want = s16 * torch.rsqrt(s16.pow(2).mean(-1, keepdim=True) + 1e-5) * gam.float()
        torch.testing.assert_close(new_res.float(), s, atol=2e-2, rtol=4e-3)
        torch.testing.assert_close(out.float(), want, atol=3e-2, rtol=1e-2)


@soft
def check_linear(comm, M, K, N, dtype=torch.float16, norm=True):
    rank = dist.get_rank()
    g = torch.Generator(device="cuda").manual_seed(300 + rank)
    x = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(dtype)
    gr = torch.Generator(device="cuda").manual_seed(77)
    res = torch.randn(M, N, device="cuda", generator=gr).to(dtype)
    gam = (torch.rand(N, device="cuda", generator=gr) + 0.5).to(dtype)
    part = (x.float() @ w.float().t()).to(dtype)
    total = torch.stack([p.float() for p in gather_inputs(part)]).sum(0)
    if norm:
        out, new_res = comm.linear_allreduce(x, w, res, gam, 1e-5, fused=None if M == 128 else True)
        torch.cuda.synchronize()
        comm.check()
        s = (total + res.float()).to(dtype).float()
        want = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * gam.float()
        torch.testing.assert_close(new_res.float(), s, atol=4e-2, rtol=2e-2)
        torch.testing.assert_close(out.float(), want, atol=4e-2, rtol=2e-2)
        outs = gather_inputs(out.clone())
        for o in outs:
            assert torch.equal(o, outs[0]), "ranks differ"
    else:
        out = comm.linear_allreduce(x, w)
        torch.cuda.synchronize()
        comm.check()
        torch.testing.assert_close(out.float(), total, atol=4e-2, rtol=2e-2)


@soft
def check_ag_linear(comm, M, K, N):
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator(device="cuda").manual_seed(900 + rank)
    shard = torch.randn(M // world, K, device="cuda", generator=g).half()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).half()
    x = torch.cat(gather_inputs(shard))
    for _ in range(3):
        out = comm.allgather_linear(shard, w, fused=(_ != 2))
        torch.cuda.synchronize()
        comm.check()
        torch.testing.assert_close(out.float(), x.float() @ w.float().t(), atol=3e-2, rtol=1e-2)


@soft
def mode_linear(comm):
    for (M, K, N) in ((128, 256, 256), (320, 448, 512), (2048, 512, 1024), (16, 512, 192)):
        check_ag_linear(comm, M, K, N)
    for (M, K, N) in ((1, 448, 8192), (16, 448, 8192), (128, 256, 1024), (300, 512, 1024), (2048, 448, 2048)):
        check_linear(comm, M, K, N, norm=True)
        check_linear(comm, M, K, N, norm=False)
    for it in range(20):
        check_linear(comm, 32, 256, 512, norm=True)
    # the same kernel without an exchange (column-parallel projections of a decode step)
    g = torch.Generator(device="cuda").manual_seed(5 + dist.get_rank())
    for (M, K, N) in ((32, 1024, 1280), (5, 448, 256)):
        for _ in range(3):
            x = torch.randn(M, K, device="cuda", generator=g).half()
            w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).half()
            y = comm.linear(x, w)
            torch.cuda.synchronize()
            comm.check()
            torch.testing.assert_close(y.float(), x.float() @ w.float().t(), atol=3e-2, rtol=2e-2)


@soft
def mode_faults(comm):
    """Rank 1 sends nothing for one collective: every rank's bounded wait ends with a status,
    nobody hangs, and after a collective reset the communicator works again."""
    rank = dist.get_rank()
    comm.set_timeout_ms(200)
    x = torch.ones(4096, device="cuda", dtype=torch.float16)
    comm.all_reduce(x, None, "simple_pcie_p", flags=2 if rank == 1 else 0)
    torch.cuda.synchronize()
    failed = False
    try:
        comm.check()
    except CollectiveError as e:
        failed = True
        assert "bounded wait" in str(e) or "aborted" in str(e)
    flags = [None] * comm.world
    dist.all_gather_object(flags, failed)
    # the rank whose wait ran out reports a timeout, every rank it aborted reports that it was aborted:
    # nobody is left believing that its (partial) output is a sum
    assert all(flags), f"ranks that did not notice the failed collective: {[i for i, f in enumerate(flags) if not f]}"
    comm.reset()
    comm.set_timeout_ms(2000)
    check_allreduce(comm, "simple_pcie_p", 4096)
    check_allreduce(comm, "bulk", 1 << 16)


def main():
    mode = sys.argv[1]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    nvls = mode == "nvls"
    backing = "host-shm" if mode == "hostmem" else "auto"
    comm = Communicator.from_torch_distributed(local, staging_bytes=64 << 20, nvls=nvls, backing=backing)
    if dist.get_rank() == 0:
        print(f"world={comm.world} backing={comm.backing} nvls={comm.nvls_note if nvls else 'off'}", flush=True)
    try:
        if mode in ("collectives", "nvls"):
            if nvls and not comm.has_nvls:
                print("NVLS-UNAVAILABLE: " + comm.nvls_note, flush=True)
            mode_collectives(comm, nvls and comm.has_nvls)
        elif mode == "hostmem":
            for algo in ("small", "simple_pcie_p", "oneshot", "simple_ring"):
                check_allreduce(comm, algo, 14336)
        elif mode == "linear":
            mode_linear(comm)
        elif mode == "faults":
            mode_faults(comm)
    except Exception as e:  # noqa: BLE001
        FAILURES.append(str(e)[:400])
    torch.cuda.synchronize()
    everyone = [None] * dist.get_world_size()
    dist.all_gather_object(everyone, FAILURES[:5])
    bad = [f for fs in everyone for f in fs]
    comm.close()
    dist.barrier()
    if dist.get_rank() == 0:
        print("WORKER-OK" if not bad else "WORKER-FAILED:\n" + "\n".join(bad), flush=True)
    dist.destroy_process_group()
    sys.exit(1 if bad else 0)


if __name__ == "__main__":
    main()
