"""Every schedule x wire format on a world emulated on ONE GPU (one cooperative launch
whose block rows are the ranks), against a plain PyTorch fp32 reference.

Mirrors the reference's verify sweeps (test/test_8tile_shapes.sh:4-19: odd sizes, odd
grids) and adds what its `-v` mode lacks: a failing comparison fails the test.
"""
import pytest
import torch

from gpu_ipc_example_b200 import Communicator, CollectiveError

pytestmark = pytest.mark.gpu

AR_ALGOS = ["small", "simple", "small_pcie_p", "simple_pcie_p", "bisect", "small_ring", "simple_ring", "small_pcie",
            "simple_pcie", "oneshot", "oneshot:ll8", "oneshot:ll128", "oneshot:ll512", "bisect:ll512", "sequential:ll8",
            "ring:ll128", "bulk"]
AG_ALGOS = ["allgather_small", "allgather_simple", "allgather_direct", "allgather_ring:ll8", "allgather_direct:ll128",
            "allgather_bulk"]
SHAPES = [128, 256, 384, 1280, 1920, 1024, 2048, 14336, 16384, 65536 + 24, 1 << 20]


@pytest.fixture(scope="module", params=[2, 4, 8])
def comm(request):
    c = Communicator.virtual(request.param, 0, staging_bytes=64 << 20)
    yield c
    c.close()


def _inputs(world, n, dtype, seed=0, uniform=False):
    xs = []
    for r in range(world):
        g = torch.Generator(device="cuda").manual_seed(seed * 100 + r)
        if uniform:
            x = torch.rand(n, generator=g, device="cuda") * 2 - 1
        else:
            x = torch.randn(n, generator=g, device="cuda")
        xs.append(x.to(dtype))
    return xs


def _check_allreduce(comm, algo, n, dtype, out_of_place=False, **kw):
    xs = _inputs(comm.world, n, dtype)
    want = torch.stack([x.float() for x in xs]).sum(0)
    if out_of_place:
        outs = [torch.full_like(x, 7.0) for x in xs]
        comm.all_reduce(xs, outs, algo, **kw)
    else:
        outs = [x.clone() for x in xs]
        comm.all_reduce(outs, None, algo, **kw)
    torch.cuda.synchronize()
    comm.check()
    tol = dict(atol=2e-2, rtol=4e-3) if dtype == torch.float16 else dict(atol=1.5e-1, rtol=3e-2)
    for o in outs:
        torch.testing.assert_close(o.float(), want, **tol)
        assert torch.equal(o, outs[0]), "ranks must hold bit-identical results"


@pytest.mark.parametrize("algo", AR_ALGOS)
def test_allreduce_shapes(comm, algo):
    for n in SHAPES:
        _check_allreduce(comm, algo, n, torch.float16)


@pytest.mark.parametrize("algo", ["small", "simple_pcie_p", "simple_ring", "bisect", "oneshot", "bulk"])
def test_allreduce_bf16_out_of_place_odd(comm, algo):
    for n in (777, 2049, 100003):
        _check_allreduce(comm, algo, n, torch.bfloat16, out_of_place=True)


@pytest.mark.parametrize("algo", ["small", "simple", "simple_pcie", "simple_ring"])
def test_allreduce_explicit_grids(comm, algo):
    # odd CTA counts as in the reference sweep; warps per CTA a multiple of the world size
    for ctas in (1, 7, 13, 19):
        _check_allreduce(comm, algo, 16384, torch.float16, ctas=ctas, warps=8)


def test_reference_grid_matrix(comm):
    """The reference's verify sweep (test/test_8tile_shapes.sh:4-19): group counts incl. odd ones x sub-group
    counts x shapes with ragged tails, on the default algorithm and one of each other schedule.  A grid the
    schedule cannot use (not a multiple of the world size, or more CTAs than can be resident at once) must be
    refused with an error, never run."""
    groups = (1, 2, 4, 8, 16, 32, 64, 7, 13, 15, 17, 19)
    subgroups = (1, 2, 4, 8, 32)  # the reference's 64 sub-groups of 16 lanes are 32 warps here
    shapes = (128, 256, 384, 1280, 1920, 1024, 2048, 14336, 16384)
    ran = refused = 0
    for algo in ("small", "simple", "simple_pcie", "simple_ring"):
        k = 0
        for g in groups:
            for w in subgroups:
                k += 1
                n = shapes[k % len(shapes)]
                try:
                    _check_allreduce(comm, algo, n, torch.float16, ctas=g, warps=w)
                    ran += 1
                except RuntimeError as e:
                    assert "multiple" in str(e) or "resident" in str(e) or "too many wires" in str(e), str(e)
                    refused += 1
    assert ran > 100 and ran + refused == 4 * len(groups) * len(subgroups)


def test_grid_not_multiple_of_world_is_refused(comm):
    if comm.world == 2:
        pytest.skip("every even grid is a multiple of 2")
    xs = _inputs(comm.world, 4096, torch.float16)
    with pytest.raises(RuntimeError, match="multiple"):
        comm.all_reduce(xs, None, "small", ctas=1, warps=comm.world + 1 if comm.world < 8 else 9)


def test_exact_pattern_matches_reference_oracle(comm):
    """(i % 32) * (rank + 1) in fp16: every partial sum is an exact integer, so results are bit exact."""
    n = 14336
    i = torch.arange(n, device="cuda") % 32
    for algo in ("small", "simple", "simple_pcie_p", "bisect", "simple_ring", "oneshot"):
        xs = [(i * (r + 1)).to(torch.float16) for r in range(comm.world)]
        want = (i * sum(r + 1 for r in range(comm.world))).to(torch.float16)
        comm.all_reduce(xs, None, algo, flags=1)
        torch.cuda.synchronize()
        comm.check()
        for x in xs:
            assert torch.equal(x, want)


@pytest.mark.parametrize("algo", AG_ALGOS)
def test_allgather(comm, algo):
    for n in (128, 1920, 14336, 65536 + 8, 1 << 18):
        xs = _inputs(comm.world, n, torch.float16, uniform=True)
        want = torch.cat(xs)
        outs = comm.all_gather(xs, None, algo)
        torch.cuda.synchronize()
        comm.check()
        for o in outs:
            assert torch.equal(o, want)


def test_allgather_in_place(comm):
    n = 4096
    xs = _inputs(comm.world, n, torch.float16, uniform=True)
    want = torch.cat(xs)
    outs = [torch.zeros(n * comm.world, dtype=torch.float16, device="cuda") for _ in range(comm.world)]
    views = []
    for r in range(comm.world):
        outs[r][r * n:(r + 1) * n] = xs[r]
        views.append(outs[r][r * n:(r + 1) * n])
    comm.all_gather(views, outs, "allgather_simple")
    torch.cuda.synchronize()
    comm.check()
    for o in outs:
        assert torch.equal(o, want)


def test_reduce_scatter(comm):
    for n in (comm.world * 1000, comm.world * 65536):
        xs = _inputs(comm.world, n, torch.float16)
        want = torch.stack([x.float() for x in xs]).sum(0)
        outs = comm.reduce_scatter(xs, None, "bulk")
        torch.cuda.synchronize()
        comm.check()
        shard = n // comm.world
        for r, o in enumerate(outs):
            torch.testing.assert_close(o.float(), want[r * shard:(r + 1) * shard], atol=2e-2, rtol=4e-3)


@pytest.mark.parametrize("algo", ["parallel:ll8", "parallel:ll16", "parallel:ll128", "parallel:ll512", "auto"])
def test_reduce_scatter_flag_in_data_back_to_back(comm, algo):
    """The flag-in-data reduce-scatter: a sender gets no reply, so launches alternate between the two
    halves of the ring.  Many launches in a row without a host sync, sizes mixed."""
    W = comm.world
    sizes = [8 * W, 960 * W, 2 * W * 777, 8 * W * 4096, 8 * W]
    cases = []
    for rep in range(4):
        for n in sizes:
            xs = _inputs(W, n, torch.float16)
            cases.append((xs, comm.reduce_scatter(xs, None, algo)))
            if algo != "auto":
                assert comm.last_info.sched == "parallel" and comm.last_info.launches == 1
    torch.cuda.synchronize()
    comm.check()
    for xs, outs in cases:
        want = torch.stack([x.float() for x in xs]).sum(0)
        shard = want.numel() // W
        for r, o in enumerate(outs):
            torch.testing.assert_close(o.float(), want[r * shard:(r + 1) * shard], atol=2e-2, rtol=4e-3)


def test_reduce_scatter_refuses_what_one_pass_cannot_hold(comm):
    n = 8 * comm.world * (1 << 18)
    xs = [torch.zeros(n, dtype=torch.float16, device="cuda") for _ in range(comm.world)]
    with pytest.raises(RuntimeError, match="more than the"):
        comm.reduce_scatter(xs, None, "parallel:ll8")
    xs = [torch.zeros(6 << 20, dtype=torch.float16, device="cuda") for _ in range(comm.world)]  # 12 MiB
    outs = comm.reduce_scatter(xs, None, "auto")  # above 8 MiB auto takes the barrier-based kernel
    torch.cuda.synchronize()
    comm.check()
    assert comm.last_info.sched in ("bulk", "nvls") and float(outs[0].abs().max()) == 0.0


def test_symmetric_tensors_are_zero_copy(comm):
    n = 8 * comm.world * 1024
    bufs = comm.empty([n], torch.float16)
    xs = _inputs(comm.world, n, torch.float16)
    for b, x in zip(bufs, xs):
        b.copy_(x)
    want = torch.stack([x.float() for x in xs]).sum(0)
    comm.all_reduce(bufs, None, "bulk")
    torch.cuda.synchronize()
    comm.check()
    assert comm.last_info.staged is False
    for b in bufs:
        torch.testing.assert_close(b.float(), want, atol=2e-2, rtol=4e-3)
    comm.free_symmetric()


def test_many_launches_keep_flags_in_step(comm):
    """Alternating schedules, sizes and geometries on the same rings: stale flags must never match."""
    algos = ["small", "oneshot", "simple_pcie_p", "simple_ring", "bisect", "simple_pcie", "oneshot:ll512", "simple"]
    sizes = [128, 8192, 1920, 65536, 384, 14336]
    for it in range(48):
        _check_allreduce(comm, algos[it % len(algos)], sizes[it % len(sizes)], torch.float16)


def test_sequence_wrap_resets_the_rings(comm):
    comm.set_seq(0xFFFFFFFA)
    for _ in range(6):
        _check_allreduce(comm, "simple_pcie_p", 65536, torch.float16)
    assert comm.seq < 0x80000000


def test_checkpoint_and_resume_of_the_only_state():
    """A communicator's state is its flag sequence number: a new communicator that starts from the saved one
    keeps producing flags no old ring entry can match."""
    with Communicator.virtual(4, 0, staging_bytes=16 << 20) as a:
        for n in (4096, 70000):
            _check_allreduce(a, "simple", n, torch.float16)
        state = a.state_dict()
        assert state["seq"] > 0 and state["world"] == 4
    with Communicator.virtual(4, 0, staging_bytes=16 << 20) as b:
        b.load_state_dict(state)
        assert b.seq == state["seq"]
        for n in (4096, 70000):
            _check_allreduce(b, "simple_pcie_p", n, torch.float16)
        assert b.seq > state["seq"]
    with Communicator.virtual(2, 0, staging_bytes=16 << 20) as c:
        with pytest.raises(ValueError):
            c.load_state_dict(state)


def test_auto_picks_by_size(comm):
    # the built-in table (measured on NVLink) must at least be correct at every size class
    for n in (1024, 70000, 300000, 1 << 20, 3 << 20):
        _check_allreduce(comm, "auto", n, torch.float16)
    assert comm.last_info.sched != "oneshot"
    # explicit cut-offs override the table
    comm.set_thresholds(32 << 10, 1 << 20)
    _check_allreduce(comm, "auto", 1024, torch.float16)
    assert comm.last_info.sched == "oneshot"
    _check_allreduce(comm, "auto", 256 * 1024, torch.float16)
    assert comm.last_info.sched == "parallel"
    _check_allreduce(comm, "auto", 2 * 1024 * 1024, torch.float16)
    assert comm.last_info.sched in ("bulk", "nvls")
    comm.set_thresholds(0, 0)


def test_fused_allreduce_residual_rmsnorm(comm):
    for rows, hidden in ((1, 8192), (4, 8192), (32, 8192), (16, 1024), (3, 4104)):
        xs = [t.view(rows, hidden) for t in _inputs(comm.world, rows * hidden, torch.float16, seed=3)]
        res = [torch.randn(rows, hidden, device="cuda", generator=torch.Generator(device="cuda").manual_seed(11)).half()
               for _ in range(comm.world)]
        gam = [torch.rand(hidden, device="cuda", generator=torch.Generator(device="cuda").manual_seed(12)).half() + 0.5
               for _ in range(comm.world)]
        outs, new_res = comm.allreduce_residual_rmsnorm(xs, res, gam, 1e-5)
        torch.cuda.synchronize()
        comm.check()
        s = torch.stack([x.float() for x in xs]).sum(0) + res[0].float()
        s16 = s.half().float()
        want = s16 * torch.rsqrt(s16.pow(2).mean(-1, keepdim=True) + 1e-5) * gam[0].float()
        for o, nr in zip(outs, new_res):
            torch.testing.assert_close(nr.float(), s, atol=2e-2, rtol=4e-3)
            torch.testing.assert_close(o.float(), want, atol=3e-2, rtol=1e-2)


def test_fused_allreduce_scale_cast(comm):
    n = 40000
    xs = _inputs(comm.world, n, torch.float16, seed=5)
    outs = comm.allreduce_scale_cast(xs, 0.125, torch.bfloat16)
    torch.cuda.synchronize()
    comm.check()
    want = torch.stack([x.float() for x in xs]).sum(0) * 0.125
    for o in outs:
        assert o.dtype == torch.bfloat16
        torch.testing.assert_close(o.float(), want, atol=5e-2, rtol=2e-2)


def test_bounded_wait_reports_instead_of_hanging():
    """A rank that sends nothing: the others' waits run out (50 ms limit), the kernel returns,
    the status block says who was waited for, and after reset() the communicator works again."""
    c = Communicator.virtual(2, 0, staging_bytes=8 << 20, timeout_ms=50)
    try:
        xs = _inputs(2, 4096, torch.float16)
        c.all_reduce(xs, None, "small", flags=2)  # FLAG_MUTE_SENDS on every emulated rank
        torch.cuda.synchronize()
        with pytest.raises(CollectiveError, match="bounded wait ran out"):
            c.check()
        sts = [c.status(i) for i in range(2)]
        assert all(st["code"] != 0 for st in sts), "every rank of a failed collective must know about it"
        timed_out = [st for st in sts if st["code"] == 1]
        assert timed_out and all(st["expected"] != st["seen"] for st in timed_out)
        c.reset()
        c.set_timeout_ms(2000)
        _check_allreduce(c, "small", 4096, torch.float16)
        xs = _inputs(2, 1 << 16, torch.float16)
        c.set_timeout_ms(50)
        c.all_reduce(xs, None, "bulk", flags=2)
        torch.cuda.synchronize()
        with pytest.raises(CollectiveError):
            c.check()
        c.reset()
        c.set_timeout_ms(2000)
        _check_allreduce(c, "bulk", 1 << 16, torch.float16)
    finally:
        c.close()


def test_device_side_sequence_numbers_survive_graph_replay():
    c = Communicator.virtual(4, 0, staging_bytes=8 << 20, device_seq=True)
    try:
        n = 8192
        xs = _inputs(4, n, torch.float16)
        src = [x.clone() for x in xs]
        want = torch.stack([x.float() for x in src]).sum(0)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            c.all_reduce(xs, None, "simple_pcie_p")  # warm-up outside the graph
            s.synchronize()
            for x, y in zip(xs, src):
                x.copy_(y)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                c.all_reduce(xs, None, "simple_pcie_p")
                c.all_reduce(xs, None, "oneshot")
            for _ in range(3):
                for x, y in zip(xs, src):
                    x.copy_(y)
                g.replay()
                s.synchronize()
                c.check()
                for x in xs:
                    torch.testing.assert_close(x.float(), want * 4, atol=1e-1, rtol=1e-2)
    finally:
        c.close()
