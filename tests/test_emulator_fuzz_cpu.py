"""Randomised sizes, grids and schedules on the CPU emulator (hypothesis): the tail handling and the
ring addressing must hold for any element count and any legal wire count."""
import numpy as np
from hypothesis import given, settings, strategies as st

import emu

AR = ["parallel", "sequential", "ring", "bisect", "oneshot"]
PROTOS = ["LL8", "LL16", "LL128", "LL512"]


@settings(max_examples=60, deadline=None)
@given(world=st.sampled_from([2, 4, 8]), op=st.sampled_from(AR), proto=st.sampled_from(PROTOS),
       n=st.integers(min_value=1, max_value=6000), groups=st.integers(min_value=1, max_value=5), seed=st.integers(0, 1000))
def test_allreduce_any_size_any_grid(world, op, proto, n, groups, seed):
    unit = world if op == "parallel" else (world // 2 if op == "bisect" else 1)
    nwires = unit * groups
    rng = np.random.default_rng(seed)
    ins = [rng.standard_normal(n).astype(np.float16) for _ in range(world)]
    outs = [np.full(n + 3, 7.0, np.float16) for _ in range(world)]  # 3 guard elements behind the output
    rc, st_ = emu.run_threads(world, op, proto, ins, [o[:n] for o in outs], n, nwires, seq=seed + 1)
    assert rc == 0, st_
    want = np.sum(np.stack([x.astype(np.float32) for x in ins]), 0)
    for o in outs:
        np.testing.assert_allclose(o[:n].astype(np.float32), want, atol=2e-2, rtol=4e-3)
        assert (o[n:] == 7.0).all(), "wrote past the end of the buffer"


@settings(max_examples=30, deadline=None)
@given(world=st.sampled_from([2, 4, 8]), op=st.sampled_from(["ag_ring", "ag_direct"]), proto=st.sampled_from(PROTOS),
       half_n=st.integers(min_value=1, max_value=2000), nwires=st.integers(min_value=1, max_value=6))
def test_allgather_any_size_any_grid(world, op, proto, half_n, nwires):
    n = 2 * half_n
    rng = np.random.default_rng(half_n)
    ins = [rng.standard_normal(n).astype(np.float16) for _ in range(world)]
    outs = [np.zeros(n * world, np.float16) for _ in range(world)]
    rc, st_ = emu.run_threads(world, op, proto, ins, outs, n, nwires)
    assert rc == 0, st_
    want = np.concatenate(ins).view(np.uint16)
    for o in outs:
        assert (o.view(np.uint16) == want).all()


@settings(max_examples=40, deadline=None)
@given(world=st.sampled_from([2, 4, 8]), proto=st.sampled_from(PROTOS), k=st.integers(min_value=1, max_value=1500),
       groups=st.integers(min_value=1, max_value=4), launches=st.integers(min_value=1, max_value=4))
def test_reduce_scatter_any_size_any_grid_back_to_back(world, proto, k, groups, launches):
    """Slices of k dwords per rank, several launches in a row on the same rings (they alternate between the two halves)."""
    import ctypes

    n = 2 * world * k
    payload = {"LL8": 32, "LL16": 64, "LL128": 30, "LL512": 120}[proto]
    while -(-k // (groups * payload)) > 8:  # a launch takes at most 8 steps
        groups += 1
    heaps = (ctypes.c_void_p * world)()
    seq = 0x1000 + k
    try:
        for it in range(launches):
            rng = np.random.default_rng(k + it)
            ins = [rng.standard_normal(n).astype(np.float16) for _ in range(world)]
            outs = [np.full(n // world + 2, 5.0, np.float16) for _ in range(world)]
            rc, st_ = emu.run_threads(world, "reduce_scatter", proto, ins, [o[:n // world] for o in outs], n, world * groups,
                                      seq=seq, heaps=heaps)
            assert rc == 0, st_
            want = np.sum(np.stack([x.astype(np.float32) for x in ins]), 0)
            c = n // world
            for r, o in enumerate(outs):
                np.testing.assert_allclose(o[:c].astype(np.float32), want[r * c:(r + 1) * c], atol=2e-2, rtol=4e-3)
                assert (o[c:] == 5.0).all(), "wrote past the end of the slice"
            seq += 2
    finally:
        emu.lib().b200emu_free_heaps(world, heaps)
