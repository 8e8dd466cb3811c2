"""The flag-in-data schedules and wire formats on the CPU emulator (no GPU): the same schedule
templates the kernels run, with a scalar backend.  Covers the reference's verify matrix
(test/test_8tile_shapes.sh: odd sizes, odd grids) for every schedule x wire format x world."""
import ctypes

import numpy as np
import pytest

import emu

AR_OPS = ["parallel", "sequential", "ring", "bisect", "oneshot"]
AG_OPS = ["ag_ring", "ag_direct"]
PROTOS = ["LL8", "LL16", "LL128", "LL512"]


def _inputs(world, n, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal(n).astype(np.float16) for _ in range(world)]


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("op", AR_OPS)
@pytest.mark.parametrize("proto", PROTOS)
def test_allreduce_matches_fp32_sum(world, op, proto):
    for n in (128, 384, 1920, 14336, 777, 65536 + 2):
        ins = _inputs(world, n)
        outs = [np.zeros(n, np.float16) for _ in range(world)]
        unit = world if op == "parallel" else (world // 2 if op == "bisect" else 1)
        nwires = unit * 3 if n > 2000 else unit
        rc, st = emu.run_threads(world, op, proto, ins, outs, n, nwires)
        assert rc == 0, st
        want = np.sum(np.stack([x.astype(np.float32) for x in ins]), 0)
        for o in outs:
            np.testing.assert_allclose(o.astype(np.float32), want, atol=2e-2, rtol=4e-3)
            assert (o.view(np.uint16) == outs[0].view(np.uint16)).all(), "ranks must agree bit for bit"


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("op", AG_OPS)
@pytest.mark.parametrize("proto", ["LL16", "LL512"])
def test_allgather_is_rank_ordered_concatenation(world, op, proto):
    for n in (128, 1922, 14336):
        ins = _inputs(world, n, seed=1)
        outs = [np.zeros(n * world, np.float16) for _ in range(world)]
        rc, st = emu.run_threads(world, op, proto, ins, outs, n, 5)
        assert rc == 0, st
        want = np.concatenate(ins)
        for o in outs:
            assert (o.view(np.uint16) == want.view(np.uint16)).all()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("proto", PROTOS)
def test_reduce_scatter_back_to_back_on_the_same_rings(world, proto):
    """Rank r ends with slice r of the sum.  A sender gets no reply in this schedule, so consecutive
    launches alternate between the two halves of the ring (bit 1 of the sequence number)."""
    L = emu.lib()
    heaps = (ctypes.c_void_p * world)()
    seq = 0xE00F100E
    try:
        for it, n in enumerate((8 * world, 960 * world, 2 * world * 777, 14336, 8 * world)):
            ins = _inputs(world, n, seed=it)
            outs = [np.zeros(n // world, np.float16) for _ in range(world)]
            nwires = world * (3 if n > 2000 else 1)
            payload = {"LL8": 32, "LL16": 64, "LL128": 30, "LL512": 120}[proto]
            while -(-(n // world // 2) // ((nwires // world) * payload)) > 8:
                nwires += world
            rc, st = emu.run_threads(world, "reduce_scatter", proto, ins, outs, n, nwires, seq=seq, heaps=heaps)
            assert rc == 0, st
            want = np.sum(np.stack([x.astype(np.float32) for x in ins]), 0)
            c = n // world
            for r, o in enumerate(outs):
                np.testing.assert_allclose(o.astype(np.float32), want[r * c:(r + 1) * c], atol=2e-2, rtol=4e-3)
            assert L.b200emu_seq_advance(emu.OPS["reduce_scatter"], emu.PROTOS[proto], world, nwires, n) == 2
            seq = (seq + 2) & 0xFFFFFFFF
    finally:
        L.b200emu_free_heaps(world, heaps)


def test_reduce_scatter_refuses_more_steps_than_ring_slots():
    ins = _inputs(2, 1 << 16)
    outs = [np.zeros(1 << 15, np.float16) for _ in range(2)]
    rc, _ = emu.run_threads(2, "reduce_scatter", "LL8", ins, outs, 1 << 16, 2)
    assert rc == 2


def test_in_place_and_pattern_exact():
    """(i % 32) * (rank + 1): the reference's verify pattern (utils.hpp:15-19); exact in fp16."""
    world, n = 8, 14336
    i = np.arange(n) % 32
    for op, proto in (("parallel", "LL8"), ("parallel", "LL128"), ("bisect", "LL128"), ("ring", "LL512"), ("oneshot", "LL16")):
        bufs = [(i * (r + 1)).astype(np.float16) for r in range(world)]
        unit = 8 if op == "parallel" else (4 if op == "bisect" else 1)
        rc, st = emu.run_threads(world, op, proto, bufs, bufs, n, unit * 2, flags=1)  # round after every add, as the reference sums
        assert rc == 0, st
        want = (i * 36).astype(np.float16)
        for b in bufs:
            assert (b == want).all()


def test_bf16():
    world, n = 4, 4096
    rng = np.random.default_rng(3)
    f = [rng.standard_normal(n).astype(np.float32) for _ in range(world)]
    L = emu.lib()
    to_bf16 = np.vectorize(lambda v: L.b200emu_from_float(1, float(v)), otypes=[np.uint16])
    from_bf16 = np.vectorize(lambda v: L.b200emu_to_float(1, int(v)), otypes=[np.float32])
    ins = [to_bf16(x) for x in f]
    outs = [np.zeros(n, np.uint16) for _ in range(world)]
    rc, st = emu.run_threads(world, "parallel", "LL512", ins, outs, n, 4, dtype=1)
    assert rc == 0, st
    want = np.sum(np.stack([from_bf16(x) for x in ins]), 0)
    np.testing.assert_allclose(from_bf16(outs[0]), want, atol=1.5e-1, rtol=3e-2)


def test_sequence_numbers_across_launches_on_the_same_rings():
    """Successive launches with different schedules, formats and grids reuse the same scratch;
    flags only grow, so nothing stale is ever accepted."""
    world = 4
    L = emu.lib()
    heaps = (ctypes.c_void_p * world)()
    seq = 0xE00F100F  # the reference CLI's default first flag (main.cpp:185)
    plan = [("parallel", "LL8", 8, 4096), ("oneshot", "LL512", 3, 1000), ("ring", "LL16", 2, 20000), ("parallel", "LL512", 4, 300),
            ("bisect", "LL128", 6, 5000), ("sequential", "LL512", 5, 4096), ("oneshot", "LL16", 7, 64), ("parallel", "LL8", 4, 4096)]
    try:
        for rep in range(3):
            for op, proto, nwires, n in plan:
                ins = _inputs(world, n, seed=rep)
                outs = [np.zeros(n, np.float16) for _ in range(world)]
                rc, st = emu.run_threads(world, op, proto, ins, outs, n, nwires, seq=seq, heaps=heaps)
                assert rc == 0, (op, proto, st)
                want = np.sum(np.stack([x.astype(np.float32) for x in ins]), 0)
                np.testing.assert_allclose(outs[world - 1].astype(np.float32), want, atol=2e-2, rtol=4e-3)
                seq = (seq + L.b200emu_seq_advance(emu.OPS[op], emu.PROTOS[proto], world, nwires, n)) & 0xFFFFFFFF
    finally:
        L.b200emu_free_heaps(world, heaps)


def test_bad_geometry_is_refused():
    ins = _inputs(4, 128)
    outs = [np.zeros(128, np.float16) for _ in range(4)]
    rc, _ = emu.run_threads(4, "parallel", "LL8", ins, outs, 128, 6)  # 6 wires is not a multiple of 4 ranks
    assert rc == 2


# ----------------------------------------------------------------------------- wire images
def test_wire_images_match_the_documented_byte_layouts():
    flag = 0xABCD0123
    p = np.arange(1, 121, dtype=np.uint32)
    img = emu.wire_image("LL8", p[:32], flag)
    assert len(img) == 64 and (img[0::2] == p[:32]).all() and (img[1::2] == flag).all()
    img = emu.wire_image("LL16", p[:64], flag)
    assert len(img) == 128 and (img[0::2] == p[:64]).all() and (img[1::2] == flag).all()
    # 120/128: flags close each 64-byte half, the displaced dword travels in slot 30 (rt64_128.hpp:539-552)
    img = emu.wire_image("LL128", p[:30], flag)
    assert len(img) == 32
    assert img[15] == flag and img[31] == flag and img[30] == p[15]
    assert (img[:15] == p[:15]).all() and (img[16:30] == p[16:30]).all()
    # 480/512: a flag ends every 64 bytes; the 7 displaced dwords sit in slots 120..126 (rt64_128.hpp:202-226)
    img = emu.wire_image("LL512", p, flag)
    assert len(img) == 128
    assert all(img[16 * j + 15] == flag for j in range(8))
    assert [int(img[120 + j]) for j in range(7)] == [int(p[16 * j + 15]) for j in range(7)]
    for k in range(120):
        if k % 16 != 15:
            assert img[k] == p[k]


def test_scatter_sink_holds_the_expected_transaction_image():
    """Stage-level oracle: after a parallel all-reduce the scatter ring of rank 1 holds, at the slot
    addressed by (group, source rank, slot), rank 0's slice of chunk 1 packed with the step's flag."""
    world, n, nwires, seq = 2, 256, 2, 77
    L = emu.lib()
    heaps = (ctypes.c_void_p * world)()
    try:
        ins = _inputs(world, n, seed=9)
        outs = [np.zeros(n, np.float16) for _ in range(world)]
        rc, st = emu.run_threads(world, "parallel", "LL128", ins, outs, n, nwires, seq=seq, heaps=heaps)
        assert rc == 0, st
        scatter_off = L.b200emu_layout(1, 0)
        got = np.zeros(32, np.uint32)
        # group 0, source rank 0, slot 0 -> transaction index (0 * world + 0) * 8 + 0
        L.b200emu_peek(heaps[1], ctypes.c_uint64(scatter_off), ctypes.c_uint64(128), got.ctypes.data_as(ctypes.c_void_p))
        chunk_dw = 64  # 256 halves = 128 dwords, 2 chunks
        payload = ins[0].view(np.uint32)[chunk_dw:chunk_dw + 30]
        want = emu.wire_image("LL128", payload, seq)
        assert (got == want).all()
    finally:
        L.b200emu_free_heaps(world, heaps)


# ----------------------------------------------------------------------------- faults (host side only)
def test_silent_rank_ends_in_a_timeout_report_not_a_hang():
    world, n = 4, 4096
    ins = _inputs(world, n)
    outs = [np.zeros(n, np.float16) for _ in range(world)]
    rc, st = emu.run_threads(world, "parallel", "LL512", ins, outs, n, 4, timeout_ms=100, mute=2)
    assert rc == 1
    codes = [row[0] for row in st]
    assert 1 in codes  # somebody's bounded wait ran out (which wait is first depends on timing:
    # ranks stuck behind the silent one stop answering their own peers too)
    assert all(c in (1, 2) for c in codes)  # and everybody else was told to abort


def test_absent_rank_is_reported():
    world, n = 4, 1024
    ins = _inputs(world, n)
    outs = [np.zeros(n, np.float16) for _ in range(world)]
    rc, st = emu.run_threads(world, "oneshot", "LL16", ins, outs, n, 2, timeout_ms=100, skip=3)
    assert rc == 1
    assert any(row[0] == 1 for row in st)
    assert st[3][0] == 0  # the absent rank never ran


def test_stale_flag_is_not_accepted():
    """A launch that reuses an old sequence number finds old flags in the rings and must not take them
    for new data when the peer is silent."""
    world, n = 2, 512
    L = emu.lib()
    heaps = (ctypes.c_void_p * world)()
    try:
        ins = _inputs(world, n)
        outs = [np.zeros(n, np.float16) for _ in range(world)]
        assert emu.run_threads(world, "parallel", "LL8", ins, outs, n, 2, seq=10, heaps=heaps)[0] == 0
        rc, st = emu.run_threads(world, "parallel", "LL8", ins, outs, n, 2, seq=12, heaps=heaps, timeout_ms=100, mute=1)
        assert rc == 1
        timed_out = [row for row in st if row[0] == 1]
        assert timed_out and all(row[5] == 12 and row[6] == 10 for row in timed_out)  # expected 12, saw the stale 10
    finally:
        L.b200emu_free_heaps(world, heaps)
