"""What a GPU rank leaves in its peers' scratch rings, byte for byte, against the definition of the wire
formats (the emulator's `wire_image`, built from proto/wire_format.h alone): sender and receiver of the
device backend share their packing code, so only a comparison with the format itself can tell a
consistent-but-wrong image from the right one.  Also the device-side trace ring.

The reference kept CPU simulators of its scratch contents for the same purpose
(allreduce.cpp:37-517, flag words at dword 15 / 31, displaced word at 30)."""
import numpy as np
import pytest
import torch

from gpu_ipc_example_b200 import Communicator

import emu

pytestmark = pytest.mark.gpu

PAYLOAD_DW = {"LL8": 32, "LL16": 64, "LL128": 30, "LL512": 120}
TXN_BYTES = {"LL8": 256, "LL16": 512, "LL128": 128, "LL512": 512}
PARALLEL_SLOTS = 8


@pytest.mark.parametrize("proto", ["LL8", "LL16", "LL128", "LL512"])
def test_scatter_and_gather_rings_hold_the_format_image(proto):
    world, n = 2, 512  # 256 dwords, two chunks of 128
    with Communicator.virtual(world, 0, staging_bytes=8 << 20, first_seq=0x1234) as comm:
        i = torch.arange(n, device="cuda") % 32
        xs = [(i * (r + 1) + r).to(torch.float16) for r in range(world)]  # small integers: every sum is exact
        src = [x.clone() for x in xs]
        comm.all_reduce(xs, None, f"parallel:{proto.lower()}", ctas=1, warps=2)  # one group of two wires per rank
        torch.cuda.synchronize()
        comm.check()
        flag = comm.last_info.first_flag
        lay = comm.heap_layout()
        pdw, txn = PAYLOAD_DW[proto], TXN_BYTES[proto]
        chunk_dw = 128
        # reduce-scatter: rank 0's wire for chunk 1 stored its slice into rank 1's scatter ring at
        # transaction (group 0 * world + source rank 0) * slots + slot 0
        got = comm.dump_heap(lay["scatter_off"], txn, local=1).numpy().view(np.uint32)
        payload = src[0].cpu().numpy().view(np.uint32)[chunk_dw:chunk_dw + pdw]
        want = emu.wire_image(proto, payload, flag)
        assert (got == want).all(), f"{proto} scatter image differs at dwords {np.nonzero(got != want)[0][:8]}"
        # all-gather: rank 1 (owner of chunk 1) stored the reduced slice into rank 0's gather ring at
        # transaction (group 0 * world + source rank 1) * slots + slot 0
        got = comm.dump_heap(lay["gather_off"] + (0 * world + 1) * PARALLEL_SLOTS * txn, txn, local=0).numpy().view(np.uint32)
        total = (src[0].float() + src[1].float()).to(torch.float16)
        payload = total.cpu().numpy().view(np.uint32)[chunk_dw:chunk_dw + pdw]
        want = emu.wire_image(proto, payload, flag)
        assert (got == want).all(), f"{proto} gather image differs at dwords {np.nonzero(got != want)[0][:8]}"
        assert torch.equal(xs[0], total) and torch.equal(xs[1], total)


def test_trace_ring_records_every_completed_wait():
    with Communicator.virtual(4, 0, staging_bytes=8 << 20) as comm:
        comm.set_trace(True)
        xs = [torch.randn(4096, device="cuda").half() for _ in range(4)]
        comm.all_reduce(xs, None, "simple_pcie_p", ctas=2, warps=4)
        torch.cuda.synchronize()
        comm.check()
        first = comm.last_info.first_flag
        events, total = comm.trace_events(0)
        # rank 0, 8 wires in 2 groups of 4: per step the owner wire completes 3 waits (scatter sink), the
        # other three wires one each (gather sink)
        steps = comm.last_info.steps
        assert total == len(events) == 2 * steps * (3 + 3)
        assert {e["site"] for e in events} == {0, 1}
        assert all(e["rank"] == 0 and 0 <= e["peer"] < 4 and e["peer"] != 0 and e["flag"] >= first for e in events)
        assert all(a["t_ns"] > 0 for a in events)
        comm.set_trace(False)
        comm.all_reduce(xs, None, "simple_pcie_p", ctas=2, warps=4)
        torch.cuda.synchronize()
        assert comm.trace_events(0)[1] == total  # nothing added once tracing is off
