"""The allocation-free all-reduce entry point (`b200ipc_allreduce_noalloc`, csrc/capi/no_alloc.h),
called through its exported C symbol the way a caller without an allocator would: raw device
pointers in, nothing allocated by the library.  Its result must equal what the communicator's
large-message all-reduce produces for the same inputs, on two calls in a row (the second call finds
the first call's leftovers in the shared scratch).  Collected last on purpose."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

PKG = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gpu_ipc_example_b200")
MAX_ELEMS = 256 * 1024


def _entry():
    from gpu_ipc_example_b200._ext import load

    load()  # makes sure the library is built
    lib = ctypes.CDLL(os.path.join(PKG, "libb200ipc.so"))
    f = lib.b200ipc_allreduce_noalloc
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    return f


def _call(f, ins, outs, dtype_code, status=None):
    world = len(ins)
    P = ctypes.c_void_p * world
    ip = P(*[t.data_ptr() for t in ins])
    op = P(*[t.data_ptr() for t in outs])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return f(ip, op, world, ins[0].numel(), dtype_code, stream, status)


@pytest.mark.parametrize("world,dtype", [(4, torch.float16), (8, torch.bfloat16), (2, torch.float16)])
def test_matches_the_communicator_twice_in_a_row(world, dtype):
    from gpu_ipc_example_b200 import Communicator

    torch.cuda.set_device(0)
    f = _entry()
    code = 0 if dtype == torch.float16 else 1
    tol = dict(atol=2e-2, rtol=4e-3) if dtype == torch.float16 else dict(atol=1.5e-1, rtol=3e-2)
    with Communicator.virtual(world, 0, staging_bytes=8 << 20) as comm:
        for call, n in enumerate((50003, MAX_ELEMS)):  # an odd size with a ragged tail, then the maximum
            xs = [torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(31 * call + r)).to(dtype)
                  for r in range(world)]
            ref = [torch.empty_like(x) for x in xs]
            comm.all_reduce(xs, ref, "bulk")  # the existing entry point
            outs = [torch.full_like(x, 3.0) for x in xs]
            status = (ctypes.c_uint32 * 8)()
            rc = _call(f, xs, outs, code, status)
            assert rc == 0
            torch.cuda.synchronize()
            comm.check()
            assert status[0] == 0, list(status)
            want = torch.stack([x.float() for x in xs]).sum(0)
            for o, r in zip(outs, ref):
                torch.testing.assert_close(o.float(), r.float(), **tol)
                torch.testing.assert_close(o.float(), want, **tol)


def test_in_place_and_refusals():
    torch.cuda.set_device(0)
    f = _entry()
    xs = [torch.ones(4096, device="cuda", dtype=torch.float16) * (r + 1) for r in range(4)]
    assert _call(f, xs, xs, 0) == 0
    torch.cuda.synchronize()
    for x in xs:
        assert torch.equal(x, torch.full_like(x, 10.0))
    big = [torch.zeros(MAX_ELEMS + 8, device="cuda", dtype=torch.float16) for _ in range(2)]
    assert _call(f, big, big, 0) == 2          # beyond the fixed scratch: refused, nothing launched
    three = [torch.zeros(64, device="cuda", dtype=torch.float16) for _ in range(3)]
    assert _call(f, three, three, 0) == 1      # world of 3 is not supported


def test_a_silent_rank_is_reported_whichever_rank_notices(monkeypatch):
    """A rank that sends nothing (test knob in the environment): some other rank's bounded wait runs out and
    the ONE status record the caller gets back says so - whichever emulated rank was the first to notice."""
    torch.cuda.set_device(0)
    f = _entry()
    monkeypatch.setenv("B200IPC_TIMEOUT_US", "50000")
    monkeypatch.setenv("B200IPC_NOALLOC_MUTE_RANK", "0")  # rank 0 is the silent one: ranks 1..3 are the ones that time out
    xs = [torch.ones(8192, device="cuda", dtype=torch.float16) for _ in range(4)]
    outs = [torch.zeros_like(x) for x in xs]
    status = (ctypes.c_uint32 * 8)()
    assert _call(f, xs, outs, 0, status) == 0
    torch.cuda.synchronize()
    assert status[0] in (1, 2), list(status)   # timed out, or told to stop by the one that did
    monkeypatch.delenv("B200IPC_NOALLOC_MUTE_RANK")
    status2 = (ctypes.c_uint32 * 8)()
    assert _call(f, xs, outs, 0, status2) == 0  # the next call clears the control words and works again
    torch.cuda.synchronize()
    assert status2[0] == 0 and float(outs[2][5]) == 4.0
