"""One rank of the CPU plumbing check: torch.distributed over gloo gives rank and world, a POSIX
shared-memory segment stands in for the peer mappings a GPU world gets from the handle exchange,
and the emulator runs this rank's side of an fp16 all-reduce of 65 536 N(0,1) values seeded by rank.
Started by tests/test_plumbing_gloo_cpu.py under torch.distributed.run."""
import ctypes
import os
import sys
from multiprocessing import shared_memory

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import emu  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    L = emu.lib()
    heap = int(L.b200emu_heap_bytes())
    name = [f"b200ipc_test_{os.getpid()}" if rank == 0 else None]
    dist.broadcast_object_list(name, src=0)
    if rank == 0:
        seg = shared_memory.SharedMemory(name=name[0], create=True, size=heap * world)  # zero-filled, pages on demand
    dist.barrier()
    if rank != 0:
        seg = shared_memory.SharedMemory(name=name[0])
    base = ctypes.addressof(ctypes.c_char.from_buffer(seg.buf))
    ok = True
    seq = 1
    n = 65536
    for op, proto, nwires in (("parallel", "LL8", 8), ("parallel", "LL512", 4), ("sequential", "LL512", 3), ("ring", "LL16", 4),
                              ("bisect", "LL128", 4), ("oneshot", "LL512", 6)):
        g = torch.Generator().manual_seed(rank)
        x = torch.randn(n, generator=g).to(torch.float16)
        xs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(xs, x)
        want = torch.stack([t.float() for t in xs]).sum(0)
        inp = x.numpy().copy()
        out = np.zeros(n, np.float16)
        st = (ctypes.c_uint32 * 8)()
        rc = L.b200emu_run_rank(base, rank, world, emu.OPS[op], emu.PROTOS[proto], 0, inp.ctypes.data, out.ctypes.data, n, nwires,
                                seq, 0, 5000, st)
        seq += L.b200emu_seq_advance(emu.OPS[op], emu.PROTOS[proto], world, nwires, n)
        good = rc == 0 and torch.allclose(torch.from_numpy(out).float(), want, atol=2e-2, rtol=4e-3)
        if not good:
            print(f"rank {rank}: {op}/{proto} failed rc={rc} status={list(st)}", flush=True)
        ok = ok and good
        dist.barrier()
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    del base
    seg.close()
    dist.barrier()
    if rank == 0:
        seg.unlink()
        print("PLUMBING-OK" if all(flags) else "PLUMBING-FAILED", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if all(flags) else 1)


if __name__ == "__main__":
    main()
