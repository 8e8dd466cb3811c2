"""Bit-exact soak of the flag-in-data wire formats over the real links.

    python -m torch.distributed.run --nproc-per-node 8 -m gpu_ipc_example_b200.soak --transactions 1000000

Every rank all-reduces the reference's integer pattern (i % 32) * (rank + 1) in fp16 again and again
(refilled before every launch) with each wire format until every format has moved the requested number
of warp transactions per rank, and counts result elements that differ from the exact sum.  One JSON
line per algorithm from rank 0; exit code 1 if anything differed.  Without a launcher it soaks an
emulated world of 8 ranks on one GPU (same kernels, no link).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--transactions", type=int, default=1000000, help="warp transactions per rank and algorithm")
    ap.add_argument("--algos", nargs="*", default=["simple_pcie_p", "simple", "small_pcie_p", "small", "simple_ring", "simple_pcie", "oneshot:ll512"])
    ap.add_argument("--nelems", type=int, default=1 << 22)
    args = ap.parse_args()
    from gpu_ipc_example_b200 import Communicator

    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        comm = Communicator.from_torch_distributed(local, staging_bytes=64 << 20)
    else:
        comm = Communicator.virtual(8, local, staging_bytes=64 << 20)
    rep = comm.soak(tuple(args.algos), args.transactions, args.nelems)
    bad = sum(v["mismatches"] for v in rep.values())
    if world > 1:
        t = torch.tensor([bad], device="cuda")
        dist.all_reduce(t)
        bad = int(t.item())
    if int(os.environ.get("RANK", 0)) == 0:
        for algo, v in rep.items():
            print(json.dumps({"soak": algo, "world": comm.world, "links": "nvlink" if world > 1 else "emulated on one GPU", **v}), flush=True)
        print(json.dumps({"soak": "total", "mismatches_all_ranks": bad}), flush=True)
    comm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
