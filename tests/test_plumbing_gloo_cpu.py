"""fp16 all-reduce correctness without a GPU: two processes over gloo, shared-memory buffers in
place of IPC peer mappings, 65 536 halves per rank, N(0,1) seeded by rank, against an fp32 sum."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 4])
def test_allreduce_over_shared_memory_with_gloo_ranks(world):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29640 + world), os.path.join(HERE, "gloo_plumbing_worker.py")]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert p.returncode == 0 and "PLUMBING-OK" in p.stdout, p.stdout[-4000:]
