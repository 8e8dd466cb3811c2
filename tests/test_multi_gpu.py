"""Real multi-GPU checks: one process per GPU under torch.distributed.run, peers mapped through the
CUDA handle exchange.  Skipped on boxes with fewer than two GPUs (the virtual-world tests cover the
protocol logic there)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode, nproc, extra_env=None, timeout=600):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(29511 + nproc), os.path.join(HERE, "multi_gpu_worker.py"), mode]
    p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout)
    assert p.returncode == 0 and "WORKER-OK" in p.stdout, p.stdout[-6000:]
    return p.stdout


def _worlds():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [w for w in (2, 4, 8) if w <= n]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_collectives(world):
    if world not in _worlds():
        pytest.skip("not enough GPUs")
    _run("collectives", world)


@pytest.mark.parametrize("world", [2, 8])
def test_nvls(world):
    if world not in _worlds():
        pytest.skip("not enough GPUs")
    out = _run("nvls", world)
    if "NVLS-UNAVAILABLE" in out:
        pytest.skip("multicast not available on this box: " + out)


@pytest.mark.parametrize("world", [2, 8])
def test_fused_gemm_allreduce(world):
    if world not in _worlds():
        pytest.skip("not enough GPUs")
    _run("linear", world)


def test_host_memory_scratch():
    if 2 not in _worlds():
        pytest.skip("not enough GPUs")
    _run("hostmem", 2)


def test_silent_rank_is_detected_not_hung():
    if 2 not in _worlds():
        pytest.skip("not enough GPUs")
    # in-switch reduction off everywhere for a test in which a rank misbehaves
    _run("faults", 2, {"NCCL_NVLS_ENABLE": "0"})
