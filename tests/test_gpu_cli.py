"""The benchmark / verification binary on one GPU (`--virtual N`: N ranks as block rows of one cooperative
launch): verify mode against the CPU oracle with the reference's option letters (main.cpp:157-222 there),
and the machine-readable rows of a timed run."""
import json
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
MAIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gpu_ipc_example_b200", "bin", "main")


def _run(*args):
    p = subprocess.run([MAIN, *args], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    return p.returncode, p.stdout


@pytest.mark.parametrize("world", [2, 8])
def test_verify_mode_every_named_algorithm(world):
    algos = "small,simple,small_pcie_p,simple_pcie_p,small_ring,simple_ring,small_pcie,simple_pcie,oneshot,bulk,auto"
    if world % 2 == 0 and world > 2:
        algos += ",bisect"
    for n in ("14336", "1920", "65560"):
        rc, out = _run("--virtual", str(world), "-a", algos, "-v", "-n", n)
        assert rc == 0, out[-3000:]
        assert out.count(": ok") == len(algos.split(",")) and "FAILED" not in out, out[-3000:]


def test_verify_all_gather_and_reduce_scatter():
    rc, out = _run("--virtual", "4", "-a", "allgather_small,allgather_simple,allgather_direct,allgather_bulk,allgather_auto", "-v", "-n", "14336")
    assert rc == 0 and out.count(": ok") == 5, out[-3000:]
    rc, out = _run("--virtual", "4", "-a", "reduce_scatter,reduce_scatter:parallel:ll512,reduce_scatter:bulk", "-v", "-n", "16384")
    assert rc == 0 and out.count(": ok") == 3, out[-3000:]


def test_explicit_grid_and_bf16_random():
    # -g groups x -w sub-groups as in the reference's scripts (test/test_8tile_shapes.sh there), bf16, random data
    rc, out = _run("--virtual", "8", "-a", "simple", "-v", "-n", "14336", "-g", "2", "-w", "8", "-t", "bf16", "--random")
    assert rc == 0 and ": ok" in out, out[-3000:]
    rc, out = _run("--virtual", "8", "-a", "small", "-v", "-n", "14336", "-g", "3", "-w", "5")  # 15 wires: not a multiple of 8
    assert rc != 0 and "multiple" in out, out[-3000:]


def test_json_rows_of_a_timed_sweep(tmp_path):
    path = tmp_path / "rows.jsonl"
    rc, out = _run("--virtual", "2", "-a", "oneshot:ll512,simple_pcie_p", "--sweep", "10:12", "--samples", "2", "--json", str(path))
    assert rc == 0, out[-3000:]
    rows = [json.loads(line) for line in path.read_text().splitlines()]
    assert len(rows) == 6
    for r in rows:
        assert r["collective"] == "all_reduce" and r["world"] == 2 and r["us_min"] <= r["us_median"] <= r["us_max"]
        assert r["bytes"] == 2 * r["elements"] and r["busbw_GBs"] > 0
