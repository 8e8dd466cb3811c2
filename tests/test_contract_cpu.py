"""Repository-level contracts that need no GPU: the reference arm of bench.py, the build entry point,
host fp16/bf16 arithmetic of the oracle."""
import json
import os
import subprocess
import sys

import numpy as np

import emu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference"], stdout=subprocess.PIPE, text=True,
                       timeout=120)
    assert p.returncode == 0
    d = json.loads(p.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and "unavailable" in d


def test_build_entry_point_compiles_and_imports():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as g

    g.build()
    for name in ("_C.so", "libb200ipc.so", "libb200ipc_emu.so", "bin/main", "bin/list_devices"):
        assert os.path.exists(os.path.join(ROOT, "gpu_ipc_example_b200", name)), name


def test_cli_help_and_unknown_algorithm():
    exe = os.path.join(ROOT, "gpu_ipc_example_b200", "bin", "main")
    p = subprocess.run([exe, "--help"], stdout=subprocess.PIPE, text=True, timeout=60)
    assert p.returncode == 0
    for flag in ("-n,", "-g,", "-w,", "-f,", "-s,", "-v,", "-a,", "-i,", "-l,", "-p,"):  # the reference's letters (main.cpp:177-198)
        assert flag in p.stdout


def test_host_half_conversion_round_trips():
    L = emu.lib()
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(2000).astype(np.float32) * s for s in (1e-6, 1e-3, 1.0, 100.0, 6e4)])
    for v in vals:
        want = np.float16(v)
        got = np.uint16(L.b200emu_from_float(0, float(v))).view(np.float16)
        assert got == want or (np.isnan(got) and np.isnan(want)) or (np.isinf(got) and np.isinf(want)), (v, got, want)
        if np.isfinite(want):
            assert L.b200emu_to_float(0, int(want.view(np.uint16))) == float(want)
