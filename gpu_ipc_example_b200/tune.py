"""Regenerates the message-size -> algorithm table of `coll/tuner.h` from device-timed sweeps.

    python -m gpu_ipc_example_b200.tune --np 8                 # runs bin/main once per algorithm on this node
    python -m gpu_ipc_example_b200.tune --from-files DIR --np 8  # re-reads saved sweep outputs (sweep_w8_<algo>.txt)

For every algorithm it runs `bin/main --np W -a <algo> --sweep LO:HI` (20 timed launches after 3
warm-ups, slowest rank), then picks the fastest algorithm per size, merges neighbouring sizes with the
same winner and prints the rows in the syntax of `tune_table()`.
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
from typing import Dict, List, Tuple

PKG = os.path.dirname(os.path.abspath(__file__))
LL_ALGOS = ["oneshot:ll512", "parallel:ll512", "bisect:ll512", "sequential:ll512", "ring:ll512", "oneshot", "small", "simple"]
BIG_ALGOS = ["bulk", "nvls"]
SCHED_ENUM = {"oneshot": "OneShot", "parallel": "Parallel", "bisect": "Bisect", "sequential": "Sequential", "ring": "Ring",
              "bulk": "Bulk", "nvls": "Nvls"}

# the reference's -a names (allreduce.cpp:1128-1185) as schedule:proto
ALIASES = {"small": "parallel:ll8", "simple": "parallel:ll128", "small_pcie_p": "parallel:ll16", "simple_pcie_p": "parallel:ll512",
           "small_pcie": "sequential:ll16", "simple_pcie": "sequential:ll512", "small_ring": "ring:ll16",
           "simple_ring": "ring:ll512", "bisect": "bisect:ll128", "oneshot": "oneshot:ll16", "bulk": "bulk:ll512", "nvls": "nvls:ll512"}

ROW = re.compile(r"^\s*(\d+)\s+(\d+)\s+(\d+)\s+(\d+)\s+([\d.]+)\s+([\d.]+)\s+([\d.]+)\s*$")


def parse_sweep(text: str) -> Dict[int, float]:
    """elements -> microseconds (max over ranks) from the table `bin/main --sweep` prints."""
    out = {}
    for line in text.splitlines():
        m = ROW.match(line)
        if m:
            out[int(m.group(1))] = float(m.group(5))
    return out


def best_per_size(tables: Dict[str, Dict[int, float]]) -> List[Tuple[int, str, float]]:
    sizes = sorted({s for t in tables.values() for s in t})
    rows = []
    for s in sizes:
        cand = [(t[s], a) for a, t in tables.items() if s in t]
        if cand:
            us, algo = min(cand)
            rows.append((s, algo, us))
    return rows


def merge_rows(rows: List[Tuple[int, str, float]]) -> List[Tuple[int, str]]:
    """[(max_bytes, algo)] with max_bytes = 0 for the open-ended last row."""
    merged: List[Tuple[int, str]] = []
    for elems, algo, _ in rows:
        nbytes = elems * 2
        if merged and merged[-1][1] == algo:
            merged[-1] = (nbytes, algo)
        else:
            merged.append((nbytes, algo))
    if merged:
        merged[-1] = (0, merged[-1][1])
    return merged


def as_cpp(merged: List[Tuple[int, str]]) -> str:
    lines = []
    for nbytes, algo in merged:
        sched, _, proto = ALIASES.get(algo, algo).partition(":")
        proto = (proto or "ll512").upper()
        bound = "0" if nbytes == 0 else (f"{nbytes // (1 << 20)} * MiB" if nbytes % (1 << 20) == 0 else f"{nbytes // 1024} * KiB")
        lines.append(f"      {{{bound}, SchedKind::{SCHED_ENUM[sched]}, ProtoKind::{proto}}},")
    return "\n".join(lines)


def run_sweep(np_: int, algo: str, lo: int, hi: int, extra: List[str]) -> str:
    exe = os.path.join(PKG, "bin", "main")
    cmd = [exe, "--np", str(np_), "-a", algo, "--sweep", f"{lo}:{hi}"] + extra
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    if p.returncode != 0:
        sys.stderr.write(f"{algo}: exit code {p.returncode}\n{p.stdout[-2000:]}\n")
    return p.stdout


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--np", type=int, default=8)
    ap.add_argument("--from-files", default=None, help="directory with sweep_w<np>_<algo>.txt files")
    ap.add_argument("--symmetric", action="store_true", help="large-message kernels on buffers inside the symmetric heap")
    args = ap.parse_args()
    tables: Dict[str, Dict[int, float]] = {}
    if args.from_files:
        prefix = f"sweep_w{args.np}_"
        for name in sorted(os.listdir(args.from_files)):
            if name.startswith(prefix) and name.endswith(".txt") and "_ag_" not in name and "nccl" not in name:
                algo = name[len(prefix):-4]
                suffix = "_sym" if args.symmetric else "_staged"
                if algo.endswith("_sym") or algo.endswith("_staged"):
                    if not algo.endswith(suffix):
                        continue
                    algo = algo[:-len(suffix)]
                with open(os.path.join(args.from_files, name)) as f:
                    t = parse_sweep(f.read())
                if t:
                    tables[algo] = t
    else:
        for algo in LL_ALGOS:
            tables[algo] = parse_sweep(run_sweep(args.np, algo, 10, 23, []))
        for algo in BIG_ALGOS:
            extra = ["--nvls"] + (["--symmetric"] if args.symmetric else [])
            tables[algo] = parse_sweep(run_sweep(args.np, algo, 14, 28, extra))
    rows = best_per_size(tables)
    print(f"# world {args.np}: fastest algorithm per size")
    for elems, algo, us in rows:
        print(f"#   {elems * 2:>12} B  {algo:<18} {us:8.1f} us")
    print(as_cpp(merge_rows(rows)))


if __name__ == "__main__":
    main()
