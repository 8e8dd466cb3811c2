"""Regenerates the message-size -> algorithm table of `coll/tuner.h` from device-timed sweeps.

    python -m gpu_ipc_example_b200.tune --np 8                   # runs bin/main on this node (two processes: LL and large)
    python -m gpu_ipc_example_b200.tune --from-json FILE --np 8  # re-reads rows written by `bin/main --json FILE`
    python -m gpu_ipc_example_b200.tune --from-files DIR --np 8  # re-reads saved text tables (sweep_w8_<algo>.txt)

The sweeps are `bin/main --np W -a <algo,algo,...> --sweep LO:HI` (rotating buffers larger than L2, 5
samples of 20 launches after 3 warm-ups, median, slowest rank).  The fastest algorithm per size is
picked and neighbouring sizes with the same winner are merged; with `--max-rows K` the table is
instead the best one with at most K rows (least total slow-down, in log time, against the per-size
winners).  The rows are printed in the syntax of `tune_table()`.
"""
from __future__ import annotations

import argparse
import json
import math
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

ROW = re.compile(r"^\s*(\d+)\s+(\d+)\s+(\d+)\s+(\d+)\s+([\d.]+)\s+([\d.]+)\s+([\d.]+)(?:\s+([\d.]+)\s+([\d.]+))?\s*$")


def parse_sweep(text: str) -> Dict[int, float]:
    """elements -> microseconds (max over ranks) from the table `bin/main --sweep` prints: the single time
    column of the seven-column form, or the median of the nine-column form (min, median, max)."""
    out = {}
    for line in text.splitlines():
        m = ROW.match(line)
        if m:
            out[int(m.group(1))] = float(m.group(6) if m.group(8) else m.group(5))
    return out


def parse_json_rows(text: str, world: int, collective: str = "all_reduce", placement: str = "in_place",
                    symmetric=None) -> Dict[str, Dict[int, float]]:
    """algo -> {elements: median microseconds} from the rows `bin/main --json` appends."""
    tables: Dict[str, Dict[int, float]] = {}
    for line in text.splitlines():
        line = line.strip()
        if not line.startswith("{"):
            continue
        r = json.loads(line)
        if r["world"] != world or r["collective"] != collective or r["placement"] != placement:
            continue
        if r["algo"] in ("auto", "allgather_auto", "reduce_scatter") or r.get("timing") == "graph_replay":
            continue
        if symmetric is not None and bool(r.get("symmetric")) != symmetric and r["algo"] in ("bulk", "nvls"):
            continue
        tables.setdefault(r["algo"], {})[int(r["elements"])] = float(r["us_median"])
    return tables


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


def best_table(tables: Dict[str, Dict[int, float]], max_rows: int, skip=("nccl",)) -> List[Tuple[int, str]]:
    """The table with at most `max_rows` rows that loses least against the per-size winners: sizes are cut
    into contiguous runs, one algorithm per run, minimising the sum of log(time / best time)."""
    tables = {a: t for a, t in tables.items() if a not in skip}
    sizes = sorted({s for t in tables.values() for s in t})
    best = {s: min(t[s] for t in tables.values() if s in t) for s in sizes}
    algos = sorted(tables)
    n = len(sizes)

    def cost(a, i, j):  # algorithm a on sizes[i:j]
        c = 0.0
        for s in sizes[i:j]:
            if s not in tables[a]:
                return math.inf
            c += math.log(tables[a][s] / best[s])
        return c

    # dp[k][j] = least cost of covering sizes[:j] with k runs
    dp = [[math.inf] * (n + 1) for _ in range(max_rows + 1)]
    arg = [[None] * (n + 1) for _ in range(max_rows + 1)]
    dp[0][0] = 0.0
    for k in range(1, max_rows + 1):
        for j in range(1, n + 1):
            for i in range(j):
                if dp[k - 1][i] == math.inf:
                    continue
                for a in algos:
                    c = dp[k - 1][i] + cost(a, i, j)
                    if c < dp[k][j]:
                        dp[k][j], arg[k][j] = c, (i, a)
    k = min(range(1, max_rows + 1), key=lambda q: dp[q][n])
    runs, j = [], n
    while j > 0:
        i, a = arg[k][j]
        runs.append((sizes[j - 1] * 2, a))
        j, k = i, k - 1
    runs.reverse()
    merged: List[Tuple[int, str]] = []
    for nbytes, a in runs:
        if merged and merged[-1][1] == a:
            merged[-1] = (nbytes, a)
        else:
            merged.append((nbytes, a))
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


def run_sweep(np_: int, algos: List[str], lo: int, hi: int, extra: List[str], json_path: str) -> None:
    exe = os.path.join(PKG, "bin", "main")
    cmd = [exe, "--np", str(np_), "-a", ",".join(algos), "--sweep", f"{lo}:{hi}", "--json", json_path] + extra
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1200)
    if p.returncode != 0:
        sys.stderr.write(f"{algos}: exit code {p.returncode}\n{p.stdout[-2000:]}\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--np", type=int, default=8)
    ap.add_argument("--from-files", default=None, help="directory with sweep_w<np>_<algo>.txt files")
    ap.add_argument("--from-json", default=None, help="file of rows written by `bin/main --json`")
    ap.add_argument("--symmetric", action="store_true", help="large-message kernels on buffers inside the symmetric heap")
    ap.add_argument("--max-rows", type=int, default=0, help="best table with at most this many rows (0: every winner)")
    ap.add_argument("--collective", default="all_reduce", choices=["all_reduce", "all_gather", "reduce_scatter"],
                    help="with --from-json: which collective's rows to read (all-gather and reduce-scatter print cut-offs "
                         "by algorithm name; their `auto` rules live in Comm::all_gather / Comm::reduce_scatter)")
    args = ap.parse_args()
    tables: Dict[str, Dict[int, float]] = {}
    if args.from_json and args.collective != "all_reduce":
        with open(args.from_json) as f:
            tables = parse_json_rows(f.read(), args.np, collective=args.collective, placement="out_of_place",
                                     symmetric=args.symmetric)
        nccl = {a: tables.pop(a) for a in [a for a in tables if a.startswith("nccl")]}
        rows = best_per_size(tables)
        print(f"# world {args.np}, {args.collective}: fastest algorithm per size (NCCL in brackets)")
        for elems, algo, us in rows:
            ref = [t[elems] for t in nccl.values() if elems in t]
            print(f"#   {elems * 2:>12} B  {algo:<32} {us:8.1f} us" + (f"   ({ref[0]:.1f})" if ref else ""))
        table = best_table(tables, args.max_rows, skip=()) if args.max_rows > 0 else merge_rows(rows)
        for nbytes, algo in table:
            print(f"up to {nbytes if nbytes else 'any size':>12} B: {algo}")
        return
    if args.from_json:
        with open(args.from_json) as f:
            tables = parse_json_rows(f.read(), args.np, symmetric=args.symmetric)
        tables.pop("nccl", None)
    elif args.from_files:
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
        import tempfile

        with tempfile.NamedTemporaryFile("r", suffix=".jsonl") as tmp:
            run_sweep(args.np, LL_ALGOS, 10, 23, [], tmp.name)
            run_sweep(args.np, BIG_ALGOS, 14, 28, ["--nvls"] + (["--symmetric"] if args.symmetric else []), tmp.name)
            tables = parse_json_rows(tmp.read(), args.np, symmetric=args.symmetric)
    rows = best_per_size(tables)
    print(f"# world {args.np}: fastest algorithm per size")
    for elems, algo, us in rows:
        print(f"#   {elems * 2:>12} B  {algo:<18} {us:8.1f} us")
    print(as_cpp(best_table(tables, args.max_rows) if args.max_rows > 0 else merge_rows(rows)))


if __name__ == "__main__":
    main()
