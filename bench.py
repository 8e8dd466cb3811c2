#!/usr/bin/env python
"""Headline benchmark: fp16 all-reduce bus bandwidth (and small-message latency) vs NCCL.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl nccl --gpus N ...                 # NCCL on the same box, same loop
    python bench.py --impl reference ...                     # the reference (not runnable here)

For N > 1 run it under `python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...`
(one rank per GPU); when started without a launcher's environment it re-launches itself that way.
With N = 1 there is no peer, so the world is emulated: 8 ranks on the one GPU, one cooperative
launch per all-reduce, "peer" traffic through L2/HBM instead of NVLink - the same kernels and
protocol, a different wire.  That is stated in `config.parallelism`.

A step is one all-reduce of the reference's default problem: 8 Mi fp16 elements (16 MiB) per rank
(`-n 8MB`, main.cpp:179, 45).  Rank 0 prints one JSON line; `value` is the NCCL-convention bus
bandwidth, busbw = bytes / time * 2 (n-1) / n, from device-side timing (CUDA events on the launching
stream, max over ranks).  Successive steps use different buffers whose total exceeds L2.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

METRIC = "fp16_allreduce_busbw_GBps"
DEFAULT_NELEMS = 8 * 1024 * 1024
L2_BYTES = 126 << 20


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "nccl", "reference"])
    p.add_argument("--nelems", type=int, default=DEFAULT_NELEMS)
    p.add_argument("--algo", default="auto")
    p.add_argument("--virtual-world", type=int, default=8, help="ranks emulated on one GPU when --gpus 1")
    p.add_argument("--no-sweep", action="store_true", help="skip the size sweep / NCCL comparison extras")
    p.add_argument("--no-nvls", action="store_true")
    return p.parse_args()


# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region is timed."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.proc.terminate()  # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm)}


def busbw(nbytes: int, seconds: float, world: int) -> float:
    return nbytes / seconds * 2 * (world - 1) / world / 1e9


# ---------------------------------------------------------------------------------------------
def relaunch_under_torchrun(args):
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
    return subprocess.call(cmd)


def main():
    args = parse_args()
    if args.impl == "reference":
        # The reference is SYCL + Level Zero + Intel vISA inline assembly built by icpx for Intel GPUs
        # (Makefile:1-42); it has no Python packaging, no CUDA path for sm_100 and needs MPI.
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is Intel-only SYCL/Level Zero/vISA code with no setup.py or pyproject.toml; "
                          "pip reports 'not installable' and no SYCL compiler or MPI exists on this image"}))
        return 0
    if args.gpus > 1 and "RANK" not in os.environ:
        return relaunch_under_torchrun(args)

    # Libraries (NCCL's version banner, for one) write to stdout; the contract is ONE JSON line
    # there.  Keep the real stdout for that line and point fd 1 at stderr for everything else.
    sys.stdout.flush()
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    state = {"comm": None, "stage": "start"}
    try:
        return run(args, json_out, state)
    except BaseException as e:  # noqa: BLE001 - a benchmark that dies must say where and why
        import traceback

        rank = int(os.environ.get("RANK", 0))
        status = None
        try:
            if state["comm"] is not None:
                status = state["comm"].status()
        except Exception:  # noqa: BLE001
            pass
        err = {"error": f"{type(e).__name__}: {e}"[:2000], "stage": state["stage"], "rank": rank, "status": status,
               "impl": args.impl, "n_gpus": args.gpus}
        sys.stderr.write(f"[bench rank {rank}] FAILED at stage '{state['stage']}': {err['error']}\nstatus: {status}\n")
        traceback.print_exc(file=sys.stderr)
        sys.stderr.flush()
        json_out.write(json.dumps(err) + "\n")
        json_out.flush()
        # the other ranks may be waiting on this one inside a collective: leave without the common teardown
        os._exit(1)


def run(args, json_out, state):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    multi = world > 1
    if multi:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    n = args.nelems
    nbytes = n * 2
    nbuf = max(2, (2 * L2_BYTES + nbytes - 1) // nbytes)  # rotate over > 2x L2 of buffers
    nbuf = min(nbuf, 32)
    steps, warmup = args.steps, max(3, args.warmup)

    from gpu_ipc_example_b200 import Communicator

    emu_world = args.virtual_world if not multi else world
    comm = None
    state["stage"] = "communicator"
    if args.impl == "ours":
        staging = nbuf * nbytes + (64 << 20) + (0 if args.no_sweep else (2 << 26) * 2 * 2 + (64 << 20))
        if multi:
            comm = Communicator.from_torch_distributed(local, staging_bytes=staging, nvls=not args.no_nvls)
        else:
            comm = Communicator.virtual(emu_world, local, staging_bytes=staging)
        state["comm"] = comm

    def make_bufs(symmetric):
        if symmetric:
            bufs = [comm.empty([n], torch.float16) for _ in range(nbuf)]  # symmetric: no staging copy
        else:
            bufs = [torch.empty(n, dtype=torch.float16, device="cuda") for _ in range(nbuf)]
        g = torch.Generator(device="cuda").manual_seed(rank)
        for b in bufs:
            for t in (b if isinstance(b, list) else [b]):
                t.copy_((torch.randn(n, device="cuda", generator=g) * 1e-3).half())
        return bufs

    state["stage"] = "buffers"
    bufs = make_bufs(args.impl == "ours")

    def step(i):
        b = bufs[i % nbuf]
        if args.impl == "ours":
            if multi:
                comm.all_reduce_(b, args.algo)
            else:
                comm.all_reduce(b, None, args.algo)
        else:
            if multi:
                dist.all_reduce(b)
            else:
                b.add_(0)  # a world of one: NCCL has nothing to do

    def sync_all():
        torch.cuda.synchronize()
        if multi:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, k):
        """k calls of fn between barriers; device time in seconds, max over ranks."""
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(k):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 1e3], device="cuda", dtype=torch.float64)
        if multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sync_all()
        if comm is not None:
            comm.check()
        return float(t.item())

    state["stage"] = "warm-up"
    for i in range(warmup):
        step(i)
    sync_all()
    if comm is not None:
        comm.check()

    state["stage"] = "timed region"
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = comm.launches if comm is not None else 0
    if sampler:
        sampler.start()
        time.sleep(0.25)
    seconds = timed(step, steps)
    # Keep the GPU busy a little longer so that the 100 ms sampler sees the loaded clocks.  Every step is
    # a collective, so every rank must issue the SAME number of extra steps: the count comes from
    # `seconds`, which is already the maximum over ranks and therefore identical everywhere.
    state["stage"] = "clock sampling tail"
    extra = int(min(20000, max(16, math.ceil(0.6 / max(seconds / steps, 1e-6)))))
    for i in range(extra):
        step(i)
        if i % 64 == 63:
            torch.cuda.synchronize()
    sync_all()
    clocks = sampler.stop() if sampler else None
    launches = (comm.launches - launches0 - extra) if comm is not None else 0
    if comm is not None:
        comm.check()
    ms_per_step = seconds / steps * 1e3
    if comm is not None:
        comm.all_reduce(bufs[0], None, args.algo)  # the reporting path, to learn which algorithm ran
    headline_algo = (comm.last_info.sched + ":" + comm.last_info.proto) if comm is not None else "nccl"
    value = busbw(nbytes, seconds / steps, emu_world)

    # ---- the comparison baseline for the same step: NCCL, same loop, same rotating-buffer discipline ----
    state["stage"] = "NCCL baseline of the headline step"
    nccl_headline = None
    if multi and args.impl == "ours":
        nb = [torch.empty(n, dtype=torch.float16, device="cuda").normal_(0, 1e-3) for _ in range(nbuf)]

        def nccl_head(i):
            dist.all_reduce(nb[i % nbuf])

        for i in range(warmup):
            nccl_head(i)
        s_n = timed(nccl_head, steps)
        nccl_headline = {"ms_per_step": round(s_n / steps * 1e3, 5), "busbw": round(busbw(nbytes, s_n / steps, world), 3)}
        del nb

    # ---- end to end through the public API: pinned host -> device, all-reduce, device -> host --------
    state["stage"] = "end-to-end"
    e2e = None
    if args.impl == "ours":
        host_in = [torch.empty(n, dtype=torch.float16).pin_memory() for _ in range(2)]
        for h in host_in:
            h.normal_(0, 1e-3)
        host_out = torch.empty(1024, dtype=torch.float16).pin_memory()

        # The upload of step i + 1 runs on its own stream while step i is reduced (the buffers rotate, so the two
        # never touch the same memory); every step still uploads its own input and reads its own result back.
        copy_stream = torch.cuda.Stream()
        uploaded = [torch.cuda.Event() for _ in range(nbuf)]
        consumed = [torch.cuda.Event() for _ in range(nbuf)]
        for ev in consumed:
            ev.record()

        def upload(i):
            b = bufs[i % nbuf]
            copy_stream.wait_event(consumed[i % nbuf])  # the all-reduce that last used this buffer is done
            with torch.cuda.stream(copy_stream):
                for t in (b if isinstance(b, list) else [b]):
                    t.copy_(host_in[i % 2], non_blocking=True)
                uploaded[i % nbuf].record(copy_stream)

        def e2e_step(i):
            b = bufs[i % nbuf]
            first = b[0] if isinstance(b, list) else b
            main = torch.cuda.current_stream()
            if i == 0:
                upload(0)
            upload(i + 1)  # one step ahead (the last call uploads one buffer that nothing consumes)
            main.wait_event(uploaded[i % nbuf])
            comm.all_reduce(b, None, args.algo)
            host_out.copy_(first[:1024], non_blocking=True)
            consumed[i % nbuf].record(main)

        for i in range(3):
            e2e_step(i)
        torch.cuda.synchronize()
        s2 = timed(e2e_step, steps)
        h2d = nbytes * (emu_world if not multi else 1)
        e2e = {"value": round(busbw(nbytes, s2 / steps, emu_world), 3), "unit": "GB/s", "ms_per_step": round(s2 / steps * 1e3, 5),
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 2048}

    # ---- extras: small-message latency and a few sizes, ours vs NCCL, outside the headline region ----
    # Both arms are replays of a CUDA graph holding `reps` back-to-back collectives, so that the host cost of
    # either library's Python entry point is out of the number; the figure is device time per collective,
    # median of three replays, max over ranks.
    sweep = None
    if not args.no_sweep and args.impl == "ours":
        state["stage"] = "size sweep"
        sweep = []

        def graph_time(fn, reps):
            """Median over three replays of a graph of `reps` calls of fn(i); seconds per call, max over ranks."""
            for i in range(3):
                fn(i)
            sync_all()
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for i in range(reps):
                        fn(i)
                runner = g.replay
            except Exception:  # noqa: BLE001 - capture not possible for this arm: time the plain loop
                g = None
                torch.cuda.synchronize()

                def runner():
                    for i in range(reps):
                        fn(i)
            runner()
            ts = [timed(lambda _i: runner(), 1) / reps for _ in range(3)]
            return statistics.median(ts), g is not None

        gcomm = None
        if multi:
            # sequence numbers kept on the device, so that a captured launch stays valid when replayed
            gcomm = Communicator.from_torch_distributed(local, staging_bytes=(2 << 26) * 2 + (64 << 20), nvls=not args.no_nvls,
                                                        device_seq=True)
        c = gcomm if gcomm is not None else comm
        pool = [c.empty([1 << 26], torch.float16) for _ in range(2)]  # slices of these are symmetric too

        def view(k, m):
            p, off = pool[k % 2], (k // 2) * m
            return [t[off:off + m] for t in p] if isinstance(p, list) else p[off:off + m]

        for e in (10, 12, 14, 16, 18, 20, 22, 23, 24, 26):
            m = 1 << e
            views = [view(k, m) for k in range(2 if e > 22 else 4)]
            reps = 100 if e <= 18 else (20 if e <= 22 else 8)

            def ours_step(i, views=views, c=c):
                if multi:
                    c.all_reduce_(views[i % len(views)], args.algo)
                else:
                    c.all_reduce(views[i % len(views)], None, args.algo)

            if multi:
                t_ours, graphed = graph_time(ours_step, reps)
            else:
                for i in range(5):
                    ours_step(i)
                t_ours, graphed = statistics.median([timed(ours_step, reps) / reps for _ in range(3)]), False
            c.all_reduce(views[0], None, args.algo)  # the reporting path, to learn which algorithm ran
            row = {"elements": m, "bytes": m * 2, "algo": c.last_info.sched + ":" + c.last_info.proto,
                   "ours_us": round(t_ours * 1e6, 3), "ours_busbw": round(busbw(m * 2, t_ours, emu_world), 3),
                   "timing": "cuda-graph replay" if graphed else "launch loop"}
            if multi:
                tv = [torch.zeros(m, dtype=torch.float16, device="cuda") for _ in range(len(views))]

                def nccl_step(i, tv=tv):
                    dist.all_reduce(tv[i % len(tv)])

                t_nccl, n_graphed = graph_time(nccl_step, reps)
                row["nccl_us"] = round(t_nccl * 1e6, 3)
                row["nccl_busbw"] = round(busbw(m * 2, t_nccl, world), 3)
                row["nccl_timing"] = "cuda-graph replay" if n_graphed else "launch loop"
                del tv
            sweep.append(row)
        if gcomm is not None:
            gcomm.check()
            gcomm.close()
        comm.check()

    state["stage"] = "report"
    if rank == 0:
        out = {
            "metric": METRIC,
            "value": round(value, 3),
            "unit": "GB/s",
            "n_gpus": args.gpus,
            "steps": steps,
            "warmup": warmup,
            "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True,
            "scaling": "weak",
            # the reference publishes no number; the comparison baseline is NCCL's all-reduce of the same step
            # on the same GPUs in the same run (none exists for a world of one GPU)
            "vs_baseline": round(value / nccl_headline["busbw"], 3) if nccl_headline else None,
            "dtype": "fp16",
            "data": "synthetic N(0,1e-3) seeded by rank",
            "impl": args.impl,
            "config": {
                "model": f"all-reduce of {n} fp16 elements ({nbytes >> 20} MiB) per rank, the reference's default -n 8MB problem",
                "global_batch": emu_world,
                "seq_len": n,
                "parallelism": (f"{world} GPUs, one rank per GPU over NVLink" if multi
                                else f"{emu_world} ranks emulated on 1 GPU (one cooperative launch; peer traffic stays in L2/HBM, no NVLink)"),
                "algo": f"{args.algo} -> {headline_algo}",
                "buffers": f"{nbuf} rotating buffers = {nbuf * nbytes >> 20} MiB > 126 MiB L2, in place, symmetric heap (no staging copy)",
                "busbw": "bytes/time*2(n-1)/n, device time by CUDA events, max over ranks",
                "baseline": ("NCCL all-reduce of the same step, same run: " + json.dumps(nccl_headline)) if nccl_headline else
                            "none at one GPU (NCCL has no peer)",
            },
            "clocks": clocks,
            "gpu_launches": launches,
        }
        if e2e:
            out["e2e"] = e2e
        if sweep:
            out["sweep"] = sweep
        if comm is not None and multi:
            out["config"]["nvls"] = comm.nvls_note
            out["config"]["backing"] = comm.backing
        json_out.write(json.dumps(out) + "\n")
        json_out.flush()
    state["stage"] = "teardown"
    if comm is not None:
        comm.close()
    if multi:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
