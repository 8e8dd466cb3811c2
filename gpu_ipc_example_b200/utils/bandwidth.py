"""Bandwidth conventions and measured peaks used by the benchmarks and reports."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

NVLINK_PEER_COPY_GBS = 770.0   # measured peer copy per direction on this class of node (900 nominal)
NVLINK_NOMINAL_GBS = 900.0


def algbw_gbs(nbytes: int, seconds: float) -> float:
    """Algorithm bandwidth: bytes of one rank's buffer per second (all-gather: total output bytes)."""
    return nbytes / seconds / 1e9


def allreduce_busbw_gbs(nbytes: int, seconds: float, world: int) -> float:
    """NCCL-convention bus bandwidth of an all-reduce: algbw * 2 (n - 1) / n."""
    return algbw_gbs(nbytes, seconds) * 2 * (world - 1) / world


def allgather_busbw_gbs(total_out_bytes: int, seconds: float, world: int) -> float:
    """Bus bandwidth of an all-gather (and reduce-scatter): algbw * (n - 1) / n."""
    return algbw_gbs(total_out_bytes, seconds) * (world - 1) / world


def allreduce_link_bound_gbs(world: int, nvls: bool, link_gbs: float = NVLINK_PEER_COPY_GBS) -> float:
    """Upper bound on all-reduce busbw from the link alone: a two-phase exchange sends 2 (n-1)/n S per GPU,
    in-switch reduction (1 + 1/n) S."""
    return link_gbs * 2 * (world - 1) / (world + 1) if nvls else link_gbs


@dataclass
class Peaks:
    bf16_tflops: float
    bf16_tflops_sustained: float
    hbm_gbs: float
    source: str  # "measured" or "fallback"


def load_peaks(repo_root: str | None = None) -> Peaks:
    """The roofline denominators: the driver-measured file at the repository root if present, else the
    fallback figures of an earlier measurement on the same kind of node."""
    root = repo_root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return Peaks(float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), float(p["hbm_gbs"]), "measured")
    except (OSError, KeyError, ValueError):
        return Peaks(1590.0, 1400.0, 6650.0, "fallback")


def fused_layer_roofline_seconds(M: int, K: int, N: int, world: int, peaks: Peaks, link_gbs: float = NVLINK_NOMINAL_GBS) -> float:
    """Slower of the GEMM at the measured tensor peak and the all-reduce bytes over NVLink (by default at the
    nominal 900 GB/s per direction; pass NVLINK_PEER_COPY_GBS for the measured peer-copy rate)."""
    flops = 2.0 * M * K * N
    link_bytes = 2.0 * (world - 1) / world * M * N * 2 if world > 1 else 0.0
    return max(flops / (peaks.bf16_tflops * 1e12), link_bytes / (link_gbs * 1e9))
