from .bandwidth import (NVLINK_NOMINAL_GBS, NVLINK_PEER_COPY_GBS, Peaks, algbw_gbs, allgather_busbw_gbs, allreduce_busbw_gbs, allreduce_link_bound_gbs,
                        fused_layer_roofline_seconds, load_peaks)

__all__ = ["NVLINK_NOMINAL_GBS", "NVLINK_PEER_COPY_GBS", "Peaks", "algbw_gbs", "allgather_busbw_gbs", "allreduce_busbw_gbs", "allreduce_link_bound_gbs",
           "fused_layer_roofline_seconds", "load_peaks"]
