from .bandwidth import (Peaks, algbw_gbs, allgather_busbw_gbs, allreduce_busbw_gbs, allreduce_link_bound_gbs,
                        fused_layer_roofline_seconds, load_peaks)

__all__ = ["Peaks", "algbw_gbs", "allgather_busbw_gbs", "allreduce_busbw_gbs", "allreduce_link_bound_gbs",
           "fused_layer_roofline_seconds", "load_peaks"]
