// Layout of a rank's symmetric heap (shared by the GPU heap and the CPU emulator).
#pragma once

#include "../coll/schedules.h"
#include "types.h"

namespace b200ipc {

inline size_t heap_round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Regions are 2 MiB aligned (the VMM mapping granularity).  The ring halves are
// sized for the largest image any schedule addresses: sequential / ring use
// world * slots * wires transactions of up to 512 B, bisect two regions of
// wires * 8.  The reference reserves world * 8 MiB per half (main.cpp:225).
inline HeapLayout make_heap_layout(size_t staging_bytes) {
  constexpr size_t kAlign = size_t(2) << 20;
  HeapLayout l{};
  size_t off = 0;
  l.ctrl_off = off;
  l.ctrl_bytes = kCtrlBytes;
  off += heap_round_up(l.ctrl_bytes, kAlign);
  l.half_bytes = size_t(kMaxRanks) * kSequentialSlots * kMaxWires * 512;
  for (int h = 0; h < 2; ++h) {
    l.half_off[h] = off;
    off += heap_round_up(l.half_bytes, kAlign);
  }
  l.oneshot_off = off;
  l.oneshot_bytes = size_t(kMaxRanks) * kMaxOneShotWires * kOneShotSlots * kOneShotStride;
  off += heap_round_up(l.oneshot_bytes, kAlign);
  l.staging_off = off;
  l.staging_bytes = heap_round_up(staging_bytes, kAlign);
  off += l.staging_bytes;
  l.total_bytes = off;
  return l;
}

}  // namespace b200ipc
