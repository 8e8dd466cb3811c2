// Message size -> algorithm table for `auto`, from device-timed sweeps on an
// 8 x B200 NVSwitch node (2^10 .. 2^28 fp16 elements, worlds of 2, 4 and 8; every
// schedule x wire format; slowest rank).  Each row is "up to this many bytes use
// that schedule and wire format"; the last row of a table has no upper bound.
//
// What the sweeps showed: one NVLink hop (one-shot) wins while the (n-1) x payload
// it pushes stays small; the two-phase flag-in-data schedules win up to a few MiB
// because they read and write the caller's buffers directly and need no barrier;
// beyond that the barrier-based kernels win - in-switch reduction (NVLS) at eight
// ranks, peer-to-peer loads and stores at two and four, where NVLS moves no fewer
// bytes per GPU.  Buffers outside the symmetric heap pay a staging copy in the
// barrier-based kernels, which moves their break-even up.
#pragma once

#include <cstddef>

#include "../common/types.h"

namespace b200ipc {

struct TuneRow {
  size_t max_bytes;  // inclusive upper bound; 0 = no bound
  SchedKind sched;
  ProtoKind proto;
};

constexpr size_t KiB = 1024, MiB = 1024 * 1024;

// `large` is filled in by the caller: Nvls or Bulk depending on what the world supports.
inline const TuneRow* tune_table(int world, bool symmetric, int* rows) {
  // 8 ranks, three rows each (the dynamic programme of tune.py over the device-timed sweep of every schedule)
  static const TuneRow w8_sym[] = {
      {64 * KiB, SchedKind::OneShot, ProtoKind::LL16}, {1 * MiB, SchedKind::Parallel, ProtoKind::LL512}, {0, SchedKind::Nvls, ProtoKind::LL512}};
  static const TuneRow w8_user[] = {
      {64 * KiB, SchedKind::OneShot, ProtoKind::LL16}, {64 * MiB, SchedKind::Parallel, ProtoKind::LL512}, {0, SchedKind::Ring, ProtoKind::LL512}};
  // 4 ranks, from the 4-GPU sweep: the in-switch kernel (8 CTAs) is ahead of peer loads from 512 KiB up
  static const TuneRow w4_sym[] = {
      {128 * KiB, SchedKind::OneShot, ProtoKind::LL16}, {1 * MiB, SchedKind::Parallel, ProtoKind::LL512}, {0, SchedKind::Nvls, ProtoKind::LL512}};
  static const TuneRow w4_user[] = {
      {256 * KiB, SchedKind::OneShot, ProtoKind::LL16}, {4 * MiB, SchedKind::Sequential, ProtoKind::LL512}, {0, SchedKind::Parallel, ProtoKind::LL512}};
  // two ranks: one hop moves as many bytes as two, so the one-shot schedule reaches far
  static const TuneRow w2_sym[] = {
      {512 * KiB, SchedKind::OneShot, ProtoKind::LL512},   {2 * MiB, SchedKind::Sequential, ProtoKind::LL512},
      {0, SchedKind::Bulk, ProtoKind::LL512}};
  // caller's buffers: the flag-in-data kernels read and write them directly, the barrier-based ones
  // pay two staging copies; measured ahead of those (and of NCCL) up to 512 MiB
  static const TuneRow w2_user[] = {
      {4 * MiB, SchedKind::OneShot, ProtoKind::LL512},     {0, SchedKind::Ring, ProtoKind::LL512}};
  if (world >= 8) {
    *rows = 3;
    return symmetric ? w8_sym : w8_user;
  }
  if (world >= 4) {
    *rows = 3;
    return symmetric ? w4_sym : w4_user;
  }
  *rows = symmetric ? 3 : 2;
  return symmetric ? w2_sym : w2_user;
}

// CTAs of the in-switch (NVLS) all-reduce.  Measured on 8 GPUs with 4, 8, 12, 16, 24, 32 and 148 CTAs from 1 MiB
// to 512 MiB: 8 CTAs were the fastest at every size (16 MiB: 49.2 us against 59.0 with 32; 512 MiB: 1120 us
// against 1175 with 148) - the switch's reduction path is saturated by a few hundred loads in flight, and every
// further CTA adds its own pair of cross-rank barriers.  Same on 4 GPUs (8 against 16 CTAs, 2 - 256 MiB).  Only for
// buffers in the symmetric heap: with staging copies the CTAs also do the copies and many are wanted.
inline int nvls_ctas_for(size_t /*bytes*/) { return 8; }

}  // namespace b200ipc
