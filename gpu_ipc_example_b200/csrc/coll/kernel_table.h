// Host-visible lookup of the compiled kernels (no device code in this header).
#pragma once

#include "../common/types.h"

namespace b200ipc {

// Mirrors LLOp in ll_kernels.cuh.
enum class LLOpId : int {
  ArParallel = 0,
  ArSequential = 1,
  ArRing = 2,
  ArBisect = 3,
  ArOneShot = 4,
  AgRing = 5,
  AgDirect = 6,
  RsParallel = 7,
};
enum class BulkModeId : int { AllReduce = 0, ReduceScatter = 1, AllGather = 2 };

using KernelFn = void (*)(const KArgs);

// nullptr when the combination is not compiled (world not in {2,4,8}).
KernelFn ll_kernel_lookup(LLOpId op, DType t, ProtoKind k, int world);
KernelFn bulk_kernel_lookup(BulkModeId m, DType t, int world, bool nvls);

constexpr int kBulkThreadsPerCta = 512;
// 16-byte vectors each thread keeps in flight per tile (host geometry and kernel agree on it).
// Peer-to-peer holds world copies of every vector in registers, the NVLS form only the result.
constexpr int bulk_unroll(int world, bool nvls) { return nvls ? 8 : (world >= 8 ? 2 : (world >= 4 ? 4 : 8)); }
// Bits of RankView::aux[1] for the bulk kernels.
constexpr uint64_t kBulkCopyInBit = 1;   // stage the caller's input into the symmetric buffer
constexpr uint64_t kBulkCopyOutBit = 2;  // copy the result from the symmetric buffer to the caller

}  // namespace b200ipc
