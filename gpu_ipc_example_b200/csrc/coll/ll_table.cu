// Maps (operation, element type, proto, world) to the kernel compiled in the
// ll_inst units.  Capability parity: the string -> template dispatch at
// allreduce.cpp:844-1213.
#include <type_traits>

#include "bulk_kernels.cuh"
#include "kernel_table.h"
#include "ll_kernels.cuh"

namespace b200ipc {

static_assert(int(LLOpId::ArParallel) == int(LLOp::ArParallel) && int(LLOpId::AgDirect) == int(LLOp::AgDirect) &&
                  int(LLOpId::RsParallel) == int(LLOp::RsParallel),
              "LLOpId must mirror LLOp");
static_assert(kBulkThreadsPerCta == kBulkThreads, "thread count mismatch");
static_assert(kBulkCopyInBit == kBulkCopyIn && kBulkCopyOutBit == kBulkCopyOut, "flag mismatch");

#define B200_DECLARE(OP)                                             \
  template <> LLKernelFn ll_lookup<LLOp::OP, __half>(ProtoKind, int); \
  template <> LLKernelFn ll_lookup<LLOp::OP, __nv_bfloat16>(ProtoKind, int);
B200_DECLARE(ArParallel)
B200_DECLARE(ArSequential)
B200_DECLARE(ArRing)
B200_DECLARE(ArBisect)
B200_DECLARE(ArOneShot)
B200_DECLARE(AgRing)
B200_DECLARE(AgDirect)
B200_DECLARE(RsParallel)
#undef B200_DECLARE

template <typename T>
static KernelFn by_op(LLOpId op, ProtoKind k, int world) {
  switch (op) {
    case LLOpId::ArParallel: return ll_lookup<LLOp::ArParallel, T>(k, world);
    case LLOpId::ArSequential: return ll_lookup<LLOp::ArSequential, T>(k, world);
    case LLOpId::ArRing: return ll_lookup<LLOp::ArRing, T>(k, world);
    case LLOpId::ArBisect: return ll_lookup<LLOp::ArBisect, T>(k, world);
    case LLOpId::ArOneShot: return ll_lookup<LLOp::ArOneShot, T>(k, world);
    case LLOpId::AgRing: return ll_lookup<LLOp::AgRing, T>(k, world);
    case LLOpId::RsParallel: return ll_lookup<LLOp::RsParallel, T>(k, world);
    default: return ll_lookup<LLOp::AgDirect, T>(k, world);
  }
}

KernelFn ll_kernel_lookup(LLOpId op, DType t, ProtoKind k, int world) {
  return t == DType::F16 ? by_op<__half>(op, k, world) : by_op<__nv_bfloat16>(op, k, world);
}

KernelFn bulk_kernel_lookup(BulkModeId m, DType t, int world, bool nvls) {
  return bulk_lookup(t, world, nvls, static_cast<BulkMode>(int(m)));
}

}  // namespace b200ipc
