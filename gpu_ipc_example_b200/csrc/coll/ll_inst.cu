// Explicit instantiation unit of the flag-in-data kernels.  Compiled once per
// (operation, element type) with -DB200_LL_OP=<LLOp enumerator> -DB200_LL_T=<type>
// so that the 7 x 2 units build in parallel; each holds 4 protos x 3 world sizes.
//
// Capability parity: the explicit instantiations for half and bfloat16, world
// 2/4/8, at allreduce.cpp:1215-1295.
#include <type_traits>

#include "ll_kernels.cuh"

#ifndef B200_LL_OP
#error "compile with -DB200_LL_OP=... -DB200_LL_T=..."
#endif

namespace b200ipc {
B200_DEFINE_LL_LOOKUP(LLOp::B200_LL_OP, B200_LL_T)
}  // namespace b200ipc
