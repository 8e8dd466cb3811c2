// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may be
// scheduled while its predecessor in the stream is still running, once every CTA of the predecessor
// has executed pdl_launch_dependents() (or exited).  Its CTAs become resident on SMs the predecessor
// has left, run whatever does not depend on the predecessor (barrier set-up, tensor-memory
// allocation, WEIGHT prefetch), and block in pdl_wait() until the predecessor has completed and its
// memory is visible.  A decode step is a chain of ~7 short kernels per layer; this takes launch
// latency and prologues off the critical path.
//
// Rules followed by every kernel that is launched this way:
//   * pdl_wait() comes before the first access to anything an earlier kernel may have written or
//     may still read (activations, flags, counters, scratch);
//   * kernels without pdl_wait() are never launched with the attribute;
//   * cooperative launches (several emulated ranks on one GPU) do not take the attribute: the two
//     instructions are then no-ops.
// B200IPC_PDL=0 in the environment turns the attribute off everywhere.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>

namespace b200ipc {

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("B200IPC_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

// cudaLaunchKernelExC with (or without) the programmatic-serialisation attribute.
inline cudaError_t launch_maybe_pdl(const void* fn, dim3 grid, dim3 block, void** params, size_t smem, cudaStream_t stream,
                                    bool pdl) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1u : 0u;
  return cudaLaunchKernelExC(&cfg, fn, params);
}

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

}  // namespace b200ipc
