// Kernel entry points of the flag-in-data collectives.  One template kernel per
// schedule; the proto, element type and world size are template parameters, the
// rank comes from the launch arguments.  gridDim.y > 1 is the single-GPU
// emulation of a whole world: block row y runs rank y (a cooperative launch
// keeps all rows resident, which the cross-rank waits need).
//
// Capability parity: AllReduce / bisectPAllReduce / AllGather functors
// (allreduce.hpp:8-125, 212-317; allgather.hpp:8-120).
#pragma once

#include "../proto/dev_backend.cuh"
#include "schedules.h"

namespace b200ipc {

template <class B>
__device__ __forceinline__ Ctx<B> make_ctx(const KArgs& args, int nwires, int wire) {
  const RankView& me = args.v[blockIdx.y];
  Ctx<B> c;
  c.me = &me;
  c.lay = &args.lay;
  c.rank = me.rank;
  c.world = me.world;
  c.nwires = nwires;
  c.seq = me.seq;
  c.flags = me.flags;
  c.in = static_cast<const uint32_t*>(me.in);
  c.out = static_cast<uint32_t*>(me.out);
  c.nelems = me.nelems;
  c.waiter.me = &me;
  c.waiter.ctrl_off = args.lay.ctrl_off;
  c.waiter.wire = wire;
  return c;
}

enum class LLOp : int {
  ArParallel,
  ArSequential,
  ArRing,
  ArBisect,
  ArOneShot,
  AgRing,
  AgDirect,
  RsParallel,
};

template <LLOp OP, ProtoKind K, typename T, int N>
__global__ void __launch_bounds__(1024) ll_kernel(const __grid_constant__ KArgs args) {
  using B = DevBackend<K, T>;
  const int warps = int(blockDim.x >> 5);
  const int wire = int(blockIdx.x) * warps + int(threadIdx.x >> 5);
  const int nwires = int(gridDim.x) * warps;
  Ctx<B> c = make_ctx<B>(args, nwires, wire);
  const RankView& me = args.v[blockIdx.y];
  // Graph-captured launches keep the running sequence number on the device: the
  // value baked into the launch is a constant base, the offset lives in memory.
  if (me.seq_dev) c.seq += ld_volatile_u32(me.seq_dev);
  if constexpr (OP == LLOp::ArParallel) run_parallel<B, N>(c, wire);
  else if constexpr (OP == LLOp::ArSequential) run_sequential<B, N>(c, wire);
  else if constexpr (OP == LLOp::ArRing) run_ring_allreduce<B, N>(c, wire);
  else if constexpr (OP == LLOp::ArBisect) run_bisect<B, N>(c, wire);
  else if constexpr (OP == LLOp::ArOneShot) run_oneshot<B, N>(c, wire);
  else if constexpr (OP == LLOp::AgRing) run_ring_allgather<B, N>(c, wire);
  else if constexpr (OP == LLOp::RsParallel) run_reduce_scatter<B, N>(c, wire);
  else run_direct_allgather<B, N>(c, wire);
  if (me.seq_dev) {
    // The last CTA to finish advances the offset; every CTA has read it by then.
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(me.seq_dev + 1, 1u) == gridDim.x - 1) {
        me.seq_dev[1] = 0;
        me.seq_dev[0] += me.seq_step;
        __threadfence();
      }
    }
  }
}

// Type-erased handle the host-side dispatcher works with.
using LLKernelFn = void (*)(const KArgs);

template <LLOp OP, ProtoKind K, typename T, int N>
inline LLKernelFn ll_kernel_ptr() {
  return reinterpret_cast<LLKernelFn>(&ll_kernel<OP, K, T, N>);
}

// Defined once per (op, element type) in coll/ll_inst_*.cu so that the 7 x 4 x 2 x 3
// instantiations compile in parallel.
template <LLOp OP, typename T>
LLKernelFn ll_lookup(ProtoKind k, int world);

#define B200_DEFINE_LL_LOOKUP(OP, T)                                                   \
  template <>                                                                          \
  LLKernelFn ll_lookup<OP, T>(ProtoKind k, int world) {                                \
    auto by_world = [&](auto kc) -> LLKernelFn {                                       \
      constexpr ProtoKind KK = decltype(kc)::value;                                    \
      switch (world) {                                                                 \
        case 2: return ll_kernel_ptr<OP, KK, T, 2>();                                  \
        case 4: return ll_kernel_ptr<OP, KK, T, 4>();                                  \
        case 8: return ll_kernel_ptr<OP, KK, T, 8>();                                  \
        default: return nullptr;                                                       \
      }                                                                                \
    };                                                                                 \
    switch (k) {                                                                       \
      case ProtoKind::LL8: return by_world(std::integral_constant<ProtoKind, ProtoKind::LL8>{});     \
      case ProtoKind::LL16: return by_world(std::integral_constant<ProtoKind, ProtoKind::LL16>{});   \
      case ProtoKind::LL128: return by_world(std::integral_constant<ProtoKind, ProtoKind::LL128>{}); \
      default: return by_world(std::integral_constant<ProtoKind, ProtoKind::LL512>{});               \
    }                                                                                  \
  }

}  // namespace b200ipc
