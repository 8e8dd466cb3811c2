#include "fused_ops.h"

#include <algorithm>
#include <cstring>

#include "../common/check.h"
#include "oneshot_fused.cuh"

namespace b200ipc {
namespace {

template <typename T, typename Tout, int EPI>
KernelFn pick_world(int world) {
  auto cast = [](auto f) { return reinterpret_cast<KernelFn>(f); };
  switch (world) {
    case 1: return cast(&oneshot_fused_kernel<T, Tout, 1, EPI>);
    case 2: return cast(&oneshot_fused_kernel<T, Tout, 2, EPI>);
    case 4: return cast(&oneshot_fused_kernel<T, Tout, 4, EPI>);
    case 8: return cast(&oneshot_fused_kernel<T, Tout, 8, EPI>);
    default: return nullptr;
  }
}

uint32_t float_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}

}  // namespace

CollInfo fused_allreduce_residual_rmsnorm(Comm& comm, DType t, const FusedNormPtrs* ptrs, int64_t rows, int64_t hidden,
                                          float eps, int ctas_req, cudaStream_t stream) {
  B200_REQUIRE(rows > 0 && hidden > 0 && hidden % 8 == 0, "hidden must be a positive multiple of 8");
  const int N = comm.world();
  KernelFn fn = t == DType::F16 ? pick_world<__half, __half, kEpiNorm>(N) : pick_world<__nv_bfloat16, __nv_bfloat16, kEpiNorm>(N);
  B200_REQUIRE(fn != nullptr, "no fused kernel for world size " << N);
  B200_CUDA_CHECK(cudaSetDevice(comm.device()));

  // Geometry: a CTA owns whole rows; its warps share the row's transactions.
  const int64_t row_dw = hidden / 2;
  const int64_t row_tx = ceil_div64(row_dw, 120);
  const int64_t want_warps = kFusedMaxThreads / 32;
  int warps = int(std::max<int64_t>(4, round_up64(std::min<int64_t>(row_tx, want_warps), 4)));
  int threads = warps * 32;
  int cap = std::min(comm.resident_ctas(fn, threads, 0), kMaxOneShotWires / warps);
  B200_REQUIRE(cap >= 1, "fused kernel does not fit");
  int ctas = ctas_req > 0 ? ctas_req : int(std::min<int64_t>(rows, cap));
  B200_REQUIRE(ctas <= cap, "requested " << ctas << " CTAs, only " << cap << " can run at once");
  const int64_t rows_per_cta = ceil_div64(rows, ctas);
  B200_REQUIRE(rows_per_cta <= kFusedMaxRowsPerCta,
               "too many rows (" << rows << ") for the one-shot fused kernel: at most " << int64_t(cap) * kFusedMaxRowsPerCta);
  const int64_t steps = ceil_div64(ceil_div64(rows_per_cta * row_dw, 120), warps);

  std::vector<const void*> ins(size_t(comm.nlocal()));
  std::vector<void*> outs(size_t(comm.nlocal()));
  for (int i = 0; i < comm.nlocal(); ++i) {
    ins[size_t(i)] = ptrs[i].x;
    outs[size_t(i)] = ptrs[i].out;
    for (const void* p : {ptrs[i].x, ptrs[i].residual, ptrs[i].gamma, static_cast<const void*>(ptrs[i].out),
                          static_cast<const void*>(ptrs[i].residual_out)})
      B200_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, "fused all-reduce + RMSNorm needs 16-byte aligned tensors");
  }
  KArgs args;
  comm.fill_views(&args, ins.data(), outs.data(), size_t(rows * hidden), 0);
  const uint32_t adv = uint32_t(steps + 1);
  const uint32_t first = comm.take_seq(adv);
  for (int i = 0; i < comm.nlocal(); ++i) {
    args.v[i].seq = first;
    args.v[i].seq_step = adv;
    args.v[i].aux[0] = reinterpret_cast<uint64_t>(ptrs[i].residual);
    args.v[i].aux[1] = reinterpret_cast<uint64_t>(ptrs[i].gamma);
    args.v[i].aux[2] = reinterpret_cast<uint64_t>(ptrs[i].residual_out);
    args.v[i].aux[3] = uint64_t(uint32_t(hidden)) | (uint64_t(float_bits(eps)) << 32);
  }
  comm.launch(fn, ctas, threads, &args, 0, stream, true);
  CollInfo info;
  info.sched = SchedKind::OneShot;
  info.proto = ProtoKind::LL512;
  info.ctas = ctas;
  info.warps = warps;
  info.nwires = ctas * warps;
  info.steps = steps;
  info.first_flag = first;
  info.launches = 1;
  return info;
}

CollInfo fused_allreduce_scale_cast(Comm& comm, DType tin, DType tout, const void* const* ins, void* const* outs,
                                    size_t nelems, float scale, int ctas_req, cudaStream_t stream) {
  B200_REQUIRE(nelems > 0 && nelems % 2 == 0, "element count must be even");
  const int N = comm.world();
  KernelFn fn;
  if (tin == DType::F16)
    fn = tout == DType::F16 ? pick_world<__half, __half, kEpiScale>(N) : pick_world<__half, __nv_bfloat16, kEpiScale>(N);
  else
    fn = tout == DType::F16 ? pick_world<__nv_bfloat16, __half, kEpiScale>(N)
                            : pick_world<__nv_bfloat16, __nv_bfloat16, kEpiScale>(N);
  B200_REQUIRE(fn != nullptr, "no fused kernel for world size " << N);
  B200_CUDA_CHECK(cudaSetDevice(comm.device()));
  const int64_t total_dw = int64_t(nelems / 2);
  const int64_t ntx = ceil_div64(total_dw, 120);
  int warps = int(std::min<int64_t>(16, std::max<int64_t>(1, ntx)));
  int threads = warps * 32;
  int cap = std::min(comm.resident_ctas(fn, threads, 0), kMaxOneShotWires / warps);
  B200_REQUIRE(cap >= 1, "fused kernel does not fit");
  int ctas = ctas_req > 0 ? ctas_req : int(std::min<int64_t>(cap, ceil_div64(ntx, warps)));
  B200_REQUIRE(ctas <= cap, "requested " << ctas << " CTAs, only " << cap << " can run at once");
  const int64_t per = round_up64(ceil_div64(total_dw, ctas), 4);
  const int64_t steps = ceil_div64(ceil_div64(per, 120), warps);

  KArgs args;
  comm.fill_views(&args, ins, outs, nelems, 0);
  const uint32_t adv = uint32_t(steps + 1);
  const uint32_t first = comm.take_seq(adv);
  for (int i = 0; i < comm.nlocal(); ++i) {
    args.v[i].seq = first;
    args.v[i].seq_step = adv;
    args.v[i].aux[3] = uint64_t(float_bits(scale)) << 32;
    B200_REQUIRE((reinterpret_cast<uintptr_t>(ins[i]) & 3) == 0 && (reinterpret_cast<uintptr_t>(outs[i]) & 3) == 0,
                 "buffers must be 4-byte aligned");
  }
  comm.launch(fn, ctas, threads, &args, 0, stream, true);
  CollInfo info;
  info.sched = SchedKind::OneShot;
  info.proto = ProtoKind::LL512;
  info.ctas = ctas;
  info.warps = warps;
  info.nwires = ctas * warps;
  info.steps = steps;
  info.first_flag = first;
  info.launches = 1;
  return info;
}

}  // namespace b200ipc
