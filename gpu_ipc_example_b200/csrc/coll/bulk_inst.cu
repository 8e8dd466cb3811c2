// Instantiations of the large-message kernels: 2 element types x 3 world sizes x
// {P2P, NVLS} x {all-reduce, reduce-scatter, all-gather}.
#include "bulk_kernels.cuh"

namespace b200ipc {
namespace {
template <typename T, int N>
BulkKernelFn pick(bool nvls, BulkMode m) {
  auto cast = [](auto f) { return reinterpret_cast<BulkKernelFn>(f); };
  switch (m) {
    case BulkMode::AllReduce:
      return nvls ? cast(&bulk_kernel<T, N, true, BulkMode::AllReduce>) : cast(&bulk_kernel<T, N, false, BulkMode::AllReduce>);
    case BulkMode::ReduceScatter:
      return nvls ? cast(&bulk_kernel<T, N, true, BulkMode::ReduceScatter>)
                  : cast(&bulk_kernel<T, N, false, BulkMode::ReduceScatter>);
    default:
      return nvls ? cast(&bulk_kernel<T, N, true, BulkMode::AllGather>) : cast(&bulk_kernel<T, N, false, BulkMode::AllGather>);
  }
}
template <typename T>
BulkKernelFn pick_world(int world, bool nvls, BulkMode m) {
  switch (world) {
    case 2: return pick<T, 2>(nvls, m);
    case 4: return pick<T, 4>(nvls, m);
    case 8: return pick<T, 8>(nvls, m);
    default: return nullptr;
  }
}
}  // namespace

BulkKernelFn bulk_lookup(DType t, int world, bool nvls, BulkMode m) {
  return t == DType::F16 ? pick_world<__half>(world, nvls, m) : pick_world<__nv_bfloat16>(world, nvls, m);
}
}  // namespace b200ipc
