// See no_alloc.h for the contract.  The kernel is the large-message all-reduce of
// coll/bulk_kernels.cuh; what differs is where its scratch comes from: a file-scope
// device array instead of a communicator's heap.
#include "no_alloc.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include <cuda_runtime.h>

#include "../coll/bulk_kernels.cuh"

namespace {

using namespace b200ipc;

// Per emulated rank: [0, 8192) control words (abort word at 0, status record at 1024,
// barrier pads from kCtrlBarrierOff), then the staging area.  In host code this name is
// only a handle for cudaGetSymbolAddress, never an address to hand to a kernel.
static __device__ __align__(256) unsigned char g_noalloc_scratch[B200IPC_NOALLOC_SCRATCH_BYTES];

constexpr size_t kCtrlRegion = 8192;
constexpr size_t kStatusOff = 1024;
constexpr int kMaxCtas = (kCtrlRegion - kCtrlBarrierOff) / (kMaxRanks * sizeof(uint32_t));  // barrier pads that fit
constexpr int kMaxDevices = 64;

std::mutex g_mu;
unsigned char* g_base[kMaxDevices] = {nullptr};

template <typename T>
const void* kernel_for(int world) {
  switch (world) {
    case 2: return reinterpret_cast<const void*>(&bulk_kernel<T, 2, false, BulkMode::AllReduce>);
    case 4: return reinterpret_cast<const void*>(&bulk_kernel<T, 4, false, BulkMode::AllReduce>);
    case 8: return reinterpret_cast<const void*>(&bulk_kernel<T, 8, false, BulkMode::AllReduce>);
    default: return nullptr;
  }
}

}  // namespace

extern "C" int b200ipc_allreduce_noalloc(const void* const* ins, void* const* outs, int world, size_t nelems, int dtype,
                                         void* stream_v, uint32_t* status_host) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (!ins || !outs || (world != 2 && world != 4 && world != 8) || nelems == 0 || (dtype != 0 && dtype != 1)) {
    std::fprintf(stderr, "b200ipc_allreduce_noalloc: bad argument (world must be 2, 4 or 8; dtype 0 or 1; nelems > 0)\n");
    return 1;
  }
  if (nelems > size_t(B200IPC_NOALLOC_MAX_ELEMS)) {
    std::fprintf(stderr,
                 "b200ipc_allreduce_noalloc: %zu elements per rank exceed the fixed scratch (maximum %d); use a "
                 "communicator for larger messages\n",
                 nelems, B200IPC_NOALLOC_MAX_ELEMS);
    return 2;
  }
  for (int r = 0; r < world; ++r)
    if (!ins[r] || !outs[r]) return 1;

  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return 100 + int(e);
  if (device < 0 || device >= kMaxDevices) return 1;

  // One-time set-up per device, with that device current: the device address of the array.
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_base[device] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess) {
        std::fprintf(stderr, "b200ipc_allreduce_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
        return 100 + int(e);
      }
      g_base[device] = static_cast<unsigned char*>(p);
    }
    base = g_base[device];
  }

  const void* fn = dtype == 0 ? kernel_for<__half>(world) : kernel_for<__nv_bfloat16>(world);

  // Two knobs read from the environment, for tests of the failure report: the time limit of a
  // device-side wait (B200IPC_TIMEOUT_US, as everywhere in the library) and a rank that sends
  // nothing (B200IPC_NOALLOC_MUTE_RANK), which makes the others' bounded waits run out.
  uint64_t timeout_ns = 2000000000ull;
  if (const char* t = std::getenv("B200IPC_TIMEOUT_US")) {
    const long long us = std::atoll(t);
    if (us > 0) timeout_ns = uint64_t(us) * 1000ull;
  }
  int mute_rank = -1;
  if (const char* m = std::getenv("B200IPC_NOALLOC_MUTE_RANK")) mute_rank = std::atoi(m);

  // Geometry: as many CTAs per rank as the barrier pads, the work and co-residency allow.
  int per_sm = 0, sms = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kBulkThreads, 0);
  if (e != cudaSuccess) return 100 + int(e);
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) return 100 + int(e);
  const long long shard_vec = ((long long)((nelems + 7) / 8) + world - 1) / world;
  long long slabs = (shard_vec + kBulkThreads - 1) / kBulkThreads;
  if (slabs < 1) slabs = 1;
  long long ctas = (long long)per_sm * sms / world;
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (ctas > slabs) ctas = slabs;
  if (ctas < 1) return 1;

  // Words that must start at zero: abort word, status record, barrier pads of every rank.
  e = cudaMemset2DAsync(base, B200IPC_NOALLOC_RANK_STRIDE, 0, kCtrlRegion, size_t(world), stream);
  if (e != cudaSuccess) return 100 + int(e);

  KArgs args;
  std::memset(&args, 0, sizeof(args));
  args.lay.ctrl_off = 0;
  args.lay.ctrl_bytes = kCtrlRegion;
  args.lay.staging_off = kCtrlRegion;
  args.lay.staging_bytes = B200IPC_NOALLOC_RANK_STRIDE - kCtrlRegion;
  args.lay.total_bytes = B200IPC_NOALLOC_RANK_STRIDE;
  for (int r = 0; r < world; ++r) {
    RankView& v = args.v[r];
    v.rank = r;
    v.world = world;
    v.heap = reinterpret_cast<char*>(base + size_t(r) * B200IPC_NOALLOC_RANK_STRIDE);
    for (int q = 0; q < kMaxRanks; ++q)
      v.peer[q] = reinterpret_cast<char*>(base + size_t(q < world ? q : r) * B200IPC_NOALLOC_RANK_STRIDE);
    v.in = ins[r];
    v.out = outs[r];
    v.nelems = nelems;
    // ONE record for the whole emulated world (the one in rank 0's region): whichever rank's wait
    // runs out first writes it, and that is the record copied back to the caller below.
    v.status = reinterpret_cast<StatusBlock*>(base + kStatusOff);
    v.timeout_ns = timeout_ns;
    if (r == mute_rank) v.flags |= kMuteSends;
    v.bar_seq = 0;
    v.aux[0] = kCtrlRegion;                  // staging area inside each rank's region
    v.aux[1] = kBulkCopyIn | kBulkCopyOut;   // the caller's buffers are ordinary memory
  }
  void* params[] = {&args};
  e = cudaLaunchCooperativeKernel(fn, dim3(unsigned(ctas), unsigned(world), 1), dim3(kBulkThreads, 1, 1), params, 0, stream);
  if (e != cudaSuccess) {
    std::fprintf(stderr, "b200ipc_allreduce_noalloc: launch failed: %s\n", cudaGetErrorString(e));
    return 100 + int(e);
  }
  if (status_host) {
    e = cudaMemcpyAsync(status_host, base + kStatusOff, 8 * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return 100 + int(e);
  }
  return 0;
}
