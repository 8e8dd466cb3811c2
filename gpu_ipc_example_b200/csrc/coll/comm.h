// The communicator: owns the symmetric heap(s), the sequence numbers and the
// status blocks, turns (algorithm, size) into a launch geometry and launches the
// kernels stream-ordered.
//
// A communicator drives either ONE rank of a multi-process world (one process
// per GPU; peers mapped through the heap) or ALL ranks of a "virtual world" on a
// single GPU (one cooperative launch whose block rows are the ranks) - the
// second form exists so that every protocol can be exercised on one GPU.
//
// Capability parity: launch geometry and sequence-number advance
// (allreduce.hpp:37-74, 238-269; allgather.hpp:31-70), the -a name table
// (allreduce.cpp:1121-1213), the host-side validation the reference lacks
// (a grid that is not a multiple of the world size loops forever there,
// allreduce.hpp:86-92).
#pragma once

#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include <cuda_runtime_api.h>

#include "../mem/symm_heap.h"
#include "kernel_table.h"

namespace b200ipc {

struct AlgoSpec {
  SchedKind sched = SchedKind::Parallel;
  ProtoKind proto = ProtoKind::LL8;
  bool direct_allgather = false;  // all-gather: push to every peer instead of the ring
  bool automatic = false;         // pick from the size table at call time
};

// Accepts the reference's names (small, simple, small_pcie_p, simple_pcie_p, bisect,
// small_ring, simple_ring, small_pcie, simple_pcie, allgather_small, allgather_simple),
// the additions (oneshot, bulk, nvls, auto, allgather_direct, allgather_bulk,
// allgather_nvls) and the generic form "<schedule>:<proto>", e.g. "sequential:ll8".
// Returns false for an unknown name.  *is_allgather tells which collective is meant.
bool parse_algo(const std::string& name, AlgoSpec* spec, bool* is_allgather);
std::string algo_names_help();
const char* sched_name(SchedKind s);

struct LaunchGeom {
  int ctas = 0;   // 0 = choose
  int warps = 0;  // warps per CTA, 0 = choose
};

struct CollInfo {
  SchedKind sched;
  ProtoKind proto;
  int ctas = 0;
  int warps = 0;
  int nwires = 0;
  int64_t steps = 0;
  uint32_t first_flag = 0;
  int launches = 0;
  bool staged = false;  // bulk/nvls: went through the staging buffer
};

struct CommOptions {
  HeapOptions heap;
  uint64_t timeout_ms = 2000;
  uint32_t first_seq = 1;
  bool device_seq = false;  // keep sequence numbers on the device (CUDA-graph capture)
  int max_ctas = 0;         // cap on CTAs per launch (0 = fill the GPU)
};

// Largest input (bytes) that `auto` gives to the flag-in-data reduce-scatter: a launch takes at most
// kParallelSlots steps, and 8 MiB fit in them at the default geometry with the 512-byte format (half of
// that with the 8-byte-granule fallback).  Measured on two B200s: ahead of the barrier-based kernel and of
// NCCL at every size up to there (8 MiB: 16.5 us against 26.1 and 29.3).
constexpr size_t kReduceScatterLLMaxBytes = size_t(8) << 20;

class Comm {
 public:
  static std::unique_ptr<Comm> create(UnixMesh& mesh, int device, const CommOptions& opt);
  static std::unique_ptr<Comm> create_virtual(int world, int device, const CommOptions& opt);
  ~Comm();
  Comm(const Comm&) = delete;
  Comm& operator=(const Comm&) = delete;

  int world() const { return world_; }
  int nlocal() const { return int(heaps_.size()); }
  int rank(int local = 0) const { return heaps_[size_t(local)]->rank(); }
  int device() const { return device_; }
  bool is_virtual() const { return mesh_ == nullptr && world_ > 1; }
  bool has_nvls() const { return heaps_[0]->multicast() != nullptr; }
  const SymmHeap& heap(int local = 0) const { return *heaps_[size_t(local)]; }
  UnixMesh* mesh() const { return mesh_; }
  int sm_count() const { return sm_count_; }

  // ins / outs hold nlocal() pointers (one per local rank).  nelems counts 16-bit
  // elements of one rank's buffer.  in == out means in place.
  CollInfo all_reduce(AlgoSpec algo, DType t, const void* const* ins, void* const* outs, size_t nelems,
                      LaunchGeom geom, cudaStream_t stream, uint32_t extra_flags = 0);
  // nelems = one rank's shard; every out holds world * nelems.  in == out + rank * nelems means in place.
  CollInfo all_gather(AlgoSpec algo, DType t, const void* const* ins, void* const* outs, size_t nelems,
                      LaunchGeom geom, cudaStream_t stream, uint32_t extra_flags = 0);
  // nelems = whole input (multiple of world); every out holds nelems / world.
  CollInfo reduce_scatter(AlgoSpec algo, DType t, const void* const* ins, void* const* outs, size_t nelems,
                          LaunchGeom geom, cudaStream_t stream, uint32_t extra_flags = 0);

  // Size -> algorithm choice used for AlgoSpec::automatic: the measured table of tuner.h unless
  // set_thresholds() installed explicit cut-offs (0, 0 restores the table).
  AlgoSpec choose_all_reduce(size_t bytes, bool symmetric) const;
  void set_thresholds(size_t oneshot_max_bytes, size_t ll_max_bytes) {
    oneshot_max_bytes_ = oneshot_max_bytes;
    ll_max_bytes_ = ll_max_bytes;
  }

  // Symmetric allocations from the staging region.  Every rank must make the same
  // calls in the same order; the returned offset is valid on every rank.
  size_t sym_alloc(size_t bytes, size_t align = 256);
  void sym_free_all() { sym_used_ = 0; }
  // Virtual world: the offset handed to local rank 0 is reused for the other local ranks.
  void set_last_sym_offset(size_t off) { last_sym_off_ = off; }
  size_t last_sym_offset() const { return last_sym_off_; }
  char* sym_ptr(size_t heap_offset, int local = 0) const { return heaps_[size_t(local)]->base() + heap_offset; }
  // Offset inside the heap if p points into this rank's staging region, else SIZE_MAX.
  size_t sym_offset_of(const void* p, int local = 0) const;

  StatusBlock status(int local = 0) const;
  // Throws b200ipc::Error describing the first recorded failure, if any.
  void raise_if_failed() const;
  // After a failure: waits for the device, clears rings, flags and status.  Collective
  // (host barrier) in a multi-process world.
  void reset();
  uint32_t seq() const { return seq_; }
  bool device_seq() const { return device_seq_; }
  void set_seq(uint32_t s) { seq_ = s; }
  uint64_t launches() const { return launches_; }
  // After a failed self-test of the 64-byte-segment wire formats (LL128 / LL512 rely on a warp's aligned
  // 64-byte store arriving whole): `auto` then only uses formats whose atomic unit is an 8-byte granule.
  void set_safe_protos(bool on) { safe_protos_ = on; }
  bool safe_protos() const { return safe_protos_; }
  bool trace_wires() const { return trace_wires_; }
  void set_trace_wires(bool on) { trace_wires_ = on; }
  void set_timeout_ms(uint64_t ms) { timeout_ns_ = ms * 1000000ull; }
  // Host barrier (no-op in a virtual world).
  void host_barrier();
  // Collective teardown of the multicast binding; call before destruction in a
  // multi-process world that enabled NVLS.
  void finalize();

  // Launch plumbing shared with the fused ops.
  void fill_views(KArgs* args, const void* const* ins, void* const* outs, size_t nelems, uint32_t flags) const;
  void launch(KernelFn fn, int ctas, int threads, KArgs* args, size_t smem, cudaStream_t stream, bool pdl = false);
  int resident_ctas(KernelFn fn, int threads, size_t smem);
  uint32_t take_seq(uint32_t advance);
  uint32_t take_barrier();
  // Launch with caller-built parameters (cooperative when this communicator drives several ranks).
  // pdl: the kernel executes griddepcontrol.wait before it touches anything an earlier kernel wrote, so it may be
  // launched with programmatic stream serialisation (single-rank launches only; see common/pdl.h)
  void launch_raw(const void* fn, int ctas, int threads, void** params, size_t smem, cudaStream_t stream, bool pdl = false);
  // Running total of the delivery counter of the fused GEMM kernels: returns the value the
  // counter reaches after `inc` more deliveries.
  uint32_t take_done(uint32_t inc) {
    gemm_done_ += inc;
    return gemm_done_;
  }
  // The same for the arrival counters of the all-gather + GEMM kernel; the second value is the
  // parity of the launch (which of the two gathered-input buffers it uses).
  uint32_t take_arrivals(uint32_t inc, int* parity) {
    ag_arrive_ += inc;
    *parity = int(ag_launches_++ & 1u);
    return ag_arrive_;
  }
  // Launch number of the fused GEMM kernels (flag value; its parity picks the half of the one-shot
  // landing zone).  Never reset: a stale flag must not equal a later launch's number.
  uint32_t take_gemm_epoch() {
    if (device_seq_) return gemm_epoch_ + 1;  // the device adds its own running offset
    ++gemm_epoch_;
    if (gemm_epoch_ == 0) gemm_epoch_ = 1;
    return gemm_epoch_;
  }
  void reset_fused_counters() {
    gemm_done_ = 0;
    ag_arrive_ = 0;
  }

 private:
  Comm() = default;
  void common_init(const CommOptions& opt);
  CollInfo launch_ll(LLOpId op, AlgoSpec algo, DType t, const void* const* ins, void* const* outs, size_t nelems,
                     LaunchGeom geom, cudaStream_t stream, uint32_t flags);
  CollInfo launch_bulk(BulkModeId mode, bool nvls, DType t, const void* const* ins, void* const* outs, size_t nelems,
                       LaunchGeom geom, cudaStream_t stream, uint32_t flags);

  int world_ = 1;
  int device_ = 0;
  int sm_count_ = 0;
  UnixMesh* mesh_ = nullptr;
  std::vector<std::unique_ptr<SymmHeap>> heaps_;
  std::vector<StatusBlock*> status_;  // pinned, one per local rank
  uint32_t seq_ = 1;
  uint32_t bar_seq_ = 0;
  uint32_t gemm_done_ = 0;
  uint32_t gemm_epoch_ = 0;
  uint32_t ag_arrive_ = 0;
  uint32_t ag_launches_ = 0;
  bool device_seq_ = false;
  bool safe_protos_ = false;
  bool trace_wires_ = false;  // B200IPC_DEBUG=1: kernels leave a record per completed wait in the trace ring
  uint64_t timeout_ns_ = 2000000000ull;
  int max_ctas_ = 0;
  size_t sym_used_ = 0;
  size_t last_sym_off_ = 0;
  size_t oneshot_max_bytes_ = 0;
  size_t ll_max_bytes_ = 0;
  uint64_t launches_ = 0;
  std::map<std::pair<const void*, int>, int> occupancy_cache_;
};

}  // namespace b200ipc
