#include "comm.h"

#include "../common/pdl.h"

#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <sstream>

#include <nvtx3/nvToolsExt.h>

#include "../common/check.h"
#include "../proto/wire_format.h"
#include "schedules.h"
#include "tuner.h"

namespace b200ipc {

// ----------------------------------------------------------------------------
// Algorithm names
// ----------------------------------------------------------------------------
const char* sched_name(SchedKind s) {
  switch (s) {
    case SchedKind::Parallel: return "parallel";
    case SchedKind::Sequential: return "sequential";
    case SchedKind::Ring: return "ring";
    case SchedKind::Bisect: return "bisect";
    case SchedKind::OneShot: return "oneshot";
    case SchedKind::Bulk: return "bulk";
    default: return "nvls";
  }
}

namespace {

// NVTX range around the host side of a collective (what a timeline tool shows next to the kernel);
// costs a null check when no tool is attached.
struct NvtxRange {
  explicit NvtxRange(const char* what, const AlgoSpec& a, size_t bytes) {
    char buf[96];
    std::snprintf(buf, sizeof(buf), "b200ipc::%s[%s:%s] %zu B", what, a.automatic ? "auto" : sched_name(a.sched), proto_name(a.proto), bytes);
    nvtxRangePushA(buf);
  }
  ~NvtxRange() { nvtxRangePop(); }
};

struct NamedAlgo {
  const char* name;
  SchedKind sched;
  ProtoKind proto;
  bool allgather;
  bool direct;
};

// The first eleven rows are the reference's -a values (allreduce.cpp:1128-1212).
const NamedAlgo kNamed[] = {
    {"small", SchedKind::Parallel, ProtoKind::LL8, false, false},
    {"simple", SchedKind::Parallel, ProtoKind::LL128, false, false},
    {"small_pcie_p", SchedKind::Parallel, ProtoKind::LL16, false, false},
    {"simple_pcie_p", SchedKind::Parallel, ProtoKind::LL512, false, false},
    {"bisect", SchedKind::Bisect, ProtoKind::LL128, false, false},
    {"small_ring", SchedKind::Ring, ProtoKind::LL16, false, false},
    {"simple_ring", SchedKind::Ring, ProtoKind::LL512, false, false},
    {"small_pcie", SchedKind::Sequential, ProtoKind::LL16, false, false},
    {"simple_pcie", SchedKind::Sequential, ProtoKind::LL512, false, false},
    {"allgather_small", SchedKind::Ring, ProtoKind::LL16, true, false},
    {"allgather_simple", SchedKind::Ring, ProtoKind::LL512, true, false},
    // additions
    {"oneshot", SchedKind::OneShot, ProtoKind::LL16, false, false},
    {"bulk", SchedKind::Bulk, ProtoKind::LL512, false, false},
    {"nvls", SchedKind::Nvls, ProtoKind::LL512, false, false},
    {"allgather_direct", SchedKind::Ring, ProtoKind::LL512, true, true},
    {"allgather_bulk", SchedKind::Bulk, ProtoKind::LL512, true, false},
    {"allgather_nvls", SchedKind::Nvls, ProtoKind::LL512, true, false},
};

std::string lower(std::string s) {
  for (char& c : s) c = char(std::tolower(static_cast<unsigned char>(c)));
  return s;
}

bool parse_proto(const std::string& s, ProtoKind* k) {
  if (s == "ll8") *k = ProtoKind::LL8;
  else if (s == "ll16") *k = ProtoKind::LL16;
  else if (s == "ll128") *k = ProtoKind::LL128;
  else if (s == "ll512") *k = ProtoKind::LL512;
  else return false;
  return true;
}

}  // namespace

bool parse_algo(const std::string& name_in, AlgoSpec* spec, bool* is_allgather) {
  const std::string name = lower(name_in);
  *is_allgather = false;
  *spec = AlgoSpec{};
  if (name == "auto") {
    spec->automatic = true;
    return true;
  }
  if (name == "allgather_auto" || name == "allgather") {
    spec->automatic = true;
    *is_allgather = true;
    return true;
  }
  for (const NamedAlgo& n : kNamed) {
    if (name == n.name) {
      spec->sched = n.sched;
      spec->proto = n.proto;
      spec->direct_allgather = n.direct;
      *is_allgather = n.allgather;
      return true;
    }
  }
  // "<schedule>:<proto>"
  size_t colon = name.find(':');
  if (colon == std::string::npos) return false;
  std::string s = name.substr(0, colon);
  std::string p = name.substr(colon + 1);
  if (!parse_proto(p, &spec->proto)) return false;
  if (s == "parallel") spec->sched = SchedKind::Parallel;
  else if (s == "sequential") spec->sched = SchedKind::Sequential;
  else if (s == "ring") spec->sched = SchedKind::Ring;
  else if (s == "bisect") spec->sched = SchedKind::Bisect;
  else if (s == "oneshot") spec->sched = SchedKind::OneShot;
  else if (s == "allgather_ring") { spec->sched = SchedKind::Ring; *is_allgather = true; }
  else if (s == "allgather_direct") { spec->sched = SchedKind::Ring; spec->direct_allgather = true; *is_allgather = true; }
  else return false;
  return true;
}

std::string algo_names_help() {
  std::ostringstream os;
  for (const NamedAlgo& n : kNamed) os << n.name << " ";
  os << "auto allgather_auto <parallel|sequential|ring|bisect|oneshot|allgather_ring|allgather_direct>:<ll8|ll16|ll128|ll512>";
  return os.str();
}

// ----------------------------------------------------------------------------
// Construction
// ----------------------------------------------------------------------------
void Comm::common_init(const CommOptions& opt) {
  seq_ = opt.first_seq == 0 ? 1 : opt.first_seq;
  device_seq_ = opt.device_seq;
  timeout_ns_ = opt.timeout_ms * 1000000ull;
  max_ctas_ = opt.max_ctas;
  B200_CUDA_CHECK(cudaSetDevice(device_));
  B200_CUDA_CHECK(cudaDeviceGetAttribute(&sm_count_, cudaDevAttrMultiProcessorCount, device_));
  status_.assign(heaps_.size(), nullptr);
  for (size_t i = 0; i < heaps_.size(); ++i) {
    void* p = nullptr;
    B200_CUDA_CHECK(cudaHostAlloc(&p, sizeof(StatusBlock), cudaHostAllocMapped | cudaHostAllocPortable));
    std::memset(p, 0, sizeof(StatusBlock));
    status_[i] = static_cast<StatusBlock*>(p);
  }
  if (const char* e = std::getenv("B200IPC_DEBUG")) trace_wires_ = std::atoi(e) != 0;
  if (const char* e = std::getenv("B200IPC_TIMEOUT_US")) {
    long long us = std::atoll(e);
    if (us > 0) timeout_ns_ = uint64_t(us) * 1000ull;
  }
}

std::unique_ptr<Comm> Comm::create(UnixMesh& mesh, int device, const CommOptions& opt) {
  std::unique_ptr<Comm> c(new Comm());
  c->world_ = mesh.world();
  c->device_ = device;
  c->mesh_ = &mesh;
  if (mesh.world() == 1) {
    HeapOptions ho = opt.heap;
    c->heaps_ = SymmHeap::make_virtual(1, device, ho);
    c->mesh_ = nullptr;
  } else {
    c->heaps_.push_back(std::make_unique<SymmHeap>(mesh, device, opt.heap));
  }
  c->common_init(opt);
  return c;
}

std::unique_ptr<Comm> Comm::create_virtual(int world, int device, const CommOptions& opt) {
  std::unique_ptr<Comm> c(new Comm());
  c->world_ = world;
  c->device_ = device;
  c->mesh_ = nullptr;
  c->heaps_ = SymmHeap::make_virtual(world, device, opt.heap);
  c->common_init(opt);
  return c;
}

void Comm::finalize() {
  if (mesh_ && !heaps_.empty()) heaps_[0]->release_multicast(mesh_);
}

Comm::~Comm() {
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  heaps_.clear();
  for (StatusBlock* s : status_)
    if (s) cudaFreeHost(s);
}

void Comm::host_barrier() {
  if (mesh_) mesh_->barrier();
}

// ----------------------------------------------------------------------------
// Status
// ----------------------------------------------------------------------------
StatusBlock Comm::status(int local) const {
  StatusBlock s;
  std::memcpy(&s, status_[size_t(local)], sizeof(s));
  return s;
}

void Comm::raise_if_failed() const {
  // A rank whose own wait ran out knows whom it was waiting for; a rank that was told to stop only
  // knows that.  Report the first kind if any local rank has it.
  int pick = -1;
  for (size_t i = 0; i < status_.size(); ++i) {
    const uint32_t code = status(int(i)).code;
    if (code == kOk) continue;
    if (pick < 0 || (code == kTimeout && status(pick).code != kTimeout)) pick = int(i);
  }
  if (pick < 0) return;
  const StatusBlock s = status(pick);
  std::ostringstream os;
  os << "[b200ipc] collective failed on rank " << s.rank << ": ";
  if (s.code == kTimeout) {
    os << "bounded wait ran out (site " << s.where << ", waiting for rank " << s.peer << ", wire " << s.wire << ", step "
       << s.step << ", expected flag 0x" << std::hex << s.expected << ", saw 0x" << s.seen << ")";
  } else {
    os << "aborted because another wire or rank gave up a bounded wait (site " << s.where
       << "); its output is incomplete";
  }
  throw Error(os.str());
}

void Comm::reset() {
  B200_CUDA_CHECK(cudaSetDevice(device_));
  B200_CUDA_CHECK(cudaDeviceSynchronize());
  host_barrier();  // nobody is still storing into my heap
  for (auto& h : heaps_) h->clear(false);
  B200_CUDA_CHECK(cudaDeviceSynchronize());
  for (StatusBlock* s : status_) std::memset(s, 0, sizeof(StatusBlock));
  // Start a fresh epoch well away from anything that may still sit in a ring.
  seq_ = (seq_ + 0x10000u) | 1u;
  bar_seq_ = 0;
  gemm_done_ = 0;
  ag_arrive_ = 0;
  host_barrier();
}

// ----------------------------------------------------------------------------
// Launch plumbing
// ----------------------------------------------------------------------------
size_t Comm::sym_alloc(size_t bytes, size_t align) {
  const HeapLayout& lay = heaps_[0]->layout();
  size_t start = (sym_used_ + align - 1) / align * align;
  B200_REQUIRE(start + bytes <= lay.staging_bytes,
               "symmetric allocation of " << bytes << " B does not fit (staging region " << lay.staging_bytes
                                          << " B, used " << sym_used_ << " B)");
  sym_used_ = start + bytes;
  return lay.staging_off + start;
}

size_t Comm::sym_offset_of(const void* p, int local) const {
  const SymmHeap& h = *heaps_[size_t(local)];
  const char* c = static_cast<const char*>(p);
  const char* lo = h.base() + h.layout().staging_off;
  const char* hi = lo + h.layout().staging_bytes;
  if (c >= lo && c < hi) return size_t(c - h.base());
  return SIZE_MAX;
}

void Comm::fill_views(KArgs* args, const void* const* ins, void* const* outs, size_t nelems, uint32_t flags) const {
  std::memset(args, 0, sizeof(KArgs));
  args->lay = heaps_[0]->layout();
  for (size_t i = 0; i < heaps_.size(); ++i) {
    const SymmHeap& h = *heaps_[i];
    RankView& v = args->v[i];
    v.rank = h.rank();
    v.world = world_;
    v.flags = flags | (trace_wires_ ? uint32_t(kTraceWires) : 0u);
    v.heap = h.base();
    for (int r = 0; r < kMaxRanks; ++r) v.peer[r] = r < world_ ? h.peer(r) : h.base();
    v.mc = h.multicast();
    v.in = ins ? ins[i] : nullptr;
    v.out = outs ? outs[i] : nullptr;
    v.nelems = nelems;
    v.status = status_[i];
    v.timeout_ns = timeout_ns_;
    v.seq_dev = device_seq_ ? reinterpret_cast<uint32_t*>(h.base() + h.layout().ctrl_off + kCtrlSeqOff) : nullptr;
  }
}

int Comm::resident_ctas(KernelFn fn, int threads, size_t smem) {
  auto key = std::make_pair(reinterpret_cast<const void*>(fn), threads);
  auto it = occupancy_cache_.find(key);
  int per_sm = 0;
  if (it == occupancy_cache_.end()) {
    B200_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, reinterpret_cast<const void*>(fn), threads, smem));
    occupancy_cache_[key] = per_sm;
  } else {
    per_sm = it->second;
  }
  int total = per_sm * sm_count_;
  if (nlocal() > 1) total /= nlocal();  // the virtual world's ranks share the GPU
  if (max_ctas_ > 0) total = std::min(total, max_ctas_);
  return total;
}

void Comm::launch(KernelFn fn, int ctas, int threads, KArgs* args, size_t smem, cudaStream_t stream, bool pdl) {
  void* params[] = {args};
  launch_raw(reinterpret_cast<const void*>(fn), ctas, threads, params, smem, stream, pdl);
}

void Comm::launch_raw(const void* fn, int ctas, int threads, void** params, size_t smem, cudaStream_t stream, bool pdl) {
  dim3 grid(unsigned(ctas), unsigned(nlocal()), 1);
  dim3 block(unsigned(threads), 1, 1);
  if (nlocal() > 1) {
    // ranks wait on each other inside the kernel: all block rows must be resident
    B200_CUDA_CHECK(cudaLaunchCooperativeKernel(fn, grid, block, params, smem, stream));
  } else {
    B200_CUDA_CHECK(launch_maybe_pdl(fn, grid, block, params, smem, stream, pdl));
  }
  ++launches_;
}

uint32_t Comm::take_seq(uint32_t advance) {
  if (device_seq_) return seq_;  // the device adds its own running offset
  // Flags only ever grow, which is what makes a stale ring entry harmless.  Before the
  // 32-bit counter would wrap, clear the rings and start over.
  // Every rank reaches the wrap at the same call, so the (collective) reset is safe.
  if (seq_ + advance + 1 < seq_) reset();
  uint32_t s = seq_;
  seq_ += advance;
  return s;
}

uint32_t Comm::take_barrier() {
  if (device_seq_) return 0;
  uint32_t b = bar_seq_;
  bar_seq_ += 4;
  return b;
}

// ----------------------------------------------------------------------------
// Geometry of the flag-in-data kernels
// ----------------------------------------------------------------------------
namespace {

struct LLPlan {
  int warps = 0, ctas = 0, nwires = 0;
  int64_t steps = 0;
  int slots = 1;
  bool per_step_flag = false;
};

int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace

CollInfo Comm::launch_ll(LLOpId op, AlgoSpec algo, DType t, const void* const* ins, void* const* outs, size_t nelems,
                         LaunchGeom geom, cudaStream_t stream, uint32_t flags) {
  const int N = world_;
  KernelFn fn = ll_kernel_lookup(op, t, algo.proto, N);
  B200_REQUIRE(fn != nullptr, "no kernel for world size " << N << " (supported: 2, 4, 8)");
  const int payload = payload_dw_of(algo.proto);
  const int txn = txn_bytes_of(algo.proto);
  const HeapLayout& lay = heaps_[0]->layout();

  // unit = wires that cooperate on one offset; need = wires that cover the data in one step
  int unit = 1;
  int64_t need = 1;
  int slots = kSequentialSlots;
  int max_wires = kMaxWires;
  switch (op) {
    case LLOpId::ArParallel: {
      unit = N;
      need = cdiv(make_partition(nelems, N).chunk_dw, payload) * N;
      slots = kParallelSlots;
      break;
    }
    case LLOpId::ArBisect: {
      B200_REQUIRE(N % 2 == 0, "bisect needs an even world size");
      unit = N / 2;
      int64_t chunk = round_up64(ceil_div64(make_partition(nelems, 2).chunk_dw, unit), 4);
      need = cdiv(chunk, payload) * unit;
      slots = kParallelSlots;
      break;
    }
    case LLOpId::ArSequential:
    case LLOpId::ArRing:
      need = cdiv(make_partition(nelems, N).chunk_dw, payload);
      break;
    case LLOpId::ArOneShot:
      need = cdiv(int64_t((nelems + 1) / 2), payload);
      max_wires = kMaxOneShotWires;
      slots = 1;
      break;
    case LLOpId::AgRing:
    case LLOpId::AgDirect:
      B200_REQUIRE(nelems % 2 == 0, "all-gather needs an even element count per rank (shards start on a dword)");
      need = cdiv(int64_t(nelems / 2), payload);
      break;
    case LLOpId::RsParallel:
      B200_REQUIRE(nelems % (2 * size_t(N)) == 0,
                   "flag-in-data reduce-scatter needs a multiple of 2 x world elements (slices start on a dword)");
      unit = N;
      need = cdiv(int64_t(nelems / size_t(N) / 2), payload) * N;
      slots = kParallelSlots;
      break;
  }
  if (need < unit) need = unit;

  LLPlan p;
  if (geom.warps > 0) {
    p.warps = geom.warps;
  } else {
    // small jobs: few warps per CTA so that wires spread over SMs; large: 16 warps
    int64_t w = need >= 16 * int64_t(sm_count_) ? 16 : (need >= 4 * int64_t(sm_count_) ? 8 : 4);
    w = std::min<int64_t>(w, need);
    p.warps = int(round_up64(w, unit));
  }
  B200_REQUIRE(p.warps >= 1 && p.warps <= 32, "warps per CTA must be 1..32, got " << p.warps);
  const int threads = p.warps * 32;
  int cap_ctas = resident_ctas(fn, threads, 0);
  B200_REQUIRE(cap_ctas >= 1, "kernel does not fit on the device with " << threads << " threads");
  cap_ctas = std::min<int>(cap_ctas, max_wires / p.warps);
  if (geom.ctas > 0) {
    p.ctas = geom.ctas;
    B200_REQUIRE(p.ctas <= cap_ctas, "requested " << p.ctas << " CTAs x " << p.warps << " warps, but only " << cap_ctas
                                                  << " CTAs can be resident at once (all wires of all ranks must run "
                                                     "concurrently) or fit the scratch rings");
  } else {
    p.ctas = int(std::min<int64_t>(cdiv(need, p.warps), cap_ctas));
  }
  p.nwires = p.ctas * p.warps;
  // The reference loops forever when the wire count is not a multiple of the group
  // size (allreduce.hpp:86-92); refuse instead.
  B200_REQUIRE(p.nwires % unit == 0 && p.nwires >= unit,
               "CTAs x warps = " << p.nwires << " must be a positive multiple of " << unit << " for this schedule");
  B200_REQUIRE(p.nwires <= max_wires, "too many wires: " << p.nwires << " > " << max_wires);

  switch (op) {
    case LLOpId::ArParallel: p.steps = parallel_steps(nelems, N, p.nwires, payload); break;
    case LLOpId::ArBisect: p.steps = bisect_steps(nelems, N, p.nwires, payload); break;
    case LLOpId::ArSequential:
    case LLOpId::ArRing: p.steps = sequential_steps(nelems, N, p.nwires, payload); break;
    case LLOpId::ArOneShot: p.steps = oneshot_steps(nelems, p.nwires, payload); break;
    case LLOpId::RsParallel:
      p.steps = reduce_scatter_steps(nelems, N, p.nwires, payload);
      B200_REQUIRE(p.steps <= kParallelSlots, "flag-in-data reduce-scatter: " << nelems << " elements need " << p.steps
                                                  << " steps on " << p.nwires << " wires, more than the "
                                                  << kParallelSlots << " a launch may take; use more wires or bulk/nvls");
      break;
    default: p.steps = allgather_steps(nelems, p.nwires, payload); break;
  }

  // Ring capacity (bytes) of what this geometry addresses.
  size_t ring_bytes = 0;
  switch (op) {
    case LLOpId::ArParallel: ring_bytes = size_t(p.nwires) * kParallelSlots * txn; break;
    case LLOpId::ArBisect: ring_bytes = size_t(kBisectFarBase + int64_t(p.nwires) * kParallelSlots) * txn; break;
    case LLOpId::ArOneShot: ring_bytes = 0; break;
    case LLOpId::RsParallel: ring_bytes = 2 * size_t(p.nwires) * kParallelSlots * txn; break;
    default: ring_bytes = size_t(N) * kSequentialSlots * p.nwires * txn; break;
  }
  B200_REQUIRE(ring_bytes <= lay.half_bytes, "scratch ring too small for this geometry");

  // reduce-scatter: always 2, so that bit 1 of the sequence number (the ring half) alternates
  const uint32_t adv = (op == LLOpId::ArOneShot)    ? uint32_t(p.steps + 1)
                       : (op == LLOpId::RsParallel) ? 2u
                                                    : seq_advance(p.steps, slots);
  const uint32_t first = take_seq(adv);

  KArgs args;
  fill_views(&args, ins, outs, nelems, flags);
  for (int i = 0; i < nlocal(); ++i) {
    args.v[i].seq = first;
    args.v[i].seq_step = adv;
    if (op == LLOpId::AgRing || op == LLOpId::AgDirect) {
      const char* o = static_cast<const char*>(outs[i]);
      if (static_cast<const char*>(ins[i]) == o + size_t(args.v[i].rank) * nelems * 2) args.v[i].flags |= kInPlace;
    }
  }
  launch(fn, p.ctas, threads, &args, 0, stream);

  CollInfo info;
  info.sched = algo.sched;
  info.proto = algo.proto;
  info.ctas = p.ctas;
  info.warps = p.warps;
  info.nwires = p.nwires;
  info.steps = p.steps;
  info.first_flag = first;
  info.launches = 1;
  return info;
}

// ----------------------------------------------------------------------------
// Large messages
// ----------------------------------------------------------------------------
CollInfo Comm::launch_bulk(BulkModeId mode, bool nvls, DType t, const void* const* ins, void* const* outs,
                           size_t nelems, LaunchGeom geom, cudaStream_t stream, uint32_t flags) {
  const int N = world_;
  if (nvls) B200_REQUIRE(has_nvls(), "NVLS was not set up for this communicator: " << heaps_[0]->nvls_note());
  KernelFn fn = bulk_kernel_lookup(mode, t, N, nvls);
  B200_REQUIRE(fn != nullptr, "no kernel for world size " << N << " (supported: 2, 4, 8)");
  const HeapLayout& lay = heaps_[0]->layout();
  if (mode == BulkModeId::ReduceScatter) B200_REQUIRE(nelems % size_t(N) == 0, "reduce-scatter input must divide by the world size");

  // Shard geometry, as in the kernel.
  int64_t shard_elems, shard_vec;
  if (mode == BulkModeId::AllReduce) {
    shard_vec = cdiv(cdiv(int64_t(nelems), 8), N);
    shard_elems = shard_vec * 8;
  } else if (mode == BulkModeId::ReduceScatter) {
    shard_elems = int64_t(nelems) / N;
    shard_vec = cdiv(shard_elems, 8);
  } else {
    shard_elems = int64_t(nelems);
    shard_vec = cdiv(shard_elems, 8);
  }
  const size_t sym_bytes = size_t(shard_vec) * 16 * size_t(N);
  const bool exact = (mode == BulkModeId::AllReduce) ? (nelems % (8 * size_t(N)) == 0) : (shard_elems % 8 == 0);

  // Zero-copy when the caller's buffers already live in the symmetric heap at the
  // same offset on every rank and the shards are vector-exact.
  //   all-reduce: in place on a symmetric buffer
  //   reduce-scatter: symmetric input
  //   all-gather: symmetric output
  size_t sym_off = SIZE_MAX;
  uint64_t copy_flags = 0;
  {
    const void* probe = (mode == BulkModeId::AllGather) ? static_cast<const void*>(outs[0]) : ins[0];
    size_t off = exact ? sym_offset_of(probe, 0) : SIZE_MAX;
    bool ok = off != SIZE_MAX && off % 16 == 0;
    for (int i = 0; ok && i < nlocal(); ++i) {
      const void* pi = (mode == BulkModeId::AllGather) ? static_cast<const void*>(outs[i]) : ins[i];
      ok = sym_offset_of(pi, i) == off;
    }
    if (ok) sym_off = off;
  }
  if (sym_off != SIZE_MAX) {
    if (mode == BulkModeId::AllReduce) {
      bool in_place = true;
      for (int i = 0; i < nlocal(); ++i) in_place &= (ins[i] == outs[i]);
      if (!in_place) copy_flags |= kBulkCopyOutBit;
    } else if (mode == BulkModeId::AllGather) {
      bool in_place = true;
      for (int i = 0; i < nlocal(); ++i)
        in_place &= (static_cast<const char*>(ins[i]) == static_cast<const char*>(outs[i]) + size_t(rank(i)) * nelems * 2);
      if (!in_place) copy_flags |= kBulkCopyInBit;
    }
  } else {
    // staged through what is left of the staging region after symmetric allocations
    size_t start = (sym_used_ + 255) / 256 * 256;
    B200_REQUIRE(start + sym_bytes <= lay.staging_bytes,
                 "message of " << nelems * 2 << " B needs " << sym_bytes << " B of staging, only "
                               << (lay.staging_bytes - start) << " B left; create the communicator with a larger staging region");
    sym_off = lay.staging_off + start;
    copy_flags = (mode == BulkModeId::ReduceScatter) ? kBulkCopyInBit : (kBulkCopyInBit | kBulkCopyOutBit);
  }

  const int threads = kBulkThreadsPerCta;
  int cap = std::min(resident_ctas(fn, threads, 0), kMaxBarrierCtas);
  B200_REQUIRE(cap >= 1, "bulk kernel does not fit on the device");
  const int64_t tile_vec = int64_t(threads);  // a slab: one vector per thread; a CTA keeps kU slabs in flight
  // Spread the tiles evenly: with T tiles and room for `cap` CTAs, every CTA gets
  // ceil(T / cap) tiles (a grid of `cap` would leave some CTAs with one tile more).
  const int64_t ntiles = std::max<int64_t>(1, cdiv(shard_vec, tile_vec));
  const int64_t rounds = cdiv(ntiles, cap);
  int ctas = geom.ctas > 0 ? geom.ctas : int(cdiv(ntiles, rounds));
  if (geom.ctas <= 0 && nvls && mode == BulkModeId::AllReduce && copy_flags == 0) {
    // The in-switch reduction is fed by few CTAs: every CTA runs its own cross-rank barrier pair, and a handful
    // of CTAs already keeps the links busy (16 MiB on 8 GPUs: 47.7 us with 8 CTAs, 58.3 us with 64).
    int want = nvls_ctas_for(nelems * 2);
    if (const char* e = std::getenv("B200IPC_NVLS_CTAS")) want = std::atoi(e);
    if (want > 0) ctas = int(std::min<int64_t>(std::min<int64_t>(want, cap), ntiles));
  }
  B200_REQUIRE(ctas <= cap, "requested " << ctas << " CTAs but only " << cap << " can be resident");

  KArgs args;
  fill_views(&args, ins, outs, nelems, flags);
  const uint32_t bar = take_barrier();
  for (int i = 0; i < nlocal(); ++i) {
    args.v[i].bar_seq = bar;
    args.v[i].aux[0] = sym_off;
    args.v[i].aux[1] = copy_flags;
  }
  launch(fn, ctas, threads, &args, 0, stream);

  CollInfo info;
  info.sched = nvls ? SchedKind::Nvls : SchedKind::Bulk;
  info.proto = ProtoKind::LL512;
  info.ctas = ctas;
  info.warps = threads / 32;
  info.nwires = ctas * threads / 32;
  info.steps = cdiv(cdiv(shard_vec, tile_vec), ctas);
  info.first_flag = bar;
  info.launches = 1;
  info.staged = copy_flags != 0;
  return info;
}

// ----------------------------------------------------------------------------
// Public collectives
// ----------------------------------------------------------------------------
AlgoSpec Comm::choose_all_reduce(size_t bytes, bool symmetric) const {
  AlgoSpec a;
  if (const char* e = std::getenv("B200IPC_PROTO")) {
    bool ag = false;
    AlgoSpec forced;
    if (parse_algo(e, &forced, &ag) && !ag && !forced.automatic) return forced;
  }
  if (oneshot_max_bytes_ != 0 || ll_max_bytes_ != 0) {
    // thresholds set by the caller override the built-in table
    if (bytes <= oneshot_max_bytes_) {
      a.sched = SchedKind::OneShot;
      a.proto = safe_protos_ ? ProtoKind::LL16 : ProtoKind::LL512;
    } else if (bytes <= ll_max_bytes_) {
      a.sched = SchedKind::Parallel;
      a.proto = safe_protos_ ? ProtoKind::LL16 : ProtoKind::LL512;
    } else {
      a.sched = (has_nvls() && world_ >= 8) ? SchedKind::Nvls : SchedKind::Bulk;
      a.proto = ProtoKind::LL512;
    }
    return a;
  }
  int rows = 0;
  const TuneRow* t = tune_table(world_, symmetric, &rows);
  for (int i = 0; i < rows; ++i) {
    if (t[i].max_bytes == 0 || bytes <= t[i].max_bytes) {
      a.sched = t[i].sched;
      a.proto = t[i].proto;
      break;
    }
  }
  if (a.sched == SchedKind::Nvls && !has_nvls()) a.sched = SchedKind::Bulk;
  if (safe_protos_ && (a.proto == ProtoKind::LL512 || a.proto == ProtoKind::LL128)) a.proto = ProtoKind::LL16;
  return a;
}

CollInfo Comm::all_reduce(AlgoSpec algo, DType t, const void* const* ins, void* const* outs, size_t nelems,
                          LaunchGeom geom, cudaStream_t stream, uint32_t extra_flags) {
  B200_REQUIRE(nelems > 0, "empty all-reduce");
  NvtxRange nvtx("all_reduce", algo, nelems * 2);
  B200_CUDA_CHECK(cudaSetDevice(device_));
  if (world_ == 1) {
    if (ins[0] != outs[0]) B200_CUDA_CHECK(cudaMemcpyAsync(outs[0], ins[0], nelems * 2, cudaMemcpyDeviceToDevice, stream));
    CollInfo info{};
    info.sched = SchedKind::OneShot;
    return info;
  }
  if (algo.automatic) {
    bool symmetric = true;
    for (int i = 0; i < nlocal(); ++i) symmetric &= (ins[i] == outs[i]) && sym_offset_of(ins[i], i) != SIZE_MAX;
    algo = choose_all_reduce(nelems * 2, symmetric);
  }
  for (int i = 0; i < nlocal(); ++i) {
    B200_REQUIRE((reinterpret_cast<uintptr_t>(ins[i]) & 3) == 0 && (reinterpret_cast<uintptr_t>(outs[i]) & 3) == 0,
                 "buffers must be 4-byte aligned");
  }
  switch (algo.sched) {
    case SchedKind::Parallel: return launch_ll(LLOpId::ArParallel, algo, t, ins, outs, nelems, geom, stream, extra_flags);
    case SchedKind::Sequential: return launch_ll(LLOpId::ArSequential, algo, t, ins, outs, nelems, geom, stream, extra_flags);
    case SchedKind::Ring: return launch_ll(LLOpId::ArRing, algo, t, ins, outs, nelems, geom, stream, extra_flags);
    case SchedKind::Bisect: return launch_ll(LLOpId::ArBisect, algo, t, ins, outs, nelems, geom, stream, extra_flags);
    case SchedKind::OneShot: return launch_ll(LLOpId::ArOneShot, algo, t, ins, outs, nelems, geom, stream, extra_flags);
    case SchedKind::Bulk: return launch_bulk(BulkModeId::AllReduce, false, t, ins, outs, nelems, geom, stream, extra_flags);
    default: return launch_bulk(BulkModeId::AllReduce, true, t, ins, outs, nelems, geom, stream, extra_flags);
  }
}

CollInfo Comm::all_gather(AlgoSpec algo, DType t, const void* const* ins, void* const* outs, size_t nelems,
                          LaunchGeom geom, cudaStream_t stream, uint32_t extra_flags) {
  B200_REQUIRE(nelems > 0, "empty all-gather");
  NvtxRange nvtx("all_gather", algo, nelems * 2);
  B200_CUDA_CHECK(cudaSetDevice(device_));
  if (world_ == 1) {
    if (ins[0] != outs[0]) B200_CUDA_CHECK(cudaMemcpyAsync(outs[0], ins[0], nelems * 2, cudaMemcpyDeviceToDevice, stream));
    CollInfo info{};
    info.sched = SchedKind::Ring;
    return info;
  }
  if (algo.automatic) {
    algo = AlgoSpec{};
    const size_t bytes = nelems * 2;
    // two ranks: the direct flag-in-data push moves the same bytes as any other form and needs no
    // barrier; measured ahead of the barrier-based kernels and of NCCL up to 64 MiB per rank
    // measured on 8 GPUs (bytes per rank): the direct push wins up to 1 MiB (23 us against NCCL's 47), the
    // barrier kernel with peer loads from 2 to 8 MiB, the flag-in-data ring above (level with NCCL)
    if (world_ == 2 || bytes <= (size_t(1) << 20) || nelems % 8 != 0) {
      algo.sched = SchedKind::Ring;
      algo.proto = safe_protos_ ? ProtoKind::LL16 : ProtoKind::LL512;
      algo.direct_allgather = true;
    } else if (bytes <= (size_t(8) << 20)) {
      algo.sched = SchedKind::Bulk;
    } else {
      algo.sched = SchedKind::Ring;
      algo.proto = safe_protos_ ? ProtoKind::LL16 : ProtoKind::LL512;
    }
  }
  if (algo.sched == SchedKind::Bulk || algo.sched == SchedKind::Nvls)
    return launch_bulk(BulkModeId::AllGather, algo.sched == SchedKind::Nvls, t, ins, outs, nelems, geom, stream, extra_flags);
  B200_REQUIRE(algo.sched == SchedKind::Ring, "all-gather runs on the ring, direct, bulk or nvls schedules");
  return launch_ll(algo.direct_allgather ? LLOpId::AgDirect : LLOpId::AgRing, algo, t, ins, outs, nelems, geom, stream,
                   extra_flags);
}

CollInfo Comm::reduce_scatter(AlgoSpec algo, DType t, const void* const* ins, void* const* outs, size_t nelems,
                              LaunchGeom geom, cudaStream_t stream, uint32_t extra_flags) {
  B200_REQUIRE(nelems > 0, "empty reduce-scatter");
  NvtxRange nvtx("reduce_scatter", algo, nelems * 2);
  B200_CUDA_CHECK(cudaSetDevice(device_));
  if (world_ == 1) {
    if (ins[0] != outs[0]) B200_CUDA_CHECK(cudaMemcpyAsync(outs[0], ins[0], nelems * 2, cudaMemcpyDeviceToDevice, stream));
    CollInfo info{};
    info.sched = SchedKind::Bulk;
    return info;
  }
  const bool was_auto = algo.automatic;
  if (algo.automatic) {
    algo = AlgoSpec{};
    // small inputs: one flag-in-data push to each slice's owner, no barrier
    if (nelems % (2 * size_t(world_)) == 0 && nelems * 2 <= (safe_protos_ ? kReduceScatterLLMaxBytes / 2 : kReduceScatterLLMaxBytes)) {
      algo.sched = SchedKind::Parallel;
      algo.proto = safe_protos_ ? ProtoKind::LL16 : ProtoKind::LL512;
    } else {
      // peer loads: level with or ahead of the in-switch form at 2, 4 and 8 ranks (16 MiB: 44.6 us against 48.9 on 4
      // GPUs, 50.6 against 52.1 on 8)
      algo.sched = SchedKind::Bulk;
    }
  }
  if (algo.sched == SchedKind::Parallel) {
    if (!was_auto) return launch_ll(LLOpId::RsParallel, algo, t, ins, outs, nelems, geom, stream, extra_flags);
    // `auto`: a device on which fewer wires can be resident than the cut-off assumes takes the barrier kernel instead
    // (the geometry check throws before anything is launched or any sequence number is taken)
    try {
      return launch_ll(LLOpId::RsParallel, algo, t, ins, outs, nelems, geom, stream, extra_flags);
    } catch (const std::exception&) {
      algo.sched = SchedKind::Bulk;
    }
  }
  B200_REQUIRE(algo.sched == SchedKind::Bulk || algo.sched == SchedKind::Nvls,
               "reduce-scatter runs on the parallel (flag-in-data), bulk or nvls schedules");
  return launch_bulk(BulkModeId::ReduceScatter, algo.sched == SchedKind::Nvls, t, ins, outs, nelems, geom, stream,
                     extra_flags);
}

}  // namespace b200ipc
