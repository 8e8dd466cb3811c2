// CPU emulator of the flag-in-data collectives.
//
// Runs the very schedule templates the GPU kernels run (coll/schedules.h) with
// the scalar backend of emu/host_backend.h.  A "rank" is either a thread of this
// process (b200emu_run_threads) or a separate process whose heap lives in a
// shared-memory segment that every rank has mapped (b200emu_run_rank): the
// segment plays the part of the peer mappings a GPU world gets from the CUDA
// handle exchange.  A rank executes its wires one after the other; that cannot
// deadlock because wire w only ever talks to wire w of the other ranks and all
// ranks walk the wires in the same order.
//
// Purposes: (1) the no-GPU plumbing test of the protocols, (2) the oracle for the
// byte image of a transaction (b200emu_wire_image), (3) host-side fault injection
// (a rank that never sends, a bounded wait that runs out) without touching a GPU.
//
// The reference has no such component; its place is taken there by commented-out
// stage simulators (allreduce.cpp:37-517, 588-830).
#include <sys/mman.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "../coll/schedules.h"
#include "../common/heap_layout.h"
#include "host_backend.h"

namespace b200ipc {
namespace {

struct EmuJob {
  int op;      // LLOpId numbering: 0 parallel, 1 sequential, 2 ring, 3 bisect, 4 oneshot, 5 ag ring, 6 ag direct, 7 reduce-scatter
  int proto;   // ProtoKind
  int dtype;   // DType
  int world;
  int nwires;
  uint32_t seq;
  uint32_t flags;
  uint64_t nelems;
  uint64_t timeout_ns;
};

template <class B, int N>
void run_rank_typed(const EmuJob& job, const RankView& view, const HeapLayout& lay) {
  Ctx<B> c;
  c.me = &view;
  c.lay = &lay;
  c.rank = view.rank;
  c.world = view.world;
  c.nwires = job.nwires;
  c.seq = job.seq;
  c.flags = view.flags;
  c.in = static_cast<const uint32_t*>(view.in);
  c.out = static_cast<uint32_t*>(view.out);
  c.nelems = job.nelems;
  c.waiter.abort_word = reinterpret_cast<std::atomic<uint32_t>*>(view.heap + lay.ctrl_off + kCtrlAbortOff);
  for (int r = 0; r < N; ++r)
    c.waiter.peer_abort[r] = reinterpret_cast<std::atomic<uint32_t>*>(view.peer[r] + lay.ctrl_off + kCtrlAbortOff);
  c.waiter.status = view.status;
  c.waiter.timeout_ns = job.timeout_ns;
  c.waiter.world = N;
  for (int w = 0; w < job.nwires; ++w) {
    c.waiter.wire = w;
    if (c.waiter.abort_word->load() != 0) break;
    switch (job.op) {
      case 0: run_parallel<B, N>(c, w); break;
      case 1: run_sequential<B, N>(c, w); break;
      case 2: run_ring_allreduce<B, N>(c, w); break;
      case 3: run_bisect<B, N>(c, w); break;
      case 4: run_oneshot<B, N>(c, w); break;
      case 5: run_ring_allgather<B, N>(c, w); break;
      case 7: run_reduce_scatter<B, N>(c, w); break;
      default: run_direct_allgather<B, N>(c, w); break;
    }
  }
  if (c.waiter.abort_word->load() != 0 && view.status->code == kOk) view.status->code = kAbortedByPeer;
}

template <ProtoKind K, DType T>
bool run_rank_world(const EmuJob& job, const RankView& view, const HeapLayout& lay) {
  using B = HostBackend<K, T>;
  switch (job.world) {
    case 2: run_rank_typed<B, 2>(job, view, lay); return true;
    case 4: run_rank_typed<B, 4>(job, view, lay); return true;
    case 8: run_rank_typed<B, 8>(job, view, lay); return true;
    default: return false;
  }
}

template <DType T>
bool run_rank_proto(const EmuJob& job, const RankView& view, const HeapLayout& lay) {
  switch (static_cast<ProtoKind>(job.proto)) {
    case ProtoKind::LL8: return run_rank_world<ProtoKind::LL8, T>(job, view, lay);
    case ProtoKind::LL16: return run_rank_world<ProtoKind::LL16, T>(job, view, lay);
    case ProtoKind::LL128: return run_rank_world<ProtoKind::LL128, T>(job, view, lay);
    case ProtoKind::LL512: return run_rank_world<ProtoKind::LL512, T>(job, view, lay);
  }
  return false;
}

bool run_rank(const EmuJob& job, const RankView& view, const HeapLayout& lay) {
  return job.dtype == int(DType::F16) ? run_rank_proto<DType::F16>(job, view, lay)
                                      : run_rank_proto<DType::BF16>(job, view, lay);
}

bool geometry_ok(const EmuJob& job) {
  if (job.nwires < 1) return false;
  if (job.op == 4) return job.nwires <= kMaxOneShotWires;
  if (job.nwires > kMaxWires) return false;
  if (job.op == 0) return job.nwires % job.world == 0;
  if (job.op == 7)
    return job.nwires % job.world == 0 && job.nelems % (2 * uint64_t(job.world)) == 0 &&
           reduce_scatter_steps(job.nelems, job.world, job.nwires, payload_dw_of(static_cast<ProtoKind>(job.proto))) <=
               kParallelSlots;
  if (job.op == 3) return job.world % 2 == 0 && job.nwires % (job.world / 2) == 0;
  if (job.op >= 5) return job.nelems % 2 == 0;
  return true;
}

}  // namespace
}  // namespace b200ipc

using namespace b200ipc;

extern "C" {

// Bytes of one rank's heap in the emulator (no staging region beyond the minimum).
uint64_t b200emu_heap_bytes() { return make_heap_layout(0).total_bytes; }

// How far the sequence number moves for this job (callers keep `seq` in step).
uint32_t b200emu_seq_advance(int op, int proto, int world, int nwires, uint64_t nelems) {
  const int payload = payload_dw_of(static_cast<ProtoKind>(proto));
  switch (op) {
    case 0: return seq_advance(parallel_steps(nelems, world, nwires, payload), kParallelSlots);
    case 1:
    case 2: return seq_advance(sequential_steps(nelems, world, nwires, payload), kSequentialSlots);
    case 3: return seq_advance(bisect_steps(nelems, world, nwires, payload), kParallelSlots);
    case 4: return uint32_t(oneshot_steps(nelems, nwires, payload) + 1);
    case 7: return 2;
    default: return seq_advance(allgather_steps(nelems, nwires, payload), kSequentialSlots);
  }
}

// One rank of a multi-process world.  `segment` is a mapping, shared by all ranks,
// of world * b200emu_heap_bytes() zero-initialised bytes.  Returns 0 on success, 1 when a
// bounded wait ran out or a peer aborted (details in status[8]), 2 for bad arguments.
int b200emu_run_rank(void* segment, int rank, int world, int op, int proto, int dtype, const void* in, void* out,
                     uint64_t nelems, int nwires, uint32_t seq, uint32_t flags, uint64_t timeout_ms,
                     uint32_t* status_out) {
  EmuJob job{op, proto, dtype, world, nwires, seq, flags, nelems, timeout_ms * 1000000ull};
  if (!geometry_ok(job) || rank < 0 || rank >= world) return 2;
  const HeapLayout lay = make_heap_layout(0);
  RankView v{};
  StatusBlock st{};
  v.rank = rank;
  v.world = world;
  v.flags = flags;
  char* base = static_cast<char*>(segment);
  v.heap = base + size_t(rank) * lay.total_bytes;
  for (int r = 0; r < kMaxRanks; ++r) v.peer[r] = base + size_t(r < world ? r : rank) * lay.total_bytes;
  v.in = in;
  v.out = out;
  v.nelems = nelems;
  v.status = &st;
  if (!run_rank(job, v, lay)) return 2;
  if (status_out) {
    const uint32_t s[8] = {st.code, st.rank, st.peer, st.wire, st.step, st.expected, st.seen, st.where};
    std::memcpy(status_out, s, sizeof(s));
  }
  return st.code == kOk ? 0 : 1;
}

// Whole world inside this process, one thread per rank.  ins/outs: world pointers.
// mute_rank >= 0 makes that rank skip every send (fault injection); skip_rank >= 0
// makes that rank not take part at all.  status_out: world * 8 words.
int b200emu_run_threads(int world, int op, int proto, int dtype, const void* const* ins, void* const* outs,
                        uint64_t nelems, int nwires, uint32_t seq, uint32_t flags, uint64_t timeout_ms, int mute_rank,
                        int skip_rank, uint32_t* status_out, void** heaps_inout) {
  EmuJob job{op, proto, dtype, world, nwires, seq, flags, nelems, timeout_ms * 1000000ull};
  if (!geometry_ok(job)) return 2;
  const HeapLayout lay = make_heap_layout(0);
  // Anonymous mappings: zero-filled, and untouched pages cost nothing.
  std::vector<char*> heaps(static_cast<size_t>(world), nullptr);
  const bool keep = heaps_inout != nullptr;
  for (int r = 0; r < world; ++r) {
    if (keep && heaps_inout[r]) {
      heaps[size_t(r)] = static_cast<char*>(heaps_inout[r]);
      continue;
    }
    void* p = ::mmap(nullptr, lay.total_bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (p == MAP_FAILED) return 2;
    heaps[size_t(r)] = static_cast<char*>(p);
    if (keep) heaps_inout[r] = p;
  }
  std::vector<StatusBlock> st(static_cast<size_t>(world));
  std::vector<RankView> views(static_cast<size_t>(world));
  for (int r = 0; r < world; ++r) {
    RankView& v = views[size_t(r)];
    std::memset(&v, 0, sizeof(v));
    std::memset(&st[size_t(r)], 0, sizeof(StatusBlock));
    v.rank = r;
    v.world = world;
    v.flags = flags | (r == mute_rank ? uint32_t(kMuteSends) : 0u);
    v.heap = heaps[size_t(r)];
    for (int q = 0; q < kMaxRanks; ++q) v.peer[q] = heaps[size_t(q < world ? q : r)];
    v.in = ins[r];
    v.out = outs[r];
    v.nelems = nelems;
    v.status = &st[size_t(r)];
  }
  std::vector<std::thread> threads;
  std::atomic<int> bad{0};
  for (int r = 0; r < world; ++r) {
    if (r == skip_rank) continue;
    threads.emplace_back([&, r] {
      if (!run_rank(job, views[size_t(r)], lay)) bad.store(1);
    });
  }
  for (auto& t : threads) t.join();
  int rc = bad.load() ? 2 : 0;
  for (int r = 0; r < world; ++r) {
    const StatusBlock& s = st[size_t(r)];
    if (status_out) {
      const uint32_t w[8] = {s.code, s.rank, s.peer, s.wire, s.step, s.expected, s.seen, s.where};
      std::memcpy(status_out + 8 * r, w, sizeof(w));
    }
    if (s.code != kOk && rc == 0) rc = 1;
  }
  if (!keep)
    for (char* h : heaps) ::munmap(h, lay.total_bytes);
  return rc;
}

void b200emu_free_heaps(int world, void** heaps) {
  const HeapLayout lay = make_heap_layout(0);
  for (int r = 0; r < world; ++r)
    if (heaps[r]) {
      ::munmap(heaps[r], lay.total_bytes);
      heaps[r] = nullptr;
    }
}

// Copies `bytes` at `offset` of an emulated heap (same layout as the GPU heap).
void b200emu_peek(const void* heap, uint64_t offset, uint64_t bytes, void* dst) {
  std::memcpy(dst, static_cast<const char*>(heap) + offset, bytes);
}

// region: 0 ctrl, 1 scatter half, 2 gather half, 3 one-shot, 4 staging, 5 total bytes, 6 half bytes
uint64_t b200emu_layout(int region, uint64_t staging_bytes) {
  const HeapLayout l = make_heap_layout(staging_bytes);
  switch (region) {
    case 0: return l.ctrl_off;
    case 1: return l.half_off[0];
    case 2: return l.half_off[1];
    case 3: return l.oneshot_off;
    case 4: return l.staging_off;
    case 5: return l.total_bytes;
    default: return l.half_bytes;
  }
}

// The byte image of one transaction: payload_dw dwords of payload (fewer than the
// proto's capacity are zero-padded) and the flag.  Returns the transaction size
// in dwords, or 0 for a bad proto.
int b200emu_wire_image(int proto, const uint32_t* payload, int payload_dw, uint32_t flag, uint32_t* image) {
  auto build = [&](auto wf) -> int {
    using WF = decltype(wf);
    for (int s = 0; s < WF::kTxnDw; ++s) image[s] = WF::is_flag_slot(s) ? flag : 0u;
    for (int k = 0; k < WF::kPayloadDw && k < payload_dw; ++k) image[WF::payload_slot(k)] = payload[k];
    return WF::kTxnDw;
  };
  switch (static_cast<ProtoKind>(proto)) {
    case ProtoKind::LL8: return build(WireFormat<ProtoKind::LL8>{});
    case ProtoKind::LL16: return build(WireFormat<ProtoKind::LL16>{});
    case ProtoKind::LL128: return build(WireFormat<ProtoKind::LL128>{});
    case ProtoKind::LL512: return build(WireFormat<ProtoKind::LL512>{});
  }
  return 0;
}

int b200emu_payload_dw(int proto) { return payload_dw_of(static_cast<ProtoKind>(proto)); }
int b200emu_txn_bytes(int proto) { return txn_bytes_of(static_cast<ProtoKind>(proto)); }

// fp16 / bf16 conversion helpers exposed for tests of the host arithmetic.
float b200emu_to_float(int dtype, uint16_t v) { return to_float(static_cast<DType>(dtype), v); }
uint16_t b200emu_from_float(int dtype, float f) { return from_float(static_cast<DType>(dtype), f); }

}  // extern "C"
