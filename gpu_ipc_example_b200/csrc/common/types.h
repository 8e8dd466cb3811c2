// Plain-data types shared by host code, device kernels and the CPU emulator.
// Nothing here includes a CUDA header, so the emulator builds with g++ alone.
#pragma once

#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define B200_HD __host__ __device__ __forceinline__
#else
#define B200_HD inline
#endif

namespace b200ipc {

// One NVSwitch domain of a B200 node has 8 GPUs.
constexpr int kMaxRanks = 8;
// Upper bound on concurrently running wires (warps) of one rank for the
// flag-in-data schedules; scratch rings are sized from it.  The reference uses
// the same bound (parallel_transmit.hpp:29-31, sequential_transmit.hpp:48-52).
constexpr int kMaxWires = 4096;
// Wires of the one-shot schedule (tiny messages only).
constexpr int kMaxOneShotWires = 2048;

enum class DType : int { F16 = 0, BF16 = 1 };

// Wire formats ("protos").  Names follow the message width per warp transaction.
enum class ProtoKind : int {
  LL8 = 0,    // 8 B per lane  {data32, flag32}           256 B txn, 128 B payload
  LL16 = 1,   // 16 B per lane {d0, flag, d1, flag}       512 B txn, 256 B payload
  LL128 = 2,  // 4 B per lane, flag closes each 64 B half 128 B txn, 120 B payload
  LL512 = 3,  // 16 B per lane, flag closes each 64 B     512 B txn, 480 B payload
};

// Schedules ("transmits").
enum class SchedKind : int {
  Parallel = 0,    // warp-parallel two-phase (reduce-scatter + all-gather), 2 hops
  Sequential = 1,  // one warp serves every peer
  Ring = 2,        // ring reduce-scatter + ring all-gather
  Bisect = 3,      // two-level: partner pair, then same-parity group
  OneShot = 4,     // everyone pushes everything, everyone reduces: 1 hop
  Bulk = 5,        // large messages: peer reads + pushes with per-CTA barriers
  Nvls = 6,        // NVSwitch multimem.ld_reduce / multimem.st
};

enum StatusCode : uint32_t {
  kOk = 0,
  kTimeout = 1,        // a bounded wait ran out
  kAbortedByPeer = 2,  // another wire or rank raised the abort word
  kBadArgument = 3,
};

// Written by the first wire that gives up a bounded wait; lives in pinned host
// memory so that the host can read it without touching the device.
struct StatusBlock {
  uint32_t code;
  uint32_t rank;
  uint32_t peer;
  uint32_t wire;
  uint32_t step;
  uint32_t expected;
  uint32_t seen;
  uint32_t where;  // schedule-specific site id of the wait that gave up
  uint64_t timeouts;  // how many wires reported
};

// Bits of RankView::flags.
enum ViewFlags : uint32_t {
  kRoundEachAdd = 1u << 0,  // round the running sum to T after each add (the reference sums in T)
  kMuteSends = 1u << 1,     // fault injection: this rank skips every remote store
  kInPlace = 1u << 2,
  kTraceWires = 1u << 3,    // debug: every completed wait leaves a time-stamped record in the trace ring
};

// Byte offsets of the regions inside every rank's symmetric heap.  Identical
// on all ranks, so a peer address is peer_base + the same offset.
struct HeapLayout {
  size_t ctrl_off, ctrl_bytes;          // abort word, barrier pads, device counters
  size_t half_off[2], half_bytes;       // scatter sink (0) / gather sink (1) rings
  size_t oneshot_off, oneshot_bytes;    // one-shot landing zone
  size_t staging_off, staging_bytes;    // bulk / NVLS staging and user symmetric tensors
  size_t total_bytes;
};

// Offsets inside the control region.
constexpr size_t kCtrlAbortOff = 0;            // uint32 abort word
constexpr size_t kCtrlClaimOff = 4;            // uint32: which wire writes this rank's status record (0 = nobody yet)
constexpr size_t kCtrlSeqOff = 256;            // uint32 {sequence offset, finished-CTA counter, barrier offset, -}
constexpr size_t kCtrlBarrierOff = 4096;       // uint32 pad[kMaxBarrierCtas][kMaxRanks]
constexpr int kMaxBarrierCtas = 1024;
// Debug trace ring (B200IPC_DEBUG=1): uint32 {next index, -, -, -} at kCtrlTraceOff, then
// kTraceEntries records.  The ring keeps the most recent records; the index keeps counting.
struct TraceRecord {
  uint64_t t_ns;     // global timer when the wait completed
  uint32_t wire;     // warp index of the rank
  uint32_t site;     // schedule-specific id of the wait (0 scatter sink, 1 gather sink, 2/3 bisect far, 4 one-shot, 5 fused one-shot)
  uint32_t peer;     // rank that sent the transaction
  uint32_t step;     // loop iteration of the wire
  uint32_t flag;     // the sequence flag the transaction carried
  uint32_t rank;     // this rank
};
constexpr size_t kCtrlTraceOff = 65536;
constexpr uint32_t kTraceEntries = 4096;
constexpr size_t kCtrlBytes = 2u << 20;
static_assert(kCtrlTraceOff + 16 + size_t(kTraceEntries) * sizeof(TraceRecord) <= kCtrlBytes, "trace ring must fit the control region");

// Everything one rank's kernel needs.  In the single-GPU emulation of N ranks
// ("virtual world") one launch carries N of these and blockIdx.y selects one.
struct RankView {
  int rank;
  int world;
  uint32_t seq;        // first flag value of this launch
  uint32_t flags;      // ViewFlags
  char* heap;          // my own heap base
  char* peer[kMaxRanks];   // every rank's heap base as mapped here (peer[rank] == heap)
  char* mc;            // multicast (NVLS) mapping of the heap, or nullptr
  const void* in;
  void* out;
  uint64_t nelems;
  StatusBlock* status;     // pinned host memory
  uint64_t timeout_ns;     // time limit of one bounded wait
  uint32_t bar_seq;        // barrier generation for Bulk/Nvls
  uint32_t seq_step;       // how far this launch advances the device-side sequence counter
  uint32_t* seq_dev;       // {offset, done-counter} in device memory when launches are graph-captured, else nullptr
  uint64_t aux[4];         // schedule/fusion specific (offsets, scalars)
};

struct KArgs {
  RankView v[kMaxRanks];
  HeapLayout lay;
};

B200_HD size_t dtype_size(DType) { return 2; }

}  // namespace b200ipc
