// The flag-in-data schedules, written once against a small "backend" interface
// so that the same code runs as a warp on the GPU (backend = DevBackend in
// proto/dev_backend.cuh) and as a scalar loop in the CPU emulator (backend =
// HostBackend in emu/host_backend.h).  What is shared is exactly the part that
// is easy to get wrong: who sends which piece to whom, where it lands in the
// peer's scratch ring, which flag value guards it and in which order partial
// sums are added.
//
// Vocabulary: a *wire* is one warp; it is strictly sequential.  The input of
// total_dw dwords (2 x 16-bit elements each) is cut into `world` equal chunks
// of chunk_dw dwords; chunk y is owned (reduced) by rank y.  Scratch half 0
// receives reduce-scatter traffic ("scatter sink"), half 1 receives all-gather
// traffic ("gather sink").  All polling is on the rank's own memory; the only
// traffic that crosses NVLink is B::send (a remote vector store).
//
// Backend interface used below (all static, all warp-collective on the GPU):
//   B::kPayloadDw, B::kTxnBytes
//   B::Msg, B::Acc
//   B::load(Msg&, const uint32_t* buf, int64 dw, int64 end_dw, int64 odd_dw)
//   B::store(uint32_t* buf, int64 dw, int64 end_dw, int64 odd_dw, const Msg&)
//   B::shuffle(Msg&) / B::restore(Msg&)      payload <-> wire order
//   B::set_flags(Msg&, flag)
//   B::send(char* dst, const Msg&)           remote store of one transaction
//   B::try_recv(Msg&, const char* src, flag) local load; true when complete
//   B::acc_init(Acc&, const Msg&), B::acc_add(Acc&, const Msg&, bool round_each),
//   B::acc_to_msg(Msg&, const Acc&)
// and a context Cx with the rank's pointers plus
//   bool Cx::wait(Msg&, const char* src, uint32 flag, int site, int peer, int step)
// which spins on try_recv under a time limit and returns false when the
// collective has been aborted (the wire then returns at once), and
//   bool B::wait_many<CNT>(waiter, Msg (&m)[CNT], src(i), peer(i), pending bits, flag, site, step, rank)
// which does the same for several transactions whose polls may overlap (recv_in_order below).
//
// Capability parity (schedules): parallel_transmit.hpp:62-132 (two-phase,
// sub-group parallel), sequential_transmit.hpp:82-208 (one sub-group serves all
// peers), sequential_transmit.hpp:429-516 (ring all-reduce and all-gather),
// bisect_transmit.hpp:286-424 (two-level).  The one-shot and direct all-gather
// schedules have no counterpart there.
#pragma once

#include "../common/types.h"

namespace b200ipc {

constexpr int kParallelSlots = 8;    // parallel_transmit.hpp:29
constexpr int kSequentialSlots = 4;  // sequential_transmit.hpp:48
constexpr int kRingSlots = 4;        // sequential_transmit.hpp:250
constexpr int kOneShotSlots = 4;
constexpr int kOneShotStride = 512;  // bytes per landing slot, whatever the proto
constexpr int64_t kBisectFarBase = int64_t(kMaxWires) * kParallelSlots;  // in transactions

B200_HD int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
B200_HD int64_t round_up64(int64_t a, int64_t b) { return ceil_div64(a, b) * b; }

// How a buffer of nelems 16-bit elements is cut into per-rank chunks.
struct Partition {
  int64_t total_dw;  // dwords covering the buffer (last one half-filled when nelems is odd)
  int64_t chunk_dw;  // dwords per chunk, multiple of 4 so that chunk bases stay 16 B aligned
  int64_t odd_dw;    // index of the half-filled dword, or -1
};

B200_HD Partition make_partition(uint64_t nelems, int parts) {
  Partition p;
  p.total_dw = int64_t((nelems + 1) / 2);
  p.chunk_dw = round_up64(ceil_div64(p.total_dw, parts), 4);
  if (p.chunk_dw == 0) p.chunk_dw = 4;
  p.odd_dw = (nelems & 1) ? p.total_dw - 1 : -1;
  return p;
}

B200_HD int64_t min64(int64_t a, int64_t b) { return a < b ? a : b; }

// Number of loop iterations of one launch; identical on every rank and wire,
// which is what keeps the flag sequence in step.
B200_HD int64_t parallel_steps(uint64_t nelems, int world, int nwires, int payload_dw) {
  Partition p = make_partition(nelems, world);
  return ceil_div64(p.chunk_dw, int64_t(nwires / world) * payload_dw);
}
B200_HD int64_t sequential_steps(uint64_t nelems, int world, int nwires, int payload_dw) {
  Partition p = make_partition(nelems, world);
  return ceil_div64(p.chunk_dw, int64_t(nwires) * payload_dw);
}
B200_HD int64_t bisect_steps(uint64_t nelems, int world, int nwires, int payload_dw) {
  Partition h = make_partition(nelems, 2);
  int bi = world / 2;
  int64_t chunk = round_up64(ceil_div64(h.chunk_dw, bi), 4);
  return ceil_div64(chunk, int64_t(nwires / bi) * payload_dw);
}
B200_HD int64_t oneshot_steps(uint64_t nelems, int nwires, int payload_dw) {
  int64_t total_dw = int64_t((nelems + 1) / 2);
  int64_t s = ceil_div64(total_dw, int64_t(nwires) * payload_dw);
  return s < 1 ? 1 : s;
}
B200_HD int64_t allgather_steps(uint64_t nelems_per_rank, int nwires, int payload_dw) {
  int64_t dw = int64_t((nelems_per_rank + 1) / 2);
  int64_t s = ceil_div64(dw, int64_t(nwires) * payload_dw);
  return s < 1 ? 1 : s;
}

// How far the sequence number moves per launch (flag = seq + t / slots).
// The reference over-advances by the step count (allreduce.hpp:51-56); here it is
// the number of distinct flag values used, plus one of distance.
B200_HD uint32_t seq_advance(int64_t steps, int slots) {
  return uint32_t(ceil_div64(steps, slots) + 1);
}

template <class B>
struct Ctx {
  const RankView* me;     // this rank's launch arguments (kernel parameter space on the GPU)
  const HeapLayout* lay;
  int rank;
  int world;
  int nwires;
  uint32_t seq;
  uint32_t flags;
  const uint32_t* in;
  uint32_t* out;
  uint64_t nelems;
  typename B::Waiter waiter;

  B200_HD char* sink(int half) const { return me->heap + lay->half_off[half]; }
  B200_HD char* peer_sink(int half, int r) const { return me->peer[r] + lay->half_off[half]; }
  B200_HD char* oneshot() const { return me->heap + lay->oneshot_off; }
  B200_HD char* peer_oneshot(int r) const { return me->peer[r] + lay->oneshot_off; }
  B200_HD bool round_each() const { return (flags & kRoundEachAdd) != 0; }
  B200_HD bool muted() const { return (flags & kMuteSends) != 0; }
  B200_HD void send(char* dst, const typename B::Msg& m) const {
    if (!muted()) B::send(dst, m);
  }
  B200_HD bool tracing() const { return (flags & kTraceWires) != 0; }
  B200_HD bool wait(typename B::Msg& m, const char* src, uint32_t flag, int site, int peer,
                    int64_t step) const {
    if (!B::wait(waiter, m, src, flag, site, peer, step, rank)) return false;
    if (tracing()) waiter.trace(site, peer, step, flag);
    return true;
  }
};

#define B200_WAIT(c, m, src, flag, site, peer, step) \
  if (!(c).wait(m, src, flag, site, peer, step)) return

template <class B>
B200_HD char* txn_at(char* base, int64_t idx) { return base + idx * B::kTxnBytes; }

// Transactions a wire keeps in registers while their polls overlap.  A poll is a round trip to
// L2; a wire that expects world - 1 transactions polls them in groups of this size instead of
// one after the other.
constexpr int kPollGroup = 4;

// Receives the transactions numbered LO .. HI-1 (number i sits at src(i) and was sent by rank
// peer(i)) and hands them IN ORDER to use(i, msg).  Number `skip` is not received: `own` is
// handed over in its place (-1: nothing is skipped).  Returns false when the collective was aborted.
template <class B, int LO, int HI, class SrcFn, class PeerFn, class UseFn>
B200_HD bool recv_in_order(const Ctx<B>& c, uint32_t flag, int site, int64_t step, int skip, const typename B::Msg& own,
                           SrcFn src, PeerFn peer, UseFn use) {
  if constexpr (LO >= HI) {
    return true;
  } else {
    constexpr int CNT = (HI - LO) < kPollGroup ? (HI - LO) : kPollGroup;
    typename B::Msg m[CNT];
    uint32_t pending = (1u << CNT) - 1u;
    if (skip >= LO && skip < LO + CNT) pending &= ~(1u << (skip - LO));
    if (pending != 0 &&
        !B::template wait_many<CNT>(
            c.waiter, m, [&](int k) { return src(LO + k); }, [&](int k) { return peer(LO + k); }, pending, flag, site,
            step, c.rank))
      return false;
#pragma unroll
    for (int k = 0; k < CNT; ++k) {
      if (LO + k == skip) {
        use(LO + k, own);
      } else {
        if (c.tracing()) c.waiter.trace(site, peer(LO + k), step, flag);
        use(LO + k, m[k]);
      }
    }
    return recv_in_order<B, LO + CNT, HI>(c, flag, site, step, skip, own, src, peer, use);
  }
}

// ---------------------------------------------------------------------------
// Parallel two-phase all-reduce.  Wires come in groups of `world`; wire
// (g, y) of rank r handles chunk y at the group's offset.  If y != r it pushes
// its slice to the owner and waits for the reduced slice to come back; if
// y == r it collects world-1 slices, reduces and pushes the result to everyone.
// ---------------------------------------------------------------------------
template <class B, int N>
B200_HD void run_parallel(const Ctx<B>& c, int wire) {
  const int r = c.rank;
  const int ngroups = c.nwires / N;
  const int g = wire / N;
  const int y = wire % N;
  if (g >= ngroups) return;
  const Partition p = make_partition(c.nelems, N);
  const int64_t steps = ceil_div64(p.chunk_dw, int64_t(ngroups) * B::kPayloadDw);
  const int64_t base = int64_t(y) * p.chunk_dw;
  const int64_t end = min64(base + p.chunk_dw, p.total_dw);

  for (int64_t t = 0; t < steps; ++t) {
    const uint32_t flag = c.seq + uint32_t(t / kParallelSlots);
    const int slot = int(t % kParallelSlots);
    const int64_t dw = base + (t * ngroups + g) * B::kPayloadDw;
    typename B::Msg v;
    B::load(v, c.in, dw, end, p.odd_dw);
    B::shuffle(v);
    if (y != r) {
      B::set_flags(v, flag);
      c.send(txn_at<B>(c.peer_sink(0, y), (int64_t(g) * N + r) * kParallelSlots + slot), v);
      B200_WAIT(c, v, txn_at<B>(c.sink(1), (int64_t(g) * N + y) * kParallelSlots + slot), flag, 1, y, t);
    } else {
      typename B::Acc a;
      B::acc_init(a, v);
      if (!recv_in_order<B, 1, N>(
              c, flag, 0, t, -1, v,
              [&](int i) -> const char* { return txn_at<B>(c.sink(0), (int64_t(g) * N + (r + i) % N) * kParallelSlots + slot); },
              [&](int i) { return (r + i) % N; },
              [&](int, const typename B::Msg& x) { B::acc_add(a, x, c.round_each()); }))
        return;
      B::acc_to_msg(v, a);
      B::set_flags(v, flag);
#pragma unroll
      for (int i = 1; i < N; ++i) {
        const int q = (r + i) % N;
        c.send(txn_at<B>(c.peer_sink(1, q), (int64_t(g) * N + r) * kParallelSlots + slot), v);
      }
    }
    B::restore(v);
    B::store(c.out, dw, end, p.odd_dw, v);
  }
}

// ---------------------------------------------------------------------------
// Reduce-scatter: the first phase of the parallel schedule on its own.  nelems
// counts the whole input (a multiple of 8 * world elements); rank r's output is
// the r-th of `world` equal slices, reduced.  A sender gets no reply here, so two
// things replace the request/response coupling of the all-reduce: a launch never
// takes more steps than a ring has slots (the host sees to it), and consecutive
// launches use different halves of the ring (picked by bit 1 of the sequence
// number, which advances by 2 per launch) - a rank cannot be more than one
// launch ahead of a peer, because as an owner it needs every peer's slices of
// the current launch to finish it.
// ---------------------------------------------------------------------------
B200_HD int64_t reduce_scatter_steps(uint64_t nelems, int world, int nwires, int payload_dw) {
  return ceil_div64(int64_t(nelems / uint64_t(world) / 2), int64_t(nwires / world) * payload_dw);
}

template <class B, int N>
B200_HD void run_reduce_scatter(const Ctx<B>& c, int wire) {
  const int r = c.rank;
  const int ngroups = c.nwires / N;
  const int g = wire / N;
  const int y = wire % N;
  if (g >= ngroups) return;
  const int64_t chunk_dw = int64_t(c.nelems / uint64_t(N) / 2);
  const int64_t steps = ceil_div64(chunk_dw, int64_t(ngroups) * B::kPayloadDw);
  const int64_t ring0 = int64_t((c.seq >> 1) & 1u) * c.nwires * kParallelSlots;  // this launch's half, in transactions
  const uint32_t flag = c.seq;
  for (int64_t t = 0; t < steps; ++t) {
    const int slot = int(t);
    const int64_t dw = (t * ngroups + g) * B::kPayloadDw;  // inside the chunk
    typename B::Msg v;
    B::load(v, c.in, int64_t(y) * chunk_dw + dw, int64_t(y + 1) * chunk_dw, -1);
    B::shuffle(v);
    if (y != r) {
      B::set_flags(v, flag);
      c.send(txn_at<B>(c.peer_sink(0, y), ring0 + (int64_t(g) * N + r) * kParallelSlots + slot), v);
    } else {
      typename B::Acc a;
      B::acc_init(a, v);
      if (!recv_in_order<B, 1, N>(
              c, flag, 0, t, -1, v,
              [&](int i) -> const char* { return txn_at<B>(c.sink(0), ring0 + (int64_t(g) * N + (r + i) % N) * kParallelSlots + slot); },
              [&](int i) { return (r + i) % N; },
              [&](int, const typename B::Msg& x) { B::acc_add(a, x, c.round_each()); }))
        return;
      B::acc_to_msg(v, a);
      B::restore(v);
      B::store(c.out, dw, chunk_dw, -1, v);
    }
  }
}

// ---------------------------------------------------------------------------
// Sequential all-reduce: one wire does the whole exchange for its offset, for
// all peers.  Needs no progress guarantee between warps of a rank.
// ---------------------------------------------------------------------------
template <class B, int N>
B200_HD void run_sequential(const Ctx<B>& c, int wire) {
  const int r = c.rank;
  const int nw = c.nwires;
  if (wire >= nw) return;
  const Partition p = make_partition(c.nelems, N);
  const int64_t steps = ceil_div64(p.chunk_dw, int64_t(nw) * B::kPayloadDw);

  for (int64_t t = 0; t < steps; ++t) {
    const uint32_t flag = c.seq + uint32_t(t / kSequentialSlots);
    const int slot = int(t % kSequentialSlots);
    const int64_t off = (t * nw + wire) * B::kPayloadDw;
    auto idx = [&](int src) { return (int64_t(src) * kSequentialSlots + slot) * nw + wire; };
    auto chunk_end = [&](int y) { return min64(int64_t(y + 1) * p.chunk_dw, p.total_dw); };

#pragma unroll
    for (int i = 1; i < N; ++i) {
      const int q = (r + i) % N;
      typename B::Msg m;
      B::load(m, c.in, int64_t(q) * p.chunk_dw + off, chunk_end(q), p.odd_dw);
      B::shuffle(m);
      B::set_flags(m, flag);
      c.send(txn_at<B>(c.peer_sink(0, q), idx(r)), m);
    }
    typename B::Msg v;
    B::load(v, c.in, int64_t(r) * p.chunk_dw + off, chunk_end(r), p.odd_dw);
    B::shuffle(v);
    typename B::Acc a;
    B::acc_init(a, v);
    // (this schedule polls its peers one after the other: with world - 1 outgoing and as many
    // incoming transactions per step already in registers there is no room to overlap the polls)
#pragma unroll
    for (int i = 1; i < N; ++i) {
      const int q = (r + i) % N;
      typename B::Msg m;
      B200_WAIT(c, m, txn_at<B>(c.sink(0), idx(q)), flag, 0, q, t);
      B::acc_add(a, m, c.round_each());
    }
    B::acc_to_msg(v, a);
    B::set_flags(v, flag);
#pragma unroll
    for (int i = 1; i < N; ++i) {
      const int q = (r + i) % N;
      c.send(txn_at<B>(c.peer_sink(1, q), idx(r)), v);
    }
    B::restore(v);
    B::store(c.out, int64_t(r) * p.chunk_dw + off, chunk_end(r), p.odd_dw, v);
#pragma unroll
    for (int i = 1; i < N; ++i) {
      const int q = (r + i) % N;
      typename B::Msg m;
      B200_WAIT(c, m, txn_at<B>(c.sink(1), idx(q)), flag, 1, q, t);
      B::restore(m);
      B::store(c.out, int64_t(q) * p.chunk_dw + off, chunk_end(q), p.odd_dw, m);
    }
  }
}

// ---------------------------------------------------------------------------
// Ring all-reduce: reduce-scatter around the ring through half 0, then
// all-gather around the ring through half 1.  Only `next` is ever written.
// Chunk arithmetic is signed, so any world size works (the reference's
// unsigned modulo is right for powers of two only, sequential_transmit.hpp:451).
// ---------------------------------------------------------------------------
template <class B, int N>
B200_HD void run_ring_allreduce(const Ctx<B>& c, int wire) {
  const int r = c.rank;
  const int nw = c.nwires;
  if (wire >= nw) return;
  const int next = (r + 1) % N;
  const int prev = (r + N - 1) % N;
  const Partition p = make_partition(c.nelems, N);
  const int64_t steps = ceil_div64(p.chunk_dw, int64_t(nw) * B::kPayloadDw);

  for (int64_t t = 0; t < steps; ++t) {
    const uint32_t flag = c.seq + uint32_t(t / kRingSlots);
    const int slot = int(t % kRingSlots);
    const int64_t off = (t * nw + wire) * B::kPayloadDw;
    auto idx = [&](int chunk) { return (int64_t(chunk) * kRingSlots + slot) * nw + wire; };
    auto chunk_end = [&](int y) { return min64(int64_t(y + 1) * p.chunk_dw, p.total_dw); };

    typename B::Msg v;
    {
      const int ch = r;
      B::load(v, c.in, int64_t(ch) * p.chunk_dw + off, chunk_end(ch), p.odd_dw);
      B::shuffle(v);
      B::set_flags(v, flag);
      c.send(txn_at<B>(c.peer_sink(0, next), idx(ch)), v);
    }
#pragma unroll
    for (int i = 1; i < N; ++i) {
      const int ch = (r - i + N) % N;
      typename B::Msg m;
      B::load(v, c.in, int64_t(ch) * p.chunk_dw + off, chunk_end(ch), p.odd_dw);
      B::shuffle(v);
      typename B::Acc a;
      B::acc_init(a, v);
      B200_WAIT(c, m, txn_at<B>(c.sink(0), idx(ch)), flag, 0, prev, t);
      B::acc_add(a, m, c.round_each());
      B::acc_to_msg(v, a);
      B::set_flags(v, flag);
      if (i < N - 1) {
        c.send(txn_at<B>(c.peer_sink(0, next), idx(ch)), v);
      } else {
        // chunk (r+1)%N is now complete on this rank: start the all-gather.
        c.send(txn_at<B>(c.peer_sink(1, next), idx(ch)), v);
        B::restore(v);
        B::store(c.out, int64_t(ch) * p.chunk_dw + off, chunk_end(ch), p.odd_dw, v);
      }
    }
#pragma unroll
    for (int j = 1; j < N; ++j) {
      const int ch = (r + 1 - j + N) % N;
      typename B::Msg m;
      B200_WAIT(c, m, txn_at<B>(c.sink(1), idx(ch)), flag, 1, prev, t);
      if (j < N - 1) c.send(txn_at<B>(c.peer_sink(1, next), idx(ch)), m);
      B::restore(m);
      B::store(c.out, int64_t(ch) * p.chunk_dw + off, chunk_end(ch), p.odd_dw, m);
    }
  }
}

// ---------------------------------------------------------------------------
// Ring all-gather: nelems per rank in, world * nelems out (rank order).
// nelems must be even so that every shard starts on a dword.
// ---------------------------------------------------------------------------
template <class B, int N>
B200_HD void run_ring_allgather(const Ctx<B>& c, int wire) {
  const int r = c.rank;
  const int nw = c.nwires;
  if (wire >= nw) return;
  const int next = (r + 1) % N;
  const int prev = (r + N - 1) % N;
  const int64_t shard_dw = int64_t(c.nelems / 2);
  const int64_t steps = allgather_steps(c.nelems, nw, B::kPayloadDw);
  const bool in_place = (c.flags & kInPlace) != 0;

  for (int64_t t = 0; t < steps; ++t) {
    const uint32_t flag = c.seq + uint32_t(t / kRingSlots);
    const int slot = int(t % kRingSlots);
    const int64_t off = (t * nw + wire) * B::kPayloadDw;
    auto idx = [&](int chunk) { return (int64_t(chunk) * kRingSlots + slot) * nw + wire; };

    typename B::Msg v;
    if (in_place) {
      B::load(v, c.out, int64_t(r) * shard_dw + off, int64_t(r + 1) * shard_dw, -1);
    } else {
      B::load(v, c.in, off, shard_dw, -1);
      B::store(c.out, int64_t(r) * shard_dw + off, int64_t(r + 1) * shard_dw, -1, v);
    }
    B::shuffle(v);
    B::set_flags(v, flag);
    c.send(txn_at<B>(c.peer_sink(1, next), idx(r)), v);
#pragma unroll
    for (int j = 1; j < N; ++j) {
      const int ch = (r - j + N) % N;
      typename B::Msg m;
      B200_WAIT(c, m, txn_at<B>(c.sink(1), idx(ch)), flag, 1, prev, t);
      if (j < N - 1) c.send(txn_at<B>(c.peer_sink(1, next), idx(ch)), m);
      B::restore(m);
      B::store(c.out, int64_t(ch) * shard_dw + off, int64_t(ch + 1) * shard_dw, -1, m);
    }
  }
}

// ---------------------------------------------------------------------------
// Direct all-gather: every wire pushes its piece of the shard to all peers and
// then collects the world-1 pieces that land locally.  One hop.
// ---------------------------------------------------------------------------
template <class B, int N>
B200_HD void run_direct_allgather(const Ctx<B>& c, int wire) {
  const int r = c.rank;
  const int nw = c.nwires;
  if (wire >= nw) return;
  const int64_t shard_dw = int64_t(c.nelems / 2);
  const int64_t steps = allgather_steps(c.nelems, nw, B::kPayloadDw);
  const bool in_place = (c.flags & kInPlace) != 0;

  for (int64_t t = 0; t < steps; ++t) {
    const uint32_t flag = c.seq + uint32_t(t / kSequentialSlots);
    const int slot = int(t % kSequentialSlots);
    const int64_t off = (t * nw + wire) * B::kPayloadDw;
    auto idx = [&](int src) { return (int64_t(src) * kSequentialSlots + slot) * nw + wire; };

    typename B::Msg v;
    if (in_place) {
      B::load(v, c.out, int64_t(r) * shard_dw + off, int64_t(r + 1) * shard_dw, -1);
    } else {
      B::load(v, c.in, off, shard_dw, -1);
      B::store(c.out, int64_t(r) * shard_dw + off, int64_t(r + 1) * shard_dw, -1, v);
    }
    B::shuffle(v);
    B::set_flags(v, flag);
#pragma unroll
    for (int i = 1; i < N; ++i) {
      const int q = (r + i) % N;
      c.send(txn_at<B>(c.peer_sink(1, q), idx(r)), v);
    }
    if (!recv_in_order<B, 1, N>(
            c, flag, 1, t, -1, v, [&](int i) -> const char* { return txn_at<B>(c.sink(1), idx((r + i) % N)); },
            [&](int i) { return (r + i) % N; },
            [&](int i, const typename B::Msg& x) {
              const int q = (r + i) % N;
              typename B::Msg y = x;
              B::restore(y);
              B::store(c.out, int64_t(q) * shard_dw + off, int64_t(q + 1) * shard_dw, -1, y);
            }))
      return;
  }
}

// ---------------------------------------------------------------------------
// Bisect (two-level) all-reduce.  Rank r and r^1 are partners; ranks of equal
// parity form a group of N/2.  The buffer is cut in two halves; a rank's
// "close" half is the one with its own parity.  (1) push my far half to the
// partner, (2) add the partner's contribution to my close half and run the
// parallel two-phase exchange inside my parity group, push the result to the
// partner, (3) collect the partner's result for my far half.  Every group link
// carries half of the data.
// ---------------------------------------------------------------------------
template <class B, int N>
B200_HD void run_bisect(const Ctx<B>& c, int wire) {
  constexpr int BI = N / 2;
  const int r = c.rank;
  const int partner = r ^ 1;
  const int parity = r & 1;
  const int l = r / 2;
  const int ngroups = c.nwires / BI;
  const int g = wire / BI;
  const int y = wire % BI;
  if (g >= ngroups) return;
  const Partition h = make_partition(c.nelems, 2);
  const int64_t chunk_dw = round_up64(ceil_div64(h.chunk_dw, BI), 4);
  const int64_t steps = ceil_div64(chunk_dw, int64_t(ngroups) * B::kPayloadDw);
  const int64_t close0 = int64_t(parity) * h.chunk_dw;
  const int64_t far0 = int64_t(1 - parity) * h.chunk_dw;
  const int64_t close_end = min64(min64(close0 + h.chunk_dw, h.total_dw), close0 + int64_t(y + 1) * chunk_dw);
  const int64_t far_end = min64(min64(far0 + h.chunk_dw, h.total_dw), far0 + int64_t(y + 1) * chunk_dw);

  for (int64_t t = 0; t < steps; ++t) {
    const uint32_t flag = c.seq + uint32_t(t / kParallelSlots);
    const int slot = int(t % kParallelSlots);
    const int64_t off = int64_t(y) * chunk_dw + (t * ngroups + g) * B::kPayloadDw;
    const int64_t far_idx = kBisectFarBase + int64_t(wire) * kParallelSlots + slot;

    typename B::Msg v;
    // (1) far half to the partner
    B::load(v, c.in, far0 + off, far_end, h.odd_dw);
    B::shuffle(v);
    B::set_flags(v, flag);
    c.send(txn_at<B>(c.peer_sink(0, partner), far_idx), v);

    // (2) close half: add the partner's copy, then reduce inside the parity group
    B::load(v, c.in, close0 + off, close_end, h.odd_dw);
    B::shuffle(v);
    typename B::Acc a;
    B::acc_init(a, v);
    {
      typename B::Msg m;
      B200_WAIT(c, m, txn_at<B>(c.sink(0), far_idx), flag, 2, partner, t);
      B::acc_add(a, m, c.round_each());
    }
    if (y != l) {
      B::acc_to_msg(v, a);
      B::set_flags(v, flag);
      c.send(txn_at<B>(c.peer_sink(0, 2 * y + parity), (int64_t(g) * BI + l) * kParallelSlots + slot), v);
      B200_WAIT(c, v, txn_at<B>(c.sink(1), (int64_t(g) * BI + y) * kParallelSlots + slot), flag, 1,
                2 * y + parity, t);
    } else {
      if (!recv_in_order<B, 1, BI>(
              c, flag, 0, t, -1, v,
              [&](int i) -> const char* {
                return txn_at<B>(c.sink(0), (int64_t(g) * BI + (l + i) % BI) * kParallelSlots + slot);
              },
              [&](int i) { return 2 * ((l + i) % BI) + parity; },
              [&](int, const typename B::Msg& x) { B::acc_add(a, x, c.round_each()); }))
        return;
      B::acc_to_msg(v, a);
      B::set_flags(v, flag);
#pragma unroll
      for (int i = 1; i < BI; ++i) {
        const int ql = (l + i) % BI;
        c.send(txn_at<B>(c.peer_sink(1, 2 * ql + parity), (int64_t(g) * BI + l) * kParallelSlots + slot), v);
      }
    }
    // v (wire order, flags set) is the fully reduced slice of my close half.
    c.send(txn_at<B>(c.peer_sink(1, partner), far_idx), v);
    B::restore(v);
    B::store(c.out, close0 + off, close_end, h.odd_dw, v);

    // (3) the partner's result is my far half
    B200_WAIT(c, v, txn_at<B>(c.sink(1), far_idx), flag, 3, partner, t);
    B::restore(v);
    B::store(c.out, far0 + off, far_end, h.odd_dw, v);
  }
}

// ---------------------------------------------------------------------------
// One-shot all-reduce for tiny messages: every wire pushes its slice of the
// whole buffer to every peer, then adds the world slices in rank order (so all
// ranks compute the same bits).  flag = seq + t, slot = flag % 4: consecutive
// steps and consecutive launches never share a landing slot.
// ---------------------------------------------------------------------------
template <class B, int N>
B200_HD void run_oneshot(const Ctx<B>& c, int wire) {
  const int r = c.rank;
  const int nw = c.nwires;
  if (wire >= nw) return;
  const int64_t total_dw = int64_t((c.nelems + 1) / 2);
  const int64_t odd_dw = (c.nelems & 1) ? total_dw - 1 : -1;
  const int64_t steps = oneshot_steps(c.nelems, nw, B::kPayloadDw);

  for (int64_t t = 0; t < steps; ++t) {
    const uint32_t flag = c.seq + uint32_t(t);
    const int slot = int(flag % kOneShotSlots);
    const int64_t dw = (t * nw + wire) * B::kPayloadDw;
    auto at = [&](char* base, int src) {
      return base + ((int64_t(src) * kMaxOneShotWires + wire) * kOneShotSlots + slot) * kOneShotStride;
    };
    typename B::Msg v;
    B::load(v, c.in, dw, total_dw, odd_dw);
    B::shuffle(v);
    B::set_flags(v, flag);
#pragma unroll
    for (int i = 1; i < N; ++i) {
      const int q = (r + i) % N;
      c.send(at(c.peer_oneshot(q), r), v);
    }
    // the world - 1 landing slots are polled in overlapping groups; slices are added in rank order,
    // the own one (its flag dwords differ from a received copy, but no accumulator slot reads them) at r
    typename B::Acc a;
    if (!recv_in_order<B, 0, N>(
            c, flag, 4, t, r, v, [&](int q) -> const char* { return at(c.oneshot(), q); }, [&](int q) { return q; },
            [&](int q, const typename B::Msg& x) {
              if (q == 0) B::acc_init(a, x);
              else B::acc_add(a, x, c.round_each());
            }))
      return;
    B::acc_to_msg(v, a);
    B::restore(v);
    B::store(c.out, dw, total_dw, odd_dw, v);
  }
}

}  // namespace b200ipc
