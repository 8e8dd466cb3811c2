// CPU backend of the wire formats for the schedules in coll/schedules.h: a whole
// warp transaction is one array of dwords already in wire order.  Used by the
// emulator (plumbing tests without a GPU, fault injection on the host) and as the
// oracle for the byte image a GPU rank leaves in its peers' scratch.
//
// The hardware property the protocols rely on - payload and flag of one atomic
// unit become visible together - is modelled by writing the payload first and the
// flags last with release ordering, and reading the flags first with acquire
// ordering.
#pragma once

#include <atomic>
#include <chrono>
#include <cstring>
#include <thread>

#include "../common/half_host.h"
#include "../common/types.h"
#include "../proto/wire_format.h"

namespace b200ipc {

struct HostWaiter {
  std::atomic<uint32_t>* abort_word = nullptr;              // in my heap
  std::atomic<uint32_t>* peer_abort[kMaxRanks] = {nullptr};  // the same word on every rank
  StatusBlock* status = nullptr;
  uint64_t timeout_ns = 2000000000ull;
  int world = 1;
  int wire = 0;
  void trace(int, int, int64_t, uint32_t) const {}  // the emulator has a debugger instead
};

template <ProtoKind K, DType T>
struct HostBackend : WireFormat<K> {
  using WF = WireFormat<K>;
  static constexpr int kPayloadDw = WF::kPayloadDw;
  static constexpr int kTxnDw = WF::kTxnDw;
  static constexpr int kTxnBytes = WF::kTxnDw * 4;
  using Waiter = HostWaiter;

  struct Msg { uint32_t slot[kTxnDw]; };
  struct Acc { float f[2 * kPayloadDw]; };

  static void load(Msg& v, const uint32_t* buf, int64_t dw, int64_t end_dw, int64_t odd_dw) {
    std::memset(v.slot, 0, sizeof(v.slot));
    for (int k = 0; k < kPayloadDw; ++k) {
      const int64_t i = dw + k;
      uint32_t x = 0;
      if (i < end_dw) x = (i == odd_dw) ? uint32_t(reinterpret_cast<const uint16_t*>(buf)[2 * i]) : buf[i];
      v.slot[WF::payload_slot(k)] = x;
    }
  }
  static void store(uint32_t* buf, int64_t dw, int64_t end_dw, int64_t odd_dw, const Msg& v) {
    for (int k = 0; k < kPayloadDw; ++k) {
      const int64_t i = dw + k;
      if (i >= end_dw) continue;
      const uint32_t x = v.slot[WF::payload_slot(k)];
      if (i == odd_dw) reinterpret_cast<uint16_t*>(buf)[2 * i] = uint16_t(x & 0xffffu);
      else buf[i] = x;
    }
  }
  static void shuffle(Msg&) {}  // load() already places payload in wire order
  static void restore(Msg&) {}
  static void set_flags(Msg& v, uint32_t flag) {
    for (int s = 0; s < kTxnDw; ++s)
      if (WF::is_flag_slot(s)) v.slot[s] = flag;
  }
  static void send(char* dst, const Msg& v) {
    auto* d = reinterpret_cast<std::atomic<uint32_t>*>(dst);
    for (int s = 0; s < kTxnDw; ++s)
      if (!WF::is_flag_slot(s)) d[s].store(v.slot[s], std::memory_order_relaxed);
    std::atomic_thread_fence(std::memory_order_release);
    for (int s = 0; s < kTxnDw; ++s)
      if (WF::is_flag_slot(s)) d[s].store(v.slot[s], std::memory_order_release);
  }
  static bool try_recv(Msg& v, const char* src, uint32_t flag) {
    auto* s = reinterpret_cast<const std::atomic<uint32_t>*>(src);
    for (int i = 0; i < kTxnDw; ++i)
      if (WF::is_flag_slot(i) && s[i].load(std::memory_order_acquire) != flag) return false;
    std::atomic_thread_fence(std::memory_order_acquire);
    for (int i = 0; i < kTxnDw; ++i) v.slot[i] = s[i].load(std::memory_order_relaxed);
    return true;
  }
  static bool wait(const HostWaiter& w, Msg& v, const char* src, uint32_t flag, int site, int peer, int64_t step,
                   int rank) {
    using Clock = std::chrono::steady_clock;
    const auto t0 = Clock::now();
    uint32_t spins = 0;
    for (;;) {
      if (try_recv(v, src, flag)) return true;
      if ((++spins & 0x3f) == 0) {
        if (w.abort_word->load(std::memory_order_acquire) != 0) return false;
        const uint64_t ns = uint64_t(std::chrono::duration_cast<std::chrono::nanoseconds>(Clock::now() - t0).count());
        if (ns > w.timeout_ns) {
          uint32_t expected = 0;
          if (w.abort_word->compare_exchange_strong(expected, 1u)) {
            StatusBlock* s = w.status;
            s->rank = uint32_t(rank);
            s->peer = uint32_t(peer);
            s->wire = uint32_t(w.wire);
            s->step = uint32_t(step);
            s->expected = flag;
            s->seen = reinterpret_cast<const std::atomic<uint32_t>*>(src)[kTxnDw - 1].load();
            s->where = uint32_t(site);
            s->code = kTimeout;
          }
          for (int q = 0; q < w.world; ++q)
            if (q != rank && w.peer_abort[q]) w.peer_abort[q]->store(1u, std::memory_order_release);
          return false;
        }
        std::this_thread::yield();
      }
    }
  }

  // Several transactions at once (see DevBackend::wait_many); a scalar rank has nothing to overlap.
  template <int CNT, class SrcFn, class PeerFn>
  static bool wait_many(const HostWaiter& w, Msg (&m)[CNT], SrcFn src, PeerFn peer, uint32_t pending, uint32_t flag, int site,
                        int64_t step, int rank) {
    for (int i = 0; i < CNT; ++i)
      if ((pending & (1u << i)) && !wait(w, m[i], src(i), flag, site, peer(i), step, rank)) return false;
    return true;
  }

  static void acc_init(Acc& a, const Msg& v) {
    for (int k = 0; k < kPayloadDw; ++k) {
      const uint32_t x = v.slot[WF::payload_slot(k)];
      a.f[2 * k] = to_float(T, uint16_t(x & 0xffffu));
      a.f[2 * k + 1] = to_float(T, uint16_t(x >> 16));
    }
  }
  static void acc_add(Acc& a, const Msg& v, bool round_each) {
    for (int k = 0; k < kPayloadDw; ++k) {
      const uint32_t x = v.slot[WF::payload_slot(k)];
      a.f[2 * k] += to_float(T, uint16_t(x & 0xffffu));
      a.f[2 * k + 1] += to_float(T, uint16_t(x >> 16));
      if (round_each) {
        a.f[2 * k] = to_float(T, from_float(T, a.f[2 * k]));
        a.f[2 * k + 1] = to_float(T, from_float(T, a.f[2 * k + 1]));
      }
    }
  }
  static void acc_to_msg(Msg& v, const Acc& a) {
    for (int k = 0; k < kPayloadDw; ++k)
      v.slot[WF::payload_slot(k)] = uint32_t(from_float(T, a.f[2 * k])) | (uint32_t(from_float(T, a.f[2 * k + 1])) << 16);
  }
};

}  // namespace b200ipc
