// Device (sm_100a) backend of the wire formats: one warp = one wire, lane l
// holds dwords [l*kLaneDw, (l+1)*kLaneDw) of the transaction in registers.
//
// Remote stores and local polls use .volatile vector accesses (L1 bypass; a
// lane's 8 B or 16 B store reaches the peer as one unit, a warp's coalesced
// store as full 64 B / 128 B segments).  Partial sums are kept in fp32
// registers; kRoundEachAdd rounds to T after every add to mimic summation in T
// (the reference adds in half/bf16, rt64_128.hpp:950-966).
//
// Bounded waits: a spin checks the abort word and the global timer every 256
// polls; the first wire that runs out of time records where it was, raises
// the abort word on every rank it can reach and returns, so a missing peer
// ends the kernel with a status instead of hanging the GPU.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../common/types.h"
#include "wire_format.h"

namespace b200ipc {

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_u32(void* p, uint32_t v) {
  asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void ld_volatile_v2(const void* p, uint32_t& a, uint32_t& b) {
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(a), "=r"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ void st_volatile_v2(void* p, uint32_t a, uint32_t b) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void ld_volatile_v4(const void* p, uint32_t (&d)[4]) {
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "l"(p)
               : "memory");
}
__device__ __forceinline__ void st_volatile_v4(void* p, const uint32_t (&d)[4]) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(d[0]), "r"(d[1]), "r"(d[2]),
               "r"(d[3])
               : "memory");
}

// One wire per rank writes the rank's status record (pinned host memory): the first that has
// something to report claims it, either as "my wait ran out" (kTimeout) or as "I was told to
// stop" (kAbortedByPeer).  With a single writer a record is never half one and half the other,
// and the host's check raises on every rank of an aborted collective, not only on the one whose
// wait ran out.  `abort_word` is the rank's own abort word; the claim word sits next to it.
__device__ __forceinline__ bool claim_status(uint32_t* abort_word, uint32_t kind) {
  return atomicCAS(abort_word + (kCtrlClaimOff - kCtrlAbortOff) / 4, 0u, kind) == 0u;
}
__device__ __forceinline__ void note_aborted_by_peer(uint32_t* abort_word, StatusBlock* s, int rank, int site) {
  if (!claim_status(abort_word, kAbortedByPeer)) return;
  s->rank = uint32_t(rank);
  s->where = uint32_t(site);
  __threadfence_system();
  s->code = kAbortedByPeer;
  __threadfence_system();
}

struct DevWaiter {
  const RankView* me;  // kernel parameter space
  size_t ctrl_off;
  int wire;
  // One record into the rank's trace ring (lane 0 of the calling warp); the device analogue of the
  // reference's verbose build, which printf's every wire's offsets and message words
  // (allreduce.hpp:96-101, sequential_transmit.hpp:118-124, 305-331).
  __device__ void trace(int site, int peer, int64_t step, uint32_t flag) const {
    if ((threadIdx.x & 31) != 0) return;
    char* base = me->heap + ctrl_off + kCtrlTraceOff;
    const uint32_t idx = atomicAdd(reinterpret_cast<uint32_t*>(base), 1u) % kTraceEntries;
    TraceRecord* r = reinterpret_cast<TraceRecord*>(base + 16) + idx;
    r->t_ns = globaltimer_ns();
    r->wire = uint32_t(wire);
    r->site = uint32_t(site);
    r->peer = uint32_t(peer);
    r->step = uint32_t(step);
    r->flag = flag;
    r->rank = uint32_t(me->rank);
  }
  __device__ uint32_t* abort_word() const {
    return reinterpret_cast<uint32_t*>(me->heap + ctrl_off + kCtrlAbortOff);
  }
  __device__ uint32_t* peer_abort(int r) const {
    return reinterpret_cast<uint32_t*>(me->peer[r] + ctrl_off + kCtrlAbortOff);
  }
};

template <typename T>
struct Cvt;
template <>
struct Cvt<__half> {
  __device__ static float2 up(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
  __device__ static uint32_t down(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <>
struct Cvt<__nv_bfloat16> {
  __device__ static float2 up(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
  __device__ static uint32_t down(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

__device__ __forceinline__ uint32_t ld_dw_guarded(const uint32_t* buf, int64_t i, int64_t end_dw,
                                                  int64_t odd_dw) {
  if (i >= end_dw) return 0u;
  if (i == odd_dw) return uint32_t(reinterpret_cast<const uint16_t*>(buf)[2 * i]);
  return buf[i];
}
__device__ __forceinline__ void st_dw_guarded(uint32_t* buf, int64_t i, int64_t end_dw, int64_t odd_dw,
                                              uint32_t v) {
  if (i >= end_dw) return;
  if (i == odd_dw) {
    reinterpret_cast<uint16_t*>(buf)[2 * i] = uint16_t(v & 0xffffu);
    return;
  }
  buf[i] = v;
}

template <ProtoKind K, typename T>
struct DevBackend : WireFormat<K> {
  using WF = WireFormat<K>;
  static constexpr int kLaneDw = WF::kLaneDw;
  static constexpr int kPayloadDw = WF::kPayloadDw;
  static constexpr int kTxnBytes = WF::kTxnDw * 4;
  // Payload-bearing register slots of a lane (flags excluded where the slot is
  // a flag on every lane).
  static constexpr int kAccDw = (K == ProtoKind::LL8) ? 1 : (K == ProtoKind::LL16) ? 2 : (K == ProtoKind::LL128) ? 1 : 4;
  using Waiter = DevWaiter;

  struct Msg { uint32_t d[kLaneDw]; };
  struct Acc { float f[2 * kAccDw]; };

  __device__ static constexpr int acc_slot(int j) {
    return (K == ProtoKind::LL16) ? 2 * j : j;
  }
  __device__ static int lane() { return int(threadIdx.x & 31); }

  // ---- local memory <-> registers (payload order) ---------------------------
  __device__ static void load(Msg& v, const uint32_t* buf, int64_t dw, int64_t end_dw, int64_t odd_dw) {
    const int l = lane();
    if constexpr (K == ProtoKind::LL8) {
      v.d[0] = ld_dw_guarded(buf, dw + l, end_dw, odd_dw);
      v.d[1] = 0;
    } else if constexpr (K == ProtoKind::LL16) {
      const int64_t i = dw + 2 * l;
      if (i + 2 <= end_dw && i + 1 != odd_dw && ((reinterpret_cast<uintptr_t>(buf + i) & 7) == 0)) {
        uint2 x = *reinterpret_cast<const uint2*>(buf + i);
        v.d[0] = x.x;
        v.d[2] = x.y;
      } else {
        v.d[0] = ld_dw_guarded(buf, i, end_dw, odd_dw);
        v.d[2] = ld_dw_guarded(buf, i + 1, end_dw, odd_dw);
      }
      v.d[1] = 0;
      v.d[3] = 0;
    } else if constexpr (K == ProtoKind::LL128) {
      v.d[0] = (l < 30) ? ld_dw_guarded(buf, dw + l, end_dw, odd_dw) : 0u;
    } else {
      const int64_t i = dw + 4 * l;
      if (l >= 30) {
        v.d[0] = v.d[1] = v.d[2] = v.d[3] = 0;
      } else if (i + 4 <= end_dw && i + 3 != odd_dw && ((reinterpret_cast<uintptr_t>(buf + i) & 15) == 0)) {
        uint4 x = *reinterpret_cast<const uint4*>(buf + i);
        v.d[0] = x.x; v.d[1] = x.y; v.d[2] = x.z; v.d[3] = x.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) v.d[e] = ld_dw_guarded(buf, i + e, end_dw, odd_dw);
      }
    }
  }

  __device__ static void store(uint32_t* buf, int64_t dw, int64_t end_dw, int64_t odd_dw, const Msg& v) {
    const int l = lane();
    if constexpr (K == ProtoKind::LL8) {
      st_dw_guarded(buf, dw + l, end_dw, odd_dw, v.d[0]);
    } else if constexpr (K == ProtoKind::LL16) {
      const int64_t i = dw + 2 * l;
      if (i + 2 <= end_dw && i + 1 != odd_dw && ((reinterpret_cast<uintptr_t>(buf + i) & 7) == 0)) {
        *reinterpret_cast<uint2*>(buf + i) = make_uint2(v.d[0], v.d[2]);
      } else {
        st_dw_guarded(buf, i, end_dw, odd_dw, v.d[0]);
        st_dw_guarded(buf, i + 1, end_dw, odd_dw, v.d[2]);
      }
    } else if constexpr (K == ProtoKind::LL128) {
      if (l < 30) st_dw_guarded(buf, dw + l, end_dw, odd_dw, v.d[0]);
    } else {
      const int64_t i = dw + 4 * l;
      if (l >= 30) return;
      if (i + 4 <= end_dw && i + 3 != odd_dw && ((reinterpret_cast<uintptr_t>(buf + i) & 15) == 0)) {
        *reinterpret_cast<uint4*>(buf + i) = make_uint4(v.d[0], v.d[1], v.d[2], v.d[3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) st_dw_guarded(buf, i + e, end_dw, odd_dw, v.d[e]);
      }
    }
  }

  // ---- payload order <-> wire order ------------------------------------------
  __device__ static void shuffle(Msg& v) {
    const int l = lane();
    if constexpr (K == ProtoKind::LL128) {
      // the dword that belongs at slot 15 travels in slot 30
      uint32_t x = __shfl_sync(0xffffffffu, v.d[0], 15);
      if (l == 30) v.d[0] = x;
    } else if constexpr (K == ProtoKind::LL512) {
      // element 3 of lanes 3,7,..,27 (slots 15,31,..,111) moves to slots 120..126
      const int hi = (l == 31) ? 4 : 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        uint32_t x = __shfl_sync(0xffffffffu, v.d[3], 4 * (e + hi) + 3);
        if (l >= 30) v.d[e] = x;
      }
    }
  }
  __device__ static void restore(Msg& v) {
    const int l = lane();
    if constexpr (K == ProtoKind::LL128) {
      uint32_t x = __shfl_sync(0xffffffffu, v.d[0], 30);
      if (l == 15) v.d[0] = x;
    } else if constexpr (K == ProtoKind::LL512) {
      const int j = l >> 2;  // which displaced dword belongs to this lane (if l % 4 == 3)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        uint32_t x = __shfl_sync(0xffffffffu, v.d[e], 30 + (j >> 2));
        if ((l & 3) == 3 && (j & 3) == e) v.d[3] = x;
      }
    }
  }
  __device__ static void set_flags(Msg& v, uint32_t flag) {
    const int l = lane();
    if constexpr (K == ProtoKind::LL8) {
      v.d[1] = flag;
    } else if constexpr (K == ProtoKind::LL16) {
      v.d[1] = flag;
      v.d[3] = flag;
    } else if constexpr (K == ProtoKind::LL128) {
      if (l == 15 || l == 31) v.d[0] = flag;
    } else {
      if ((l & 3) == 3) v.d[3] = flag;
    }
  }

  // ---- the wire ---------------------------------------------------------------
  __device__ static void send(char* dst, const Msg& v) {
    char* p = dst + lane() * (kLaneDw * 4);
    if constexpr (kLaneDw == 1) {
      st_volatile_u32(p, v.d[0]);
    } else if constexpr (kLaneDw == 2) {
      st_volatile_v2(p, v.d[0], v.d[1]);
    } else {
      st_volatile_v4(p, v.d);
    }
  }
  // The receive side in two halves, so that a wire expecting several transactions can have all
  // their loads in flight before it looks at any flag (a poll is a round trip to L2).
  __device__ static void recv_load(Msg& v, const char* src) {
    const char* p = src + lane() * (kLaneDw * 4);
    if constexpr (kLaneDw == 1) {
      v.d[0] = ld_volatile_u32(p);
    } else if constexpr (kLaneDw == 2) {
      ld_volatile_v2(p, v.d[0], v.d[1]);
    } else {
      ld_volatile_v4(p, v.d);
    }
  }
  // This lane's decision on its part of the transaction.
  __device__ static bool recv_ok(const Msg& v, uint32_t flag) {
    const int l = lane();
    if constexpr (K == ProtoKind::LL8) {
      return v.d[1] == flag;
    } else if constexpr (K == ProtoKind::LL16) {
      return (v.d[1] == flag) && (v.d[3] == flag);
    } else if constexpr (K == ProtoKind::LL128) {
      return !(l == 15 || l == 31) || (v.d[0] == flag);
    } else {
      return ((l & 3) != 3) || (v.d[3] == flag);
    }
  }
  // Loads the transaction; returns true (to the whole warp) when every flag matches.
  __device__ static bool try_recv(Msg& v, const char* src, uint32_t flag) {
    recv_load(v, src);
    return __all_sync(0xffffffffu, recv_ok(v, flag));
  }

  // Waits for several transactions at once: bit i of `pending` set = m[i] is still expected from
  // src(i) (sent by rank peer(i)).  Every round issues the loads of all pending transactions
  // back to back and only then tests them, so the round trips overlap instead of adding up.
  template <int CNT, class SrcFn, class PeerFn>
  __device__ static bool wait_many(const DevWaiter& w, Msg (&m)[CNT], SrcFn src, PeerFn peer, uint32_t pending,
                                   uint32_t flag, int site, int64_t step, int rank) {
    uint32_t spins = 0;
    uint64_t t0 = 0;
    for (;;) {
#pragma unroll
      for (int i = 0; i < CNT; ++i)
        if (pending & (1u << i)) recv_load(m[i], src(i));
      uint32_t mine = 0;
#pragma unroll
      for (int i = 0; i < CNT; ++i)
        if ((pending & (1u << i)) && recv_ok(m[i], flag)) mine |= 1u << i;
      pending &= ~__reduce_and_sync(0xffffffffu, mine | ~pending);
      if (pending == 0) return true;
      if ((++spins & 0xffu) == 0) {
        int give_up = 0;
        if (lane() == 0) {
          if (ld_volatile_u32(w.abort_word()) != 0) {
            give_up = 1;
          } else {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) {
              t0 = now;
            } else if (now - t0 > w.me->timeout_ns) {
              give_up = 2;
            }
          }
        }
        give_up = __shfl_sync(0xffffffffu, give_up, 0);
        if (give_up) {
          const int first = __ffs(int(pending)) - 1;
          if (give_up == 2) report_timeout(w, src(first), flag, site, peer(first), step, rank);
          else if (lane() == 0) note_aborted_by_peer(w.abort_word(), w.me->status, rank, site);
          return false;
        }
      }
    }
  }

  __device__ static bool wait(const DevWaiter& w, Msg& v, const char* src, uint32_t flag, int site, int peer,
                              int64_t step, int rank) {
    uint32_t spins = 0;
    uint64_t t0 = 0;
    for (;;) {
      if (try_recv(v, src, flag)) return true;
      if ((++spins & 0xffu) == 0) {
        int give_up = 0;
        if (lane() == 0) {
          if (ld_volatile_u32(w.abort_word()) != 0) {
            give_up = 1;
          } else {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) {
              t0 = now;
            } else if (now - t0 > w.me->timeout_ns) {
              give_up = 2;
            }
          }
        }
        give_up = __shfl_sync(0xffffffffu, give_up, 0);
        if (give_up) {
          if (give_up == 2) report_timeout(w, src, flag, site, peer, step, rank);
          else if (lane() == 0) note_aborted_by_peer(w.abort_word(), w.me->status, rank, site);
          return false;
        }
      }
    }
  }

  __device__ static void report_timeout(const DevWaiter& w, const char* src, uint32_t flag, int site, int peer,
                                        int64_t step, int rank) {
    const int l = lane();
    if (l == 0) {
      StatusBlock* s = w.me->status;
      if (claim_status(w.abort_word(), kTimeout)) {
        // first wire of this rank to give up: record the site
        s->rank = uint32_t(rank);
        s->peer = uint32_t(peer);
        s->wire = uint32_t(w.wire);
        s->step = uint32_t(step);
        s->expected = flag;
        s->seen = ld_volatile_u32(src + (kTxnBytes - 4));
        s->where = uint32_t(site);
        __threadfence_system();
        s->code = kTimeout;
      }
      __threadfence_system();
      st_volatile_u32(w.abort_word(), 1u);
    }
    if (l < w.me->world && l != rank) st_volatile_u32(w.peer_abort(l), 1u);
  }

  // ---- arithmetic ---------------------------------------------------------------
  __device__ static void acc_init(Acc& a, const Msg& v) {
#pragma unroll
    for (int j = 0; j < kAccDw; ++j) {
      float2 x = Cvt<T>::up(v.d[acc_slot(j)]);
      a.f[2 * j] = x.x;
      a.f[2 * j + 1] = x.y;
    }
  }
  __device__ static void acc_add(Acc& a, const Msg& v, bool round_each) {
#pragma unroll
    for (int j = 0; j < kAccDw; ++j) {
      float2 x = Cvt<T>::up(v.d[acc_slot(j)]);
      a.f[2 * j] += x.x;
      a.f[2 * j + 1] += x.y;
      if (round_each) {
        float2 y = Cvt<T>::up(Cvt<T>::down(a.f[2 * j], a.f[2 * j + 1]));
        a.f[2 * j] = y.x;
        a.f[2 * j + 1] = y.y;
      }
    }
  }
  __device__ static void acc_to_msg(Msg& v, const Acc& a) {
#pragma unroll
    for (int j = 0; j < kAccDw; ++j) v.d[acc_slot(j)] = Cvt<T>::down(a.f[2 * j], a.f[2 * j + 1]);
  }
};

}  // namespace b200ipc
