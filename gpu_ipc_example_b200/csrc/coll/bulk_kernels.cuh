// Large-message collectives over the symmetric heap: all-reduce, reduce-scatter
// and all-gather, each in two flavours selected by a template flag:
//   P2P   the owner of a shard loads it from every peer (16 B vectors over NVLink),
//         adds in rank order in fp32 and stores the result into every peer;
//   NVLS  multimem.ld_reduce lets the NVSwitch add the copies, multimem.st lets it
//         replicate the result: one load and one store per 16 B whatever the world.
// 100 % of the bytes on the wire are payload; ranks meet at per-CTA flag barriers
// (CTA b of every rank only ever depends on CTA b of the others), every wait is
// bounded.  These have no counterpart in the reference, whose kernels are all
// flag-in-data; they exist because at tens of megabytes the 6-50 % flag overhead
// and the register-resident messages stop paying.
#pragma once

#include "../proto/dev_backend.cuh"
#include "kernel_table.h"

namespace b200ipc {

constexpr int kBulkThreads = 512;

enum class BulkMode : int { AllReduce = 0, ReduceScatter = 1, AllGather = 2 };

// aux[1] bits
constexpr uint64_t kBulkCopyIn = 1;   // stage `in` into the symmetric buffer first
constexpr uint64_t kBulkCopyOut = 2;  // copy the result from the symmetric buffer to `out`

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <typename T>
__device__ __forceinline__ uint4 multimem_ld_reduce_add(const void* mc_addr);
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add<__half>(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add<__nv_bfloat16>(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_u4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Barrier between CTA `blockIdx.x` of every rank.  All threads call it; returns
// false (to all threads) if the wait ran out or the collective was aborted.
// `publish` = this CTA has written something the other ranks are about to read (its
// signal must then be a release); an arrival that only says "my kernel has started" is a
// plain store.  The polls are relaxed loads, and what the other ranks published is read
// afterwards with loads that go around L1 (ld.volatile / multimem), issued after the poll
// has returned: no acquire fence is paid for.
__device__ __forceinline__ bool cta_rank_barrier(const RankView& me, const HeapLayout& lay, uint32_t value,
                                                 int site, bool publish) {
  __shared__ int s_fail;
  const int tid = int(threadIdx.x);
  if (tid == 0) s_fail = 0;
  __syncthreads();  // also orders every thread's earlier writes before the signal below
  const size_t pad_off = lay.ctrl_off + kCtrlBarrierOff + size_t(blockIdx.x) * kMaxRanks * sizeof(uint32_t);
  if (tid < me.world && tid != me.rank) {
    uint32_t* abort_word = reinterpret_cast<uint32_t*>(me.heap + lay.ctrl_off + kCtrlAbortOff);
    if (!(me.flags & kMuteSends)) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(me.peer[tid] + pad_off) + me.rank;
      // st.release.sys orders the CTA's earlier accesses (made visible to this thread by the
      // barrier above) before the signal
      if (publish) st_release_sys_u32(dst, value);
      else st_relaxed_sys_u32(dst, value);
    }
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(me.heap + pad_off) + tid;
    uint32_t spins = 0;
    uint64_t t0 = 0;
    for (;;) {
      uint32_t seen = ld_relaxed_sys_u32(mine);
      if (int32_t(seen - value) >= 0) break;
      if ((++spins & 0x3fu) == 0) {
        if (ld_volatile_u32(abort_word) != 0) {
          note_aborted_by_peer(abort_word, me.status, me.rank, site);
          s_fail = 1;
          break;
        }
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) {
          t0 = now;
        } else if (now - t0 > me.timeout_ns) {
          if (claim_status(abort_word, kTimeout)) {
            StatusBlock* s = me.status;
            s->rank = uint32_t(me.rank);
            s->peer = uint32_t(tid);
            s->wire = blockIdx.x;
            s->step = 0;
            s->expected = value;
            s->seen = seen;
            s->where = uint32_t(site);
            __threadfence_system();
            s->code = kTimeout;
            __threadfence_system();
          }
          for (int q = 0; q < me.world; ++q)  // own abort word included
            st_volatile_u32(reinterpret_cast<uint32_t*>(me.peer[q] + lay.ctrl_off + kCtrlAbortOff), 1u);
          s_fail = 1;
          break;
        }
      }
    }
  }
  __syncthreads();
  return s_fail == 0;
}

template <typename T>
__device__ __forceinline__ void acc8_add(float (&a)[8], uint4 v) {
  float2 x;
  x = Cvt<T>::up(v.x); a[0] += x.x; a[1] += x.y;
  x = Cvt<T>::up(v.y); a[2] += x.x; a[3] += x.y;
  x = Cvt<T>::up(v.z); a[4] += x.x; a[5] += x.y;
  x = Cvt<T>::up(v.w); a[6] += x.x; a[7] += x.y;
}
template <typename T>
__device__ __forceinline__ uint4 acc8_pack(const float (&a)[8]) {
  return make_uint4(Cvt<T>::down(a[0], a[1]), Cvt<T>::down(a[2], a[3]), Cvt<T>::down(a[4], a[5]),
                    Cvt<T>::down(a[6], a[7]));
}

// Elements [0, nelems) of a 16-bit buffer as 16 B vectors, guarded at the tail.
__device__ __forceinline__ uint4 ld_vec_guarded(const uint16_t* src, int64_t vec, int64_t nelems) {
  const int64_t e0 = vec * 8;
  if (e0 + 8 <= nelems && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
    return *reinterpret_cast<const uint4*>(src + e0);
  }
  uint16_t t[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) t[k] = (e0 + k < nelems) ? src[e0 + k] : uint16_t(0);
  return make_uint4(uint32_t(t[0]) | (uint32_t(t[1]) << 16), uint32_t(t[2]) | (uint32_t(t[3]) << 16),
                    uint32_t(t[4]) | (uint32_t(t[5]) << 16), uint32_t(t[6]) | (uint32_t(t[7]) << 16));
}
__device__ __forceinline__ void st_vec_guarded(uint16_t* dst, int64_t vec, int64_t nelems, uint4 v) {
  const int64_t e0 = vec * 8;
  if (e0 + 8 <= nelems && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
    *reinterpret_cast<uint4*>(dst + e0) = v;
    return;
  }
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int k = 0; k < 8; ++k)
    if (e0 + k < nelems) dst[e0 + k] = uint16_t(w[k >> 1] >> ((k & 1) * 16));
}

// Work split: the buffer is `parts` shards of shard_vec vectors; inside a shard,
// tile j (kU * blockDim vectors) belongs to CTA j % gridDim.x on every rank.
template <typename T, int N, bool NVLS, BulkMode M>
__global__ void __launch_bounds__(kBulkThreads) bulk_kernel(const __grid_constant__ KArgs args) {
  const RankView& me = args.v[blockIdx.y];
  const HeapLayout& lay = args.lay;
  constexpr int kU = bulk_unroll(N, NVLS);
  const int tid = int(threadIdx.x);
  const int nthreads = int(blockDim.x);
  const int G = int(gridDim.x);
  const int b = int(blockIdx.x);
  const int r = me.rank;
  const size_t sym_off = size_t(me.aux[0]);
  const bool copy_in = (me.aux[1] & kBulkCopyIn) != 0;
  const bool copy_out = (me.aux[1] & kBulkCopyOut) != 0;

  uint32_t bar = me.bar_seq;
  if (me.seq_dev) bar += ld_volatile_u32(me.seq_dev + 2);

  // Shards.  In the caller's buffer shard s holds shard_elems elements starting at
  // s * shard_elems (AllReduce: a vector-aligned cut of the whole buffer;
  // ReduceScatter: nelems / N; AllGather: nelems = one rank's contribution).  In the
  // symmetric buffer shard s starts at vector s * shard_vec.
  const int64_t nelems = int64_t(me.nelems);
  int64_t shard_elems, shard_vec;
  if (M == BulkMode::AllReduce) {
    const int64_t total_vec = (nelems + 7) / 8;
    shard_vec = (total_vec + N - 1) / N;
    shard_elems = shard_vec * 8;
  } else if (M == BulkMode::ReduceScatter) {
    shard_elems = nelems / N;
    shard_vec = (shard_elems + 7) / 8;
  } else {
    shard_elems = nelems;
    shard_vec = (shard_elems + 7) / 8;
  }
  auto valid = [&](int s) -> int64_t {
    if (M != BulkMode::AllReduce) return shard_elems;
    int64_t v = nelems - int64_t(s) * shard_elems;
    return v < 0 ? 0 : (v > shard_elems ? shard_elems : v);
  };
  // A slab is blockDim consecutive vectors; slab j belongs to CTA j % gridDim.x on every rank
  // and a CTA keeps kU of its slabs in flight.
  const int64_t ntiles = (shard_vec + nthreads - 1) / nthreads;

  char* my_buf = me.heap + sym_off;
  const uint16_t* in16 = static_cast<const uint16_t*>(me.in);
  uint16_t* out16 = static_cast<uint16_t*>(me.out);

  // ---- phase 0: stage the input ------------------------------------------------
  if (M != BulkMode::AllGather && copy_in) {
    for (int s = 0; s < N; ++s) {
      const int64_t nv = valid(s);
      for (int64_t tile = b; tile < ntiles; tile += int64_t(G) * kU)
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int64_t i = (tile + int64_t(u) * G) * nthreads + tid;
          if (i < shard_vec && i * 8 < nv)
            *reinterpret_cast<uint4*>(my_buf + (int64_t(s) * shard_vec + i) * 16) =
                ld_vec_guarded(in16 + int64_t(s) * shard_elems, i, nv);
        }
    }
  }
  // Every rank has arrived (so it has left the previous collective and, for the
  // reducing modes, its input is in place) before any remote access.
  if (!cta_rank_barrier(me, lay, bar + 1, 10, /*publish=*/copy_in)) return;

  // ---- phase 1: the collective ---------------------------------------------------
  if (M == BulkMode::AllGather) {
    const uint16_t* src16 = copy_in ? in16 : reinterpret_cast<const uint16_t*>(my_buf + int64_t(r) * shard_vec * 16);
    for (int64_t tile = b; tile < ntiles; tile += int64_t(G) * kU) {
      uint4 v[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t i = (tile + int64_t(u) * G) * nthreads + tid;
        if (i < shard_vec) v[u] = ld_vec_guarded(src16, i, shard_elems);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t i = (tile + int64_t(u) * G) * nthreads + tid;
        if (i >= shard_vec) continue;
        const size_t off = sym_off + size_t(int64_t(r) * shard_vec + i) * 16;
        if (me.flags & kMuteSends) continue;
        if (NVLS) {
          multimem_st_v4(me.mc + off, v[u]);
        } else {
#pragma unroll
          for (int k = 0; k < N; ++k) {
            const int q = (r + k) % N;
            if (q == r && !copy_in) continue;
            *reinterpret_cast<uint4*>(me.peer[q] + off) = v[u];
          }
        }
      }
    }
  } else {
    for (int64_t tile = b; tile < ntiles; tile += int64_t(G) * kU) {
      uint4 res[kU];
      if (NVLS) {
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int64_t i = (tile + int64_t(u) * G) * nthreads + tid;
          if (i < shard_vec)
            res[u] = multimem_ld_reduce_add<T>(me.mc + sym_off + size_t(int64_t(r) * shard_vec + i) * 16);
        }
      } else {
        uint4 v[kU][N];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int64_t i = (tile + int64_t(u) * G) * nthreads + tid;
          if (i < shard_vec) {
            const size_t off = sym_off + size_t(int64_t(r) * shard_vec + i) * 16;
#pragma unroll
            for (int q = 0; q < N; ++q) v[u][q] = ld_volatile_u4(me.peer[q] + off);
          }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int q = 0; q < N; ++q) acc8_add<T>(a, v[u][q]);
          res[u] = acc8_pack<T>(a);
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t i = (tile + int64_t(u) * G) * nthreads + tid;
        if (i >= shard_vec) continue;
        if (M == BulkMode::ReduceScatter) {
          st_vec_guarded(out16, i, shard_elems, res[u]);  // my shard only, straight to the caller
        } else if (!(me.flags & kMuteSends)) {
          const size_t off = sym_off + size_t(int64_t(r) * shard_vec + i) * 16;
          if (NVLS) {
            multimem_st_v4(me.mc + off, res[u]);
          } else {
#pragma unroll
            for (int k = 0; k < N; ++k) {
              const int q = (r + k) % N;
              *reinterpret_cast<uint4*>(me.peer[q] + off) = res[u];
            }
          }
        }
      }
    }
  }

  // ---- phase 2: everyone's loads and stores are done ---------------------------------
  if (!cta_rank_barrier(me, lay, bar + 2, 11, /*publish=*/true)) return;

  // ---- phase 3: hand the result to the caller ----------------------------------------
  if (M != BulkMode::ReduceScatter && copy_out) {
    for (int s = 0; s < N; ++s) {
      const int64_t nv = valid(s);
      for (int64_t tile = b; tile < ntiles; tile += int64_t(G) * kU)
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int64_t i = (tile + int64_t(u) * G) * nthreads + tid;
          if (i < shard_vec && i * 8 < nv)
            st_vec_guarded(out16 + int64_t(s) * shard_elems, i, nv, ld_volatile_u4(my_buf + (int64_t(s) * shard_vec + i) * 16));
        }
    }
  }

  // ---- device-side sequence counter (graph-captured launches) ---------------------------
  if (me.seq_dev) {
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(me.seq_dev + 1, 1u) == gridDim.x - 1) {
        me.seq_dev[1] = 0;
        me.seq_dev[2] += 4;
        __threadfence();
      }
    }
  }
}

using BulkKernelFn = void (*)(const KArgs);
BulkKernelFn bulk_lookup(DType t, int world, bool nvls, BulkMode m);

}  // namespace b200ipc
