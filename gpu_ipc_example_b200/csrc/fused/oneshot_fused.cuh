// One-shot all-reduce fused with what follows it in a tensor-parallel layer:
//   kEpiNorm   y = RMSNorm(sum_over_ranks(x) + residual) * gamma, and the pre-norm
//              sum is written back as the new residual;
//   kEpiScale  y = cast<Tout>(sum_over_ranks(x) * scale).
// Every rank pushes its partial activations to all peers as LL512 transactions
// (480 B payload per 512 B store, a flag closing each 64 B), adds the world copies
// in rank order in fp32 registers and applies the epilogue before anything is
// written to HBM: one NVLink hop, one read of x/residual, one write of the outputs.
// A CTA owns whole rows, so the row statistic never leaves the SM.
//
// No counterpart in the reference (its collectives are not fused with compute);
// the wire format and the one-shot schedule are the ones of proto/ and coll/.
#pragma once

#include "../coll/schedules.h"
#include "../proto/dev_backend.cuh"

namespace b200ipc {

constexpr int kEpiNorm = 0;
constexpr int kEpiScale = 1;
constexpr int kFusedMaxRowsPerCta = 64;
constexpr int kFusedMaxThreads = 512;  // 16 warps: leaves 128 registers per thread for the transactions kept in flight

template <typename Tout>
__device__ __forceinline__ uint32_t pack_out(float a, float b) { return Cvt<Tout>::down(a, b); }

// The whole exchange + epilogue for the calling CTA (all its threads call it).  `me` carries the
// operands as the kernel's launch arguments do: in / out / nelems, aux[0] residual, aux[1] gamma,
// aux[2] residual_out, aux[3] = hidden | (float bits of eps or scale) << 32.  Written as a function
// so that a kernel that PRODUCES the partial activations (the fused GEMM at decode sizes) can run
// the same exchange on them without leaving the kernel; such a caller advances the device-side
// sequence words itself (`advance_seq_dev` false).
template <typename T, typename Tout, int N, int EPI>
__device__ __forceinline__ void oneshot_fused_body(const RankView& me, const HeapLayout& lay, float* s_part, int* s_abort_p,
                                                   bool advance_seq_dev) {
  using B = DevBackend<ProtoKind::LL512, T>;
  int& s_abort = *s_abort_p;
  const int r = me.rank;
  const int lane = int(threadIdx.x & 31);
  const int warp = int(threadIdx.x >> 5);
  const int warps = int(blockDim.x >> 5);
  const int wire = int(blockIdx.x) * warps + warp;

  uint32_t seq = me.seq;
  if (me.seq_dev) seq += ld_volatile_u32(me.seq_dev);

  DevWaiter waiter;
  waiter.me = &me;
  waiter.ctrl_off = lay.ctrl_off;
  waiter.wire = wire;

  const uint32_t* in = static_cast<const uint32_t*>(me.in);
  const int64_t total_dw = int64_t(me.nelems / 2);

  // This CTA's range of dwords [d0, d1).
  int64_t d0, d1;
  int row0 = 0, nrows = 0;
  int64_t row_dw = 0;
  if (EPI == kEpiNorm) {
    const int hidden = int(uint32_t(me.aux[3]));
    row_dw = hidden / 2;
    const int rows = int(total_dw / row_dw);
    const int per = (rows + int(gridDim.x) - 1) / int(gridDim.x);
    row0 = int(blockIdx.x) * per;
    int row1 = row0 + per;
    if (row1 > rows) row1 = rows;
    nrows = row1 > row0 ? row1 - row0 : 0;
    d0 = int64_t(row0) * row_dw;
    d1 = d0 + int64_t(nrows) * row_dw;
  } else {
    int64_t per = ceil_div64(total_dw, int64_t(gridDim.x));
    per = round_up64(per, 4);
    d0 = int64_t(blockIdx.x) * per;
    d1 = min64(d0 + per, total_dw);
    if (d1 < d0) d1 = d0;
  }
  const int64_t ntx = ceil_div64(d1 - d0, B::kPayloadDw);

  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();

  const uint32_t* residual = reinterpret_cast<const uint32_t*>(me.aux[0]);
  uint32_t* res_out = reinterpret_cast<uint32_t*>(me.aux[2]);
  uint32_t* out = static_cast<uint32_t*>(me.out);
  const float scale = __uint_as_float(uint32_t(me.aux[3] >> 32));  // kEpiScale: multiplier; kEpiNorm: eps

  auto slot_at = [&](char* heap, int src, uint32_t flag) {
    return heap + lay.oneshot_off +
           ((int64_t(src) * kMaxOneShotWires + wire) * kOneShotSlots + int(flag % kOneShotSlots)) * kOneShotStride;
  };
  Ctx<B> cx{};
  cx.waiter = waiter;
  cx.rank = r;
  const int64_t steps = ceil_div64(ntx, warps);  // transactions per warp, the same on every warp up to one
  bool ok = true;

  // Few transactions per warp (the decode case): every send goes out before the first wait, what
  // does not depend on the peers (residual, gamma) is fetched while the transactions fly, and with
  // one row per CTA the sums stay in registers for the normalisation.
  constexpr int KMAX = 3;
  const bool fast = steps <= KMAX;
  if (fast) {
    typename B::Msg own[KMAX], rsd[KMAX], gam[KMAX];
    const bool norm_in_regs = EPI == kEpiNorm && nrows == 1;
#pragma unroll
    for (int k = 0; k < KMAX; ++k) {
      const int64_t j = warp + int64_t(k) * warps;
      if (j >= ntx) continue;
      const uint32_t flag = seq + uint32_t(k);
      const int64_t dw = d0 + j * B::kPayloadDw;
      B::load(own[k], in, dw, d1, -1);
      B::shuffle(own[k]);
      if (N > 1) {
        B::set_flags(own[k], flag);
        if (!(me.flags & kMuteSends)) {
#pragma unroll
          for (int i = 1; i < N; ++i) B::send(slot_at(me.peer[(r + i) % N], r, flag), own[k]);
        }
      }
    }
    if (EPI == kEpiNorm) {
#pragma unroll
      for (int k = 0; k < KMAX; ++k) {
        const int64_t j = warp + int64_t(k) * warps;
        if (j >= ntx) continue;
        const int64_t dw = d0 + j * B::kPayloadDw;
        B::load(rsd[k], residual, dw, d1, -1);
        B::shuffle(rsd[k]);
        if (norm_in_regs) B::load(gam[k], reinterpret_cast<const uint32_t*>(me.aux[1]), dw - d0, row_dw, -1);
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < KMAX; ++k) {
      const int64_t j = warp + int64_t(k) * warps;
      if (j >= ntx || !ok) continue;
      const uint32_t flag = seq + uint32_t(k);
      const int64_t dw = d0 + j * B::kPayloadDw;
      typename B::Acc a;
      ok = recv_in_order<B, 0, N>(
          cx, flag, 5, k, r, own[k], [&](int q) -> const char* { return slot_at(me.heap, q, flag); }, [&](int q) { return q; },
          [&](int q, const typename B::Msg& x) {
            if (q == 0) B::acc_init(a, x);
            else B::acc_add(a, x, false);
          });
      if (!ok) continue;
      if (EPI == kEpiNorm) {
        B::acc_add(a, rsd[k], false);
        B::acc_to_msg(own[k], a);
        B::restore(own[k]);
        B::store(res_out, dw, d1, -1, own[k]);
        if (norm_in_regs && lane < 30) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (dw + 4 * lane + e < d1) {
              const float2 x = Cvt<T>::up(own[k].d[e]);
              ss += x.x * x.x + x.y * x.y;
            }
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) a.f[e] *= scale;
        typename B::Msg o;
#pragma unroll
        for (int e = 0; e < 4; ++e) o.d[e] = pack_out<Tout>(a.f[2 * e], a.f[2 * e + 1]);
        B::restore(o);
        B::store(out, dw, d1, -1, o);
      }
    }
    if (!ok) s_abort = 1;
    if (norm_in_regs) {
      // the reduction order depends on nothing but the thread index: every rank computes the same bits
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) s_part[warp] = ss;
      __syncthreads();
      if (s_abort == 0) {
        float tot = 0.f;
        for (int w = 0; w < warps; ++w) tot += s_part[w];
        const float inv = rsqrtf(tot / float(int(uint32_t(me.aux[3]))) + scale);
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
          const int64_t j = warp + int64_t(k) * warps;
          if (j >= ntx) continue;
          const int64_t dw = d0 + j * B::kPayloadDw;
          typename B::Msg y;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 xf = Cvt<T>::up(own[k].d[e]);
            const float2 gf = Cvt<T>::up(gam[k].d[e]);
            y.d[e] = Cvt<T>::down(xf.x * inv * gf.x, xf.y * inv * gf.y);
          }
          B::store(out, dw, d1, -1, y);
        }
      }
    } else {
      __syncthreads();
    }
  } else {
    for (int64_t k = 0; ok; ++k) {
      const int64_t j = warp + k * warps;
      if (j >= ntx) break;
      const uint32_t flag = seq + uint32_t(k);
      const int64_t dw = d0 + j * B::kPayloadDw;
      typename B::Msg v;
      B::load(v, in, dw, d1, -1);
      B::shuffle(v);
      if (N > 1) {
        B::set_flags(v, flag);
        if (!(me.flags & kMuteSends)) {
#pragma unroll
          for (int i = 1; i < N; ++i) B::send(slot_at(me.peer[(r + i) % N], r, flag), v);
        }
      }
      // the world - 1 landing slots are polled in overlapping groups (a poll is a round trip to L2);
      // slices are added in rank order, the own one at position r
      typename B::Acc a;
      ok = recv_in_order<B, 0, N>(
          cx, flag, 5, k, r, v, [&](int q) -> const char* { return slot_at(me.heap, q, flag); }, [&](int q) { return q; },
          [&](int q, const typename B::Msg& x) {
            if (q == 0) B::acc_init(a, x);
            else B::acc_add(a, x, false);
          });
      if (!ok) break;
      if (EPI == kEpiNorm) {
        typename B::Msg rv;
        B::load(rv, residual, dw, d1, -1);
        B::shuffle(rv);
        B::acc_add(a, rv, false);
        B::acc_to_msg(v, a);
        B::restore(v);
        B::store(res_out, dw, d1, -1, v);
      } else {
        // scale and cast; lanes 30/31 carry displaced dwords, so restore first
#pragma unroll
        for (int e = 0; e < 8; ++e) a.f[e] *= scale;
        typename B::Msg o;
#pragma unroll
        for (int e = 0; e < 4; ++e) o.d[e] = pack_out<Tout>(a.f[2 * e], a.f[2 * e + 1]);
        B::restore(o);
        B::store(out, dw, d1, -1, o);
      }
    }
    if (!ok) s_abort = 1;
    __syncthreads();
  }

  if (EPI == kEpiNorm && s_abort == 0 && !(fast && nrows == 1)) {
    const int hidden = int(uint32_t(me.aux[3]));
    const float eps = scale;
    const uint4* gamma = reinterpret_cast<const uint4*>(me.aux[1]);
    const int row_vec = hidden / 8;
    // The row statistic is taken from the rounded sums this CTA has just written, by a reduction whose
    // order depends on nothing but the thread index: every rank computes the same bits (a floating-point
    // atomic would add the warps' shares in the order they happen to arrive).
    for (int rr = 0; rr < nrows; ++rr) {
      const uint4* src = reinterpret_cast<const uint4*>(res_out + (int64_t(row0 + rr)) * row_dw);
      uint4* dst = reinterpret_cast<uint4*>(out + (int64_t(row0 + rr)) * row_dw);
      float ss = 0.f;
      for (int i = int(threadIdx.x); i < row_vec; i += int(blockDim.x)) {
        const uint4 x = src[i];
        const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 xf = Cvt<T>::up(xs[e]);
          ss += xf.x * xf.x + xf.y * xf.y;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) s_part[warp] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < warps; ++w) tot += s_part[w];
      const float inv = rsqrtf(tot / float(hidden) + eps);
      for (int i = int(threadIdx.x); i < row_vec; i += int(blockDim.x)) {
        const uint4 x = src[i];
        const uint4 g = gamma[i];
        const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
        const uint32_t gs[4] = {g.x, g.y, g.z, g.w};
        uint32_t ys[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 xf = Cvt<T>::up(xs[e]);
          const float2 gf = Cvt<T>::up(gs[e]);
          ys[e] = Cvt<T>::down(xf.x * inv * gf.x, xf.y * inv * gf.y);
        }
        dst[i] = make_uint4(ys[0], ys[1], ys[2], ys[3]);
      }
      __syncthreads();  // s_part is reused by the next row
    }
  }

  if (me.seq_dev && advance_seq_dev) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(me.seq_dev + 1, 1u) == gridDim.x - 1) {
        me.seq_dev[1] = 0;
        me.seq_dev[0] += me.seq_step;
        __threadfence();
      }
    }
  }
}

template <typename T, typename Tout, int N, int EPI>
__global__ void __launch_bounds__(kFusedMaxThreads) oneshot_fused_kernel(const __grid_constant__ KArgs args) {
  __shared__ float s_part[32];
  __shared__ int s_abort;
  oneshot_fused_body<T, Tout, N, EPI>(args.v[blockIdx.y], args.lay, s_part, &s_abort, true);
}

}  // namespace b200ipc
