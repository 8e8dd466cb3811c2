// Kernels for one decode step of a Llama-shaped tensor-parallel decoder, for the parts of the step
// that are neither a GEMM nor a collective: rotary embedding fused with the KV-cache append,
// attention of one new token over the cache (grouped-query, split over the context), SiLU(gate) * up.
// Each replaces a chain of small framework kernels with one pass over the data it has to touch;
// all three are bound by memory traffic (the attention reads batch x context x 2 x head_dim x 2 B of
// cache per KV head and nothing twice).
//
// The reference has no model code; its smoke script shows the consumer these serve: decode-sized
// activations of a tensor-parallel LLM (script/gpu_inference_test.py:29-45).
#include "decode_ops.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../common/check.h"
#include "../common/pdl.h"

namespace b200ipc {
namespace {

template <typename T>
struct Num;
template <>
struct Num<__half> {
  using T2 = __half2;
  __device__ static float2 up(T2 v) { return __half22float2(v); }
  __device__ static T2 down(float a, float b) { return __floats2half2_rn(a, b); }
};
template <>
struct Num<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  __device__ static float2 up(T2 v) { return __bfloat1622float2(v); }
  __device__ static T2 down(float a, float b) { return __floats2bfloat162_rn(a, b); }
};

// Every kernel of this file starts with pdl_launch_dependents() + pdl_wait() and is launched with programmatic
// stream serialisation: its CTAs can be resident before the previous kernel of the step has drained.
template <typename... Params, typename... Args>
void launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1u : 0u;
  B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...));
}

// ---------------------------------------------------------------------------------------------
// RoPE + cache append.  qkv: [B, (hq + 2 hkv) * D] as the QKV projection leaves it.  Rotates q in
// place (pairs (i, i + D/2)), writes the rotated k and the v of the new position into the caches
// [B, hkv, max_ctx, D] at `pos`.  One CTA per (batch row, head), one thread per pair.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_append_kernel(T* qkv, T* kcache, T* vcache, int hq, int hkv, int D,
                                      int max_ctx, int pos, float log2_theta) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const int head = blockIdx.y;  // 0..hq-1: q, hq..hq+hkv-1: k, then v
  const int half = D / 2;
  T* row = qkv + (size_t(b) * (hq + 2 * hkv) + head) * D;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    if (head < hq + hkv) {
      // angle = pos * theta^(-i / half)
      const float inv = exp2f(-log2_theta * float(i) / float(half));
      float sn, cs;
      sincosf(float(pos) * inv, &sn, &cs);
      const float x1 = float(row[i]), x2 = float(row[i + half]);
      const T y1 = T(x1 * cs - x2 * sn), y2 = T(x2 * cs + x1 * sn);
      if (head < hq) {
        row[i] = y1;
        row[i + half] = y2;
      } else {
        T* dst = kcache + ((size_t(b) * hkv + (head - hq)) * max_ctx + pos) * D;
        dst[i] = y1;
        dst[i + half] = y2;
      }
    } else {
      T* dst = vcache + ((size_t(b) * hkv + (head - hq - hkv)) * max_ctx + pos) * D;
      dst[i] = row[i];
      dst[i + half] = row[i + half];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Decode attention, head_dim 128, G = hq / hkv query heads per KV head (1, 2, 4 or 8).
// Grid (splits, hkv, B), 128 threads.  A warp walks its share of the context 16 positions at a
// time on the warp-level tensor path (mma.sync m16n8k16, fp32 accumulation); the cache goes
// from global memory straight into the operand registers with 16-byte loads, nothing is staged:
//
//   scores   S[head, pos] = Q K^T : A = Q (rows = the G heads, zero-padded to 16), B = K^T.  The
//            contraction index may be permuted as long as A and B agree, so the lane (r, c) =
//            (lane / 4, lane % 4) simply loads the 16-byte chunks c, c+4, c+8, c+12 of "its" row
//            (Q: head r, K: position r of the 8-position tile) and word 2k / 2k+1 of those 16
//            words feeds step k.
//   softmax  online, in the log2 domain, per head; a quad (the 4 lanes of one head) shares the max.
//   output   O^T[dim, head] = V^T P^T : B = P^T is exactly the register layout S came out in; for
//            A = V^T the lane loads 32 contiguous bytes (dims 16r .. 16r+15) of the four positions
//            2c, 2c+1, 2c+8, 2c+9 and a byte-permute pairs the same dimension of two positions.
//            Output rows are permuted so that the lane ends up with dims 16r .. 16r+15 of heads
//            2c and 2c+1.
//
// Warps merge in shared memory, splits through a workspace; the last CTA of a (batch, KV head)
// to arrive writes the result.
// ---------------------------------------------------------------------------------------------
constexpr int kAttnD = 128;
constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kAttnTile = 16;  // positions per warp step

template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                  uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const typename Num<T>::T2 v = Num<T>::down(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// 16 words of a 256-byte row: the 16-byte chunks c, c+4, c+8, c+12
template <typename T>
__device__ __forceinline__ void load_row_quarter(uint32_t (&w)[16], const T* row, int c) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 x = *reinterpret_cast<const uint4*>(row + (c + 4 * i) * 8);
    w[4 * i + 0] = x.x; w[4 * i + 1] = x.y; w[4 * i + 2] = x.z; w[4 * i + 3] = x.w;
  }
}

template <typename T, int G>
__global__ void __launch_bounds__(kAttnThreads, 2) decode_attention_kernel(const T* q, const T* kcache, const T* vcache, T* out,
                                                                           float* part, unsigned int* counters,
                                                                        int hq, int hkv, int max_ctx, int ctx, int q_row_stride,
                                                                        float scale_log2) {
  using T2 = typename Num<T>::T2;
  pdl_launch_dependents();
  pdl_wait();
  const int split = blockIdx.x, nsplit = gridDim.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, c = lane & 3;

  // Q operand: head r of this KV head's group (rows G..15 of the 16-row operand are zero)
  uint32_t qa[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) qa[i] = 0u;
  if (r < G) load_row_quarter<T>(qa, q + size_t(b) * q_row_stride + (size_t(h) * G + r) * kAttnD, c);

  // running state of head r (every lane of the quad holds the same m; l is a per-lane partial sum)
  float m = -INFINITY, l = 0.f;
  // O^T: acc[t][0..3] = (dim 16r+2t, head 2c), (dim 16r+2t, head 2c+1), (dim 16r+2t+1, head 2c), (dim 16r+2t+1, head 2c+1)
  float acc[8][4];
#pragma unroll
  for (int t = 0; t < 8; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;

  const int per = ((ctx + nsplit - 1) / nsplit + kAttnTile - 1) / kAttnTile * kAttnTile;  // whole tiles per split
  const int p0 = split * per;
  const int p1 = min(p0 + per, ctx);  // may be <= p0: a split without work contributes an empty state
  const T* kb = kcache + (size_t(b) * hkv + h) * size_t(max_ctx) * kAttnD;
  const T* vb = vcache + (size_t(b) * hkv + h) * size_t(max_ctx) * kAttnD;

  // one step's operands: K rows of positions base + r and base + 8 + r, V of the four positions 2c, 2c+1, 2c+8, 2c+9
  auto load_tile = [&](int base, uint32_t (&kw)[2][16], uint32_t (&vw)[4][8]) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int p = base + 8 * j + r;
      if (p < p1) {
        load_row_quarter<T>(kw[j], kb + size_t(p) * kAttnD, c);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) kw[j][i] = 0u;
      }
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int p = base + 2 * c + (x & 1) + 8 * (x >> 1);
      if (p < p1) {
        const uint4 lo = *reinterpret_cast<const uint4*>(vb + size_t(p) * kAttnD + 16 * r);
        const uint4 hi = *reinterpret_cast<const uint4*>(vb + size_t(p) * kAttnD + 16 * r + 8);
        vw[x][0] = lo.x; vw[x][1] = lo.y; vw[x][2] = lo.z; vw[x][3] = lo.w;
        vw[x][4] = hi.x; vw[x][5] = hi.y; vw[x][6] = hi.z; vw[x][7] = hi.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) vw[x][i] = 0u;
      }
    }
  };
  auto compute_tile = [&](int base, const uint32_t (&kw)[2][16], const uint32_t (&vw)[4][8]) {
    // ---- scores: s[j][0..1] = head r, positions base + 8j + 2c, + 1 --------------------------------
    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) mma_16816<T>(s[j], qa[2 * k], 0u, qa[2 * k + 1], 0u, kw[j][2 * k], kw[j][2 * k + 1]);
    }
    float sc[4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) sc[2 * j + e] = (base + 8 * j + 2 * c + e < p1) ? s[j][e] * scale_log2 : -INFINITY;
    float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mnew = fmaxf(m, mx);  // finite: position `base` exists
    const float corr = exp2f(m - mnew);
    m = mnew;
    float pr[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) pr[e] = exp2f(sc[e] - mnew);
    l = l * corr + (pr[0] + pr[1]) + (pr[2] + pr[3]);
    const uint32_t pb0 = pack2<T>(pr[0], pr[1]), pb1 = pack2<T>(pr[2], pr[3]);
    // the accumulator columns of this lane belong to heads 2c and 2c+1, whose state lives in quads 2c and 2c+1
    const float corr0 = __shfl_sync(0xffffffffu, corr, 8 * c);
    const float corr1 = __shfl_sync(0xffffffffu, corr, 8 * c + 4);
    // ---- O^T += V^T P^T --------------------------------------------------------------------------
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      acc[t][0] *= corr0; acc[t][1] *= corr1; acc[t][2] *= corr0; acc[t][3] *= corr1;
      const uint32_t a0 = __byte_perm(vw[0][t], vw[1][t], 0x5410);  // dim 16r+2t   of positions 2c, 2c+1
      const uint32_t a1 = __byte_perm(vw[0][t], vw[1][t], 0x7632);  // dim 16r+2t+1 of positions 2c, 2c+1
      const uint32_t a2 = __byte_perm(vw[2][t], vw[3][t], 0x5410);  // ... of positions 2c+8, 2c+9
      const uint32_t a3 = __byte_perm(vw[2][t], vw[3][t], 0x7632);
      mma_16816<T>(acc[t], a0, a1, a2, a3, pb0, pb1);
    }
  };
  // two register sets: the loads of the next step are in flight while this one is computed
  {
    const int stride = kAttnWarps * kAttnTile;
    uint32_t kA[2][16], vA[4][8], kB[2][16], vB[4][8];
    int base = p0 + warp * kAttnTile;
    if (base < p1) load_tile(base, kA, vA);
    while (base < p1) {
      const int nb = base + stride;
      if (nb < p1) load_tile(nb, kB, vB);
      compute_tile(base, kA, vA);
      if (nb >= p1) break;
      base = nb + stride;
      if (base < p1) load_tile(base, kA, vA);
      compute_tile(nb, kB, vB);
    }
  }
  // the quad's partial sums of l
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);

  // ---- merge the warps of the CTA -----------------------------------------------------------
  __shared__ float s_m[kAttnWarps][G], s_l[kAttnWarps][G];
  __shared__ __align__(16) float4 s_o[kAttnWarps][G][32];
  __shared__ int s_last;
  if (c == 0 && r < G) {
    s_m[warp][r] = m;
    s_l[warp][r] = l;
  }
  {
    float* so = reinterpret_cast<float*>(&s_o[warp][0][0]);  // [head][dim]
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      if (2 * c < G) {
        so[(2 * c) * kAttnD + 16 * r + 2 * t] = acc[t][0];
        so[(2 * c) * kAttnD + 16 * r + 2 * t + 1] = acc[t][2];
      }
      if (2 * c + 1 < G) {
        so[(2 * c + 1) * kAttnD + 16 * r + 2 * t] = acc[t][1];
        so[(2 * c + 1) * kAttnD + 16 * r + 2 * t + 1] = acc[t][3];
      }
    }
  }
  __syncthreads();
  // thread t merges (head g = t / 32 ... ) : G * 32 items, 128 threads
  const size_t part_stride = size_t(G) * (4 + kAttnD);  // per (b, h, split): G x {m, l, -, -, o[128]}
  float* mine = part + ((size_t(b) * hkv + h) * nsplit + split) * part_stride;
  for (int item = threadIdx.x; item < G * 32; item += kAttnThreads) {
    const int g = item >> 5, ln = item & 31;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, s_m[w][g]);
    float ll = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float c = s_m[w][g] == -INFINITY ? 0.f : exp2f(s_m[w][g] - mm);
      ll += s_l[w][g] * c;
      const float4 v = s_o[w][g][ln];
      acc.x += v.x * c; acc.y += v.y * c; acc.z += v.z * c; acc.w += v.w * c;
    }
    float* dst = mine + size_t(g) * (4 + kAttnD);
    if (ln == 0) {
      dst[0] = mm;
      dst[1] = ll;
    }
    *reinterpret_cast<float4*>(dst + 4 + ln * 4) = acc;
  }
  // ---- the last CTA of this (batch, KV head) merges the splits ---------------------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&counters[b * hkv + h], 1u) == unsigned(nsplit - 1));
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* all = part + (size_t(b) * hkv + h) * nsplit * part_stride;
  for (int item = threadIdx.x; item < G * 32; item += kAttnThreads) {
    const int g = item >> 5, ln = item & 31;
    // eight splits per round: all their loads are in flight together (one L2 round trip per round)
    float mm = -INFINITY, ll = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < nsplit; s0 += 8) {
      float2 ml[8];
      float4 ov[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool in = s0 + j < nsplit;
        const float* src = all + size_t(in ? s0 + j : s0) * part_stride + size_t(g) * (4 + kAttnD);
        ml[j] = __ldcg(reinterpret_cast<const float2*>(src));
        ov[j] = __ldcg(reinterpret_cast<const float4*>(src + 4 + ln * 4));
        if (!in) ml[j].x = -INFINITY;
      }
      float mnew = mm;
#pragma unroll
      for (int j = 0; j < 8; ++j) mnew = fmaxf(mnew, ml[j].x);
      if (mnew == -INFINITY) continue;
      const float c0 = exp2f(mm - mnew);  // 0 on the first round (mm = -inf)
      ll *= c0;
      acc.x *= c0; acc.y *= c0; acc.z *= c0; acc.w *= c0;
      mm = mnew;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float cj = ml[j].x == -INFINITY ? 0.f : exp2f(ml[j].x - mm);
        ll += ml[j].y * cj;
        acc.x += ov[j].x * cj; acc.y += ov[j].y * cj; acc.z += ov[j].z * cj; acc.w += ov[j].w * cj;
      }
    }
    const float inv = 1.f / ll;
    T* dst = out + size_t(b) * hq * kAttnD + (size_t(h) * G + g) * kAttnD + ln * 4;
    *reinterpret_cast<T2*>(dst) = Num<T>::down(acc.x * inv, acc.y * inv);
    *reinterpret_cast<T2*>(dst + 2) = Num<T>::down(acc.z * inv, acc.w * inv);
  }
  if (threadIdx.x == 0) counters[b * hkv + h] = 0;  // ready for the next launch
}

// ---------------------------------------------------------------------------------------------
// act[b, f] = silu(gu[b, f]) * gu[b, F + f]
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* gu, T* act, int64_t rows, int F) {
  using T2 = typename Num<T>::T2;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t vec_per_row = F / 8;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row, c = i % vec_per_row;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * F + c * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c * 8);
    const T2* pg = reinterpret_cast<const T2*>(&g);
    const T2* pu = reinterpret_cast<const T2*>(&u);
    uint4 o;
    T2* po = reinterpret_cast<T2*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = Num<T>::up(pg[e]);
      const float2 b = Num<T>::up(pu[e]);
      po[e] = Num<T>::down(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    *reinterpret_cast<uint4*>(act + r * F + c * 8) = o;
  }
}

// ---------------------------------------------------------------------------------------------
// res_out = x + residual ; out = RMSNorm(res_out) * gamma.  One CTA per row, one pass: the row's sum stays in
// registers between the statistic and the scaling (rows of up to 8 x 4 x 256 elements, else a second read).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const T* x, const T* residual, const T* __restrict__ gamma, T* out,
                                                           T* res_out, int hidden, float eps) {
  using T2 = typename Num<T>::T2;
  pdl_launch_dependents();
  pdl_wait();
  constexpr int U = 4;
  const int64_t row = blockIdx.x;
  const int nvec = hidden / 8;
  const T* xr = x + row * hidden;
  const T* rr = residual + row * hidden;
  T* orow = out + row * hidden;
  T* srow = res_out + row * hidden;
  __shared__ float s_part[8];
  uint4 keep[U];
  float ss = 0.f;
  const bool in_regs = nvec <= U * int(blockDim.x);
  for (int v0 = threadIdx.x; v0 < nvec; v0 += U * blockDim.x) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * blockDim.x;
      if (v >= nvec) continue;
      const uint4 a = *reinterpret_cast<const uint4*>(xr + size_t(v) * 8);
      const uint4 b = *reinterpret_cast<const uint4*>(rr + size_t(v) * 8);
      const T2* pa = reinterpret_cast<const T2*>(&a);
      const T2* pb = reinterpret_cast<const T2*>(&b);
      uint4 o;
      T2* po = reinterpret_cast<T2*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fa = Num<T>::up(pa[e]), fb = Num<T>::up(pb[e]);
        po[e] = Num<T>::down(fa.x + fb.x, fa.y + fb.y);
        const float2 r = Num<T>::up(po[e]);
        ss += r.x * r.x + r.y * r.y;
      }
      *reinterpret_cast<uint4*>(srow + size_t(v) * 8) = o;
      if (in_regs) keep[u] = o;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < int(blockDim.x >> 5); ++w) tot += s_part[w];
  const float inv = rsqrtf(tot / float(hidden) + eps);
  for (int v0 = threadIdx.x; v0 < nvec; v0 += U * blockDim.x) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * blockDim.x;
      if (v >= nvec) continue;
      const uint4 xv = in_regs ? keep[u] : *reinterpret_cast<const uint4*>(srow + size_t(v) * 8);
      const uint4 g = *reinterpret_cast<const uint4*>(gamma + size_t(v) * 8);
      const T2* px = reinterpret_cast<const T2*>(&xv);
      const T2* pg = reinterpret_cast<const T2*>(&g);
      uint4 o;
      T2* po = reinterpret_cast<T2*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fx = Num<T>::up(px[e]), fg = Num<T>::up(pg[e]);
        po[e] = Num<T>::down(fx.x * inv * fg.x, fx.y * inv * fg.y);
      }
      *reinterpret_cast<uint4*>(orow + size_t(v) * 8) = o;
    }
  }
}

template <typename T>
void launch_attention(int G, dim3 grid, cudaStream_t stream, const T* q, const T* k, const T* v, T* out, float* part,
                      unsigned int* counters, int hq, int hkv, int max_ctx, int ctx, int q_row_stride, float scale_log2) {
  switch (G) {
    case 1: launch_pdl(decode_attention_kernel<T, 1>, grid, dim3(kAttnThreads), stream, q, k, v, out, part, counters, hq, hkv, max_ctx, ctx, q_row_stride, scale_log2); break;
    case 2: launch_pdl(decode_attention_kernel<T, 2>, grid, dim3(kAttnThreads), stream, q, k, v, out, part, counters, hq, hkv, max_ctx, ctx, q_row_stride, scale_log2); break;
    case 4: launch_pdl(decode_attention_kernel<T, 4>, grid, dim3(kAttnThreads), stream, q, k, v, out, part, counters, hq, hkv, max_ctx, ctx, q_row_stride, scale_log2); break;
    case 8: launch_pdl(decode_attention_kernel<T, 8>, grid, dim3(kAttnThreads), stream, q, k, v, out, part, counters, hq, hkv, max_ctx, ctx, q_row_stride, scale_log2); break;
    default: B200_REQUIRE(false, "decode attention supports 1, 2, 4 or 8 query heads per KV head, got " << G);
  }
}

}  // namespace

void rope_kv_append(DType t, void* qkv, void* kcache, void* vcache, int batch, int hq, int hkv, int head_dim, int max_ctx, int pos,
                    float theta, cudaStream_t stream) {
  B200_REQUIRE(head_dim % 2 == 0 && pos >= 0 && pos < max_ctx, "rope_kv_append: bad head_dim or position");
  const dim3 grid(static_cast<unsigned>(batch), static_cast<unsigned>(hq + 2 * hkv));
  const int threads = head_dim / 2 < 32 ? 32 : head_dim / 2;
  const float l2 = log2f(theta);
  if (t == DType::F16)
    launch_pdl(rope_kv_append_kernel<__half>, grid, dim3(unsigned(threads)), stream, static_cast<__half*>(qkv),
               static_cast<__half*>(kcache), static_cast<__half*>(vcache), hq, hkv, head_dim, max_ctx, pos, l2);
  else
    launch_pdl(rope_kv_append_kernel<__nv_bfloat16>, grid, dim3(unsigned(threads)), stream, static_cast<__nv_bfloat16*>(qkv),
               static_cast<__nv_bfloat16*>(kcache), static_cast<__nv_bfloat16*>(vcache), hq, hkv, head_dim, max_ctx, pos, l2);
  B200_CUDA_CHECK(cudaGetLastError());
}

size_t decode_attention_workspace_bytes(int batch, int hq, int hkv, int splits) {
  const int G = hq / hkv;
  return (size_t(batch) * hkv * splits * G * (4 + kAttnD) * sizeof(float) + 255) / 256 * 256 + size_t(batch) * hkv * sizeof(unsigned int);
}

int decode_attention_splits(int batch, int hkv, int ctx, int sm_count) {
  // two CTAs fit on an SM: as many splits as keep the whole grid resident at once, at least 64 positions each;
  // a power of two where that is close, so that a power-of-two context divides into whole, equal warp shares
  int s = (2 * sm_count) / (batch * hkv);
  if (s >= 8 && s < 12) s = 8;
  else if (s >= 4 && s < 6) s = 4;
  if (const char* e = std::getenv("B200IPC_ATTN_SPLITS")) s = std::atoi(e);  // experiments
  const int by_len = (ctx + 63) / 64;
  if (s > by_len) s = by_len;
  if (s < 1) s = 1;
  if (s > 32) s = 32;
  return s;
}

void decode_attention(DType t, const void* q, int q_row_stride, const void* kcache, const void* vcache, void* out, void* workspace,
                      int batch, int hq, int hkv, int head_dim, int max_ctx, int ctx, int splits, cudaStream_t stream) {
  B200_REQUIRE(head_dim == kAttnD, "decode attention is written for head_dim 128, got " << head_dim);
  B200_REQUIRE(hq % hkv == 0 && ctx >= 1 && ctx <= max_ctx && splits >= 1, "decode attention: bad shapes");
  const int G = hq / hkv;
  float* part = static_cast<float*>(workspace);
  // the arrival counters sit behind the partial results; they start at zero and every launch leaves them at zero
  unsigned int* counters = reinterpret_cast<unsigned int*>(
      static_cast<char*>(workspace) + (size_t(batch) * hkv * splits * G * (4 + kAttnD) * sizeof(float) + 255) / 256 * 256);
  const dim3 grid(static_cast<unsigned>(splits), static_cast<unsigned>(hkv), static_cast<unsigned>(batch));
  const float scale_log2 = 1.4426950408889634f / sqrtf(float(head_dim));
  if (t == DType::F16)
    launch_attention<__half>(G, grid, stream, static_cast<const __half*>(q), static_cast<const __half*>(kcache),
                             static_cast<const __half*>(vcache), static_cast<__half*>(out), part, counters, hq, hkv, max_ctx, ctx,
                             q_row_stride, scale_log2);
  else
    launch_attention<__nv_bfloat16>(G, grid, stream, static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(kcache),
                                    static_cast<const __nv_bfloat16*>(vcache), static_cast<__nv_bfloat16*>(out), part, counters, hq, hkv,
                                    max_ctx, ctx, q_row_stride, scale_log2);
  B200_CUDA_CHECK(cudaGetLastError());
}

void add_rmsnorm(DType t, const void* x, const void* residual, const void* gamma, void* out, void* res_out, int64_t rows, int hidden,
                 float eps, cudaStream_t stream) {
  B200_REQUIRE(hidden % 8 == 0 && rows > 0, "add_rmsnorm: hidden must be a multiple of 8");
  if (t == DType::F16)
    launch_pdl(add_rmsnorm_kernel<__half>, dim3(unsigned(rows)), dim3(256), stream, static_cast<const __half*>(x),
               static_cast<const __half*>(residual), static_cast<const __half*>(gamma), static_cast<__half*>(out),
               static_cast<__half*>(res_out), hidden, eps);
  else
    launch_pdl(add_rmsnorm_kernel<__nv_bfloat16>, dim3(unsigned(rows)), dim3(256), stream, static_cast<const __nv_bfloat16*>(x),
               static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(gamma),
               static_cast<__nv_bfloat16*>(out), static_cast<__nv_bfloat16*>(res_out), hidden, eps);
  B200_CUDA_CHECK(cudaGetLastError());
}

void silu_mul(DType t, const void* gate_up, void* act, int64_t rows, int ffn, int sm_count, cudaStream_t stream) {
  B200_REQUIRE(ffn % 8 == 0, "silu_mul: the FFN width must be a multiple of 8");
  const int64_t total = rows * (ffn / 8);
  const int threads = 256;
  int64_t blocks = (total + threads - 1) / threads;
  if (blocks > int64_t(sm_count) * 8) blocks = int64_t(sm_count) * 8;
  if (blocks < 1) blocks = 1;
  if (t == DType::F16)
    launch_pdl(silu_mul_kernel<__half>, dim3(unsigned(blocks)), dim3(unsigned(threads)), stream, static_cast<const __half*>(gate_up),
               static_cast<__half*>(act), rows, ffn);
  else
    launch_pdl(silu_mul_kernel<__nv_bfloat16>, dim3(unsigned(blocks)), dim3(unsigned(threads)), stream,
               static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(act), rows, ffn);
  B200_CUDA_CHECK(cudaGetLastError());
}

}  // namespace b200ipc
