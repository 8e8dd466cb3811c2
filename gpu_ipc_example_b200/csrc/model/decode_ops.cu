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

// ---------------------------------------------------------------------------------------------
// RoPE + cache append.  qkv: [B, (hq + 2 hkv) * D] as the QKV projection leaves it.  Rotates q in
// place (pairs (i, i + D/2)), writes the rotated k and the v of the new position into the caches
// [B, hkv, max_ctx, D] at `pos`.  One CTA per (batch row, head), one thread per pair.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_append_kernel(T* __restrict__ qkv, T* __restrict__ kcache, T* __restrict__ vcache, int hq, int hkv, int D,
                                      int max_ctx, int pos, float log2_theta) {
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
// Grid (splits, hkv, B), 128 threads.  A warp walks its share of the context four positions at a
// time: for the scores eight lanes share a position (16 elements of the 256-byte K row each, two
// 16-byte loads, so a warp instruction reads 1 KiB of contiguous cache); for the weighted sum a lane
// owns 4 of the 128 dimensions of every position.  Online softmax per head in fp32.  Warps merge in
// shared memory, splits through a workspace; the last CTA of a (batch, KV head) to arrive writes
// the result.
// ---------------------------------------------------------------------------------------------
constexpr int kAttnD = 128;
constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = kAttnThreads / 32;

template <typename T, int G>
__global__ void __launch_bounds__(kAttnThreads) decode_attention_kernel(const T* __restrict__ q, const T* __restrict__ kcache,
                                                                        const T* __restrict__ vcache, T* __restrict__ out,
                                                                        float* __restrict__ part, unsigned int* __restrict__ counters,
                                                                        int hq, int hkv, int max_ctx, int ctx, int q_row_stride,
                                                                        float scale_log2) {
  using T2 = typename Num<T>::T2;
  const int split = blockIdx.x, nsplit = gridDim.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, sub = lane & 7;  // score phase: position within the four, 16-element slice of the row

  // the G query rows, pre-scaled by softmax scale * log2(e), in shared memory: [head][16-element slice][16 + 4 pad]
  // (the pad spreads the eight slices over all banks; the four lanes that share a slice read one address)
  __shared__ __align__(16) float s_q[G][8][20];
  for (int i = threadIdx.x; i < G * kAttnD; i += kAttnThreads) {
    const int g = i / kAttnD, d = i % kAttnD;
    s_q[g][d / 16][d % 16] = float(q[size_t(b) * q_row_stride + (size_t(h) * G + g) * kAttnD + d]) * scale_log2;
  }
  __syncthreads();

  float m[G], l[G], o[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
    o[g][0] = o[g][1] = o[g][2] = o[g][3] = 0.f;
  }

  const int per = (ctx + nsplit - 1) / nsplit;
  const int p0 = split * per;
  const int p1 = min(p0 + per, ctx);
  const T* kb = kcache + (size_t(b) * hkv + h) * size_t(max_ctx) * kAttnD;
  const T* vb = vcache + (size_t(b) * hkv + h) * size_t(max_ctx) * kAttnD;

  for (int base = p0 + warp * 4; base < p1; base += kAttnWarps * 4) {
    const int p = base + grp;
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    if (p < p1) {
      const uint4 a = *reinterpret_cast<const uint4*>(kb + size_t(p) * kAttnD + sub * 16);
      const uint4 c = *reinterpret_cast<const uint4*>(kb + size_t(p) * kAttnD + sub * 16 + 8);
      const T2* pa = reinterpret_cast<const T2*>(&a);
      const T2* pc = reinterpret_cast<const T2*>(&c);
      float2 kf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        kf[e] = Num<T>::up(pa[e]);
        kf[4 + e] = Num<T>::up(pc[e]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float4* qv = reinterpret_cast<const float4*>(&s_q[g][sub][0]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float4 qq = qv[e];
          s[g] = fmaf(qq.x, kf[2 * e].x, fmaf(qq.y, kf[2 * e].y, fmaf(qq.z, kf[2 * e + 1].x, fmaf(qq.w, kf[2 * e + 1].y, s[g]))));
        }
      }
    }
    // the eight lanes of a position add their slices
#pragma unroll
    for (int g = 0; g < G; ++g) {
      s[g] += __shfl_xor_sync(0xffffffffu, s[g], 1);
      s[g] += __shfl_xor_sync(0xffffffffu, s[g], 2);
      s[g] += __shfl_xor_sync(0xffffffffu, s[g], 4);
      if (p >= p1) s[g] = -INFINITY;
    }
    // V rows of the four positions: a lane owns dimensions 4 * lane .. + 3
    float4 vf[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      vf[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (base + j < p1) {
        const uint2 raw = *reinterpret_cast<const uint2*>(vb + size_t(base + j) * kAttnD + lane * 4);
        const float2 lo = Num<T>::up(*reinterpret_cast<const T2*>(&raw.x));
        const float2 hi = Num<T>::up(*reinterpret_cast<const T2*>(&raw.y));
        vf[j] = make_float4(lo.x, lo.y, hi.x, hi.y);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      // scores of the four positions to every lane
      float sj[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) sj[j] = __shfl_sync(0xffffffffu, s[g], j * 8);
      const float mx = fmaxf(fmaxf(sj[0], sj[1]), fmaxf(sj[2], sj[3]));
      const float mnew = fmaxf(m[g], mx);  // finite: position `base` always exists
      const float corr = exp2f(m[g] - mnew);
      m[g] = mnew;
      float pj[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) pj[j] = exp2f(sj[j] - mnew);
      l[g] = l[g] * corr + (pj[0] + pj[1]) + (pj[2] + pj[3]);
      o[g][0] = o[g][0] * corr + pj[0] * vf[0].x + pj[1] * vf[1].x + pj[2] * vf[2].x + pj[3] * vf[3].x;
      o[g][1] = o[g][1] * corr + pj[0] * vf[0].y + pj[1] * vf[1].y + pj[2] * vf[2].y + pj[3] * vf[3].y;
      o[g][2] = o[g][2] * corr + pj[0] * vf[0].z + pj[1] * vf[1].z + pj[2] * vf[2].z + pj[3] * vf[3].z;
      o[g][3] = o[g][3] * corr + pj[0] * vf[0].w + pj[1] * vf[1].w + pj[2] * vf[2].w + pj[3] * vf[3].w;
    }
  }

  // ---- merge the warps of the CTA -----------------------------------------------------------
  __shared__ float s_m[kAttnWarps][G], s_l[kAttnWarps][G];
  __shared__ float4 s_o[kAttnWarps][G][32];
  __shared__ int s_last;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      s_m[warp][g] = m[g];
      s_l[warp][g] = l[g];
    }
    s_o[warp][g][lane] = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
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
    float mm = -INFINITY;
    for (int s2 = 0; s2 < nsplit; ++s2) mm = fmaxf(mm, __ldcg(all + s2 * part_stride + size_t(g) * (4 + kAttnD)));
    float ll = 0.f;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (int s2 = 0; s2 < nsplit; ++s2) {
      const float* src = all + s2 * part_stride + size_t(g) * (4 + kAttnD);
      const float ms = __ldcg(src);
      const float c = ms == -INFINITY ? 0.f : exp2f(ms - mm);
      ll += __ldcg(src + 1) * c;
      a0 += __ldcg(src + 4 + ln * 4 + 0) * c;
      a1 += __ldcg(src + 4 + ln * 4 + 1) * c;
      a2 += __ldcg(src + 4 + ln * 4 + 2) * c;
      a3 += __ldcg(src + 4 + ln * 4 + 3) * c;
    }
    const float inv = 1.f / ll;
    T* dst = out + size_t(b) * hq * kAttnD + (size_t(h) * G + g) * kAttnD + ln * 4;
    *reinterpret_cast<T2*>(dst) = Num<T>::down(a0 * inv, a1 * inv);
    *reinterpret_cast<T2*>(dst + 2) = Num<T>::down(a2 * inv, a3 * inv);
  }
  if (threadIdx.x == 0) counters[b * hkv + h] = 0;  // ready for the next launch
}

// ---------------------------------------------------------------------------------------------
// act[b, f] = silu(gu[b, f]) * gu[b, F + f]
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ act, int64_t rows, int F) {
  using T2 = typename Num<T>::T2;
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
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ residual,
                                                           const T* __restrict__ gamma, T* __restrict__ out, T* __restrict__ res_out,
                                                           int hidden, float eps) {
  using T2 = typename Num<T>::T2;
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
    case 1: decode_attention_kernel<T, 1><<<grid, kAttnThreads, 0, stream>>>(q, k, v, out, part, counters, hq, hkv, max_ctx, ctx, q_row_stride, scale_log2); break;
    case 2: decode_attention_kernel<T, 2><<<grid, kAttnThreads, 0, stream>>>(q, k, v, out, part, counters, hq, hkv, max_ctx, ctx, q_row_stride, scale_log2); break;
    case 4: decode_attention_kernel<T, 4><<<grid, kAttnThreads, 0, stream>>>(q, k, v, out, part, counters, hq, hkv, max_ctx, ctx, q_row_stride, scale_log2); break;
    case 8: decode_attention_kernel<T, 8><<<grid, kAttnThreads, 0, stream>>>(q, k, v, out, part, counters, hq, hkv, max_ctx, ctx, q_row_stride, scale_log2); break;
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
    rope_kv_append_kernel<__half><<<grid, threads, 0, stream>>>(static_cast<__half*>(qkv), static_cast<__half*>(kcache),
                                                                static_cast<__half*>(vcache), hq, hkv, head_dim, max_ctx, pos, l2);
  else
    rope_kv_append_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(static_cast<__nv_bfloat16*>(qkv),
                                                                       static_cast<__nv_bfloat16*>(kcache),
                                                                       static_cast<__nv_bfloat16*>(vcache), hq, hkv, head_dim, max_ctx,
                                                                       pos, l2);
  B200_CUDA_CHECK(cudaGetLastError());
}

size_t decode_attention_workspace_bytes(int batch, int hq, int hkv, int splits) {
  const int G = hq / hkv;
  return (size_t(batch) * hkv * splits * G * (4 + kAttnD) * sizeof(float) + 255) / 256 * 256 + size_t(batch) * hkv * sizeof(unsigned int);
}

int decode_attention_splits(int batch, int hkv, int ctx, int sm_count) {
  // enough CTAs to fill the GPU twice over, at least 64 positions per split
  int s = (2 * sm_count + batch * hkv - 1) / (batch * hkv);
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
    add_rmsnorm_kernel<__half><<<unsigned(rows), 256, 0, stream>>>(static_cast<const __half*>(x), static_cast<const __half*>(residual),
                                                                  static_cast<const __half*>(gamma), static_cast<__half*>(out),
                                                                  static_cast<__half*>(res_out), hidden, eps);
  else
    add_rmsnorm_kernel<__nv_bfloat16><<<unsigned(rows), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(gamma),
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
    silu_mul_kernel<__half><<<unsigned(blocks), threads, 0, stream>>>(static_cast<const __half*>(gate_up), static_cast<__half*>(act), rows, ffn);
  else
    silu_mul_kernel<__nv_bfloat16><<<unsigned(blocks), threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(gate_up),
                                                                            static_cast<__nv_bfloat16*>(act), rows, ffn);
  B200_CUDA_CHECK(cudaGetLastError());
}

}  // namespace b200ipc
