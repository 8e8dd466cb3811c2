// Host entry points of the decode-step kernels (model/decode_ops.cu): rotary embedding + KV-cache
// append, attention of one new token over the cache, SiLU(gate) * up.  All stream-ordered, no
// allocation inside.  No counterpart in the reference (it has no model code).
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_runtime_api.h>

#include "../common/types.h"

namespace b200ipc {

// qkv: [batch, (hq + 2 hkv) * head_dim].  q is rotated in place; the rotated k and v of this step are
// written to kcache / vcache [batch, hkv, max_ctx, head_dim] at position `pos`.
void rope_kv_append(DType t, void* qkv, void* kcache, void* vcache, int batch, int hq, int hkv, int head_dim, int max_ctx, int pos,
                    float theta, cudaStream_t stream);

// How many pieces the context is cut into (more CTAs than SMs, at least 64 positions each).
int decode_attention_splits(int batch, int hkv, int ctx, int sm_count);
// Bytes of workspace for `splits` pieces; must be zero before the first use (the kernel leaves its
// counters at zero again).
size_t decode_attention_workspace_bytes(int batch, int hq, int hkv, int splits);
// out[batch, hq * head_dim] = softmax(q k^T / sqrt(head_dim)) v over positions [0, ctx) of the caches; q row b
// starts at q + b * q_row_stride elements, head j at + j * head_dim (the layout rope_kv_append leaves).
void decode_attention(DType t, const void* q, int q_row_stride, const void* kcache, const void* vcache, void* out, void* workspace,
                      int batch, int hq, int hkv, int head_dim, int max_ctx, int ctx, int splits, cudaStream_t stream);

// res_out = x + residual ; out = RMSNorm(res_out) * gamma, row by row ([rows, hidden], 16-byte aligned).  The local
// half of "all-reduce, then residual add and RMSNorm" when the all-reduce is too large for the one-shot fused kernel.
void add_rmsnorm(DType t, const void* x, const void* residual, const void* gamma, void* out, void* res_out, int64_t rows, int hidden,
                 float eps, cudaStream_t stream);

// act[rows, ffn] = silu(gate_up[:, :ffn]) * gate_up[:, ffn:]
void silu_mul(DType t, const void* gate_up, void* act, int64_t rows, int ffn, int sm_count, cudaStream_t stream);

}  // namespace b200ipc
