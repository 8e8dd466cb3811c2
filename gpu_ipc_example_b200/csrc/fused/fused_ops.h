// Host entry points of the fused collectives (all-reduce + residual-add + RMSNorm,
// all-reduce + scale/cast, row-parallel GEMM + all-reduce).  No counterpart in the
// reference; they serve the tensor-parallel inference use it was written for
// (script/gpu_inference_test.py:29-45 all-reduces decode-sized activations).
#pragma once

#include "../coll/comm.h"

namespace b200ipc {

struct FusedNormPtrs {
  const void* x;         // [rows, hidden] partial activations of this rank
  const void* residual;  // [rows, hidden]
  const void* gamma;     // [hidden]
  void* out;             // [rows, hidden] normalised
  void* residual_out;    // [rows, hidden] sum + residual (may alias residual)
};

// out = RMSNorm(all_reduce(x) + residual) * gamma ; residual_out = all_reduce(x) + residual.
// One kernel, one NVLink hop.  hidden must be a multiple of 8.  ptrs holds nlocal() entries.
CollInfo fused_allreduce_residual_rmsnorm(Comm& comm, DType t, const FusedNormPtrs* ptrs, int64_t rows, int64_t hidden,
                                          float eps, int ctas, cudaStream_t stream);

// out = cast<tout>(all_reduce(in) * scale).
CollInfo fused_allreduce_scale_cast(Comm& comm, DType tin, DType tout, const void* const* ins, void* const* outs,
                                    size_t nelems, float scale, int ctas, cudaStream_t stream);

}  // namespace b200ipc

namespace b200ipc {

// Row-parallel linear layer fused with its all-reduce (and residual-add + RMSNorm): see gemm_ar.cuh.
struct GemmArPtrs {
  const void* x;         // [M, K] this rank's activation slice, K contiguous
  const void* w;         // [N, K] this rank's weight slice (nn.Linear layout), K contiguous; or, with packed_kblocks > 0,
                         // the same weight packed as [N/64][packed_kblocks][64][64] swizzled blocks (pack_weight)
  const void* residual;  // [M, N] or nullptr
  const void* gamma;     // [N] or nullptr
  void* out;             // [M, N] in the symmetric heap
  void* res_out;         // [M, N] in the symmetric heap, or nullptr
  void* workspace;       // gemm_ar_workspace() bytes in the symmetric heap, zeroed once before first use
  int packed_kblocks = 0;  // 0: w is [N, K]; else the number of 64-column blocks per row block of the packed w
};
struct GemmArWorkspace {
  size_t landing_bytes = 0;  // partial products landing here
  size_t flags_bytes = 0;    // one flag per (source, tile, row group)
  size_t inv_bytes = 0;      // 1/rms of every row, written by the row's owner
  size_t total() const { return landing_bytes + flags_bytes + inv_bytes; }
};
GemmArWorkspace gemm_ar_workspace(int world, int64_t M, int64_t N);
// local_only: no exchange, out = this rank's own x @ w^T (the weight-streaming kernel for M <= 32 rows as a plain
// GEMM: column-parallel projections of a decode step); needs M <= 32 and N a multiple of 128.
CollInfo fused_gemm_allreduce(Comm& comm, DType t, const GemmArPtrs* ptrs, int64_t M, int64_t N, int64_t K, float eps,
                              bool with_norm, int ctas, cudaStream_t stream, bool local_only = false);

// All-gather of row-sharded activations fused with the GEMM that consumes them: see ag_gemm.cuh.
struct AgGemmPtrs {
  const void* x_shard;  // [M / world, K] this rank's rows
  const void* w;        // [N_local, K] this rank's weight slice (nn.Linear layout)
  void* out;            // [M, N_local]
  void* workspace;      // 2 * M * K * 2 bytes in the symmetric heap (two gathered-input buffers)
};
CollInfo fused_allgather_gemm(Comm& comm, DType t, const AgGemmPtrs* ptrs, int64_t M, int64_t N, int64_t K, int ctas,
                              cudaStream_t stream);

}  // namespace b200ipc
