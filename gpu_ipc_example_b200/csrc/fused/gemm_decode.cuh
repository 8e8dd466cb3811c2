// The row-parallel linear layer fused with its all-reduce (+ residual + RMSNorm) at DECODE sizes
// (M <= 32 rows): a weight-streaming problem, so everything is arranged around reading W once at
// the rate HBM delivers it.
//
//   * The operands are swapped: the tensor core's 128-row side is a tile of 128 rows of W, the
//     narrow side is the batch (padded to 32).  One tcgen05.mma (M = 128, N = 32, K = 16) then
//     consumes 4 KiB of W; with W on the narrow side (N = 64) an instruction consumes 2 KiB and the
//     instruction rate, not memory, bounds the stream.
//   * K is split so that the tiles x splits fill the GPU (N = 8192: 64 tiles x 2).  Every CTA adds
//     its fp32 accumulator into one fp32 copy of the product in LOCAL memory (red.global.add.f32)
//     and raises a flag per 32 rows of W (device scope).
//   * TMA (no multicast) brings W tiles [128 x 64] and X tiles [32 x 64] through a five-stage ring
//     of two 64-column sub-tiles; a weight packed by pack_weight comes as contiguous 8 KiB blocks.
//   * The exchange is the one-shot flag-in-data exchange of oneshot_fused.cuh, run in place by the
//     CTAs that hold rows once every flag is up: LL512 transactions to every peer (one NVLink hop,
//     no fence), world copies added in rank order, + residual, RMSNorm.  Reading the fp32 product
//     rounds it and leaves zeros behind for the next launch.
//
// Every wait is bounded; tensor memory is returned before anything waits on a peer.
// No counterpart in the reference.
#pragma once

#include "gemm_ar.cuh"

namespace b200ipc {

constexpr int kDecTileRows = 128;  // rows of W per tile: the tensor core's M
constexpr int kDecXRows = 32;      // batch rows, padded: the tensor core's N
constexpr int kDecKSub = 2;        // 64-column sub-tiles per stage
constexpr int kDecStages = 5;      // 5 x 2 x (16 KiB + 4 KiB) = 200 KiB

struct DecodeSmem {
  alignas(1024) unsigned char a[kDecStages][kDecKSub][kDecTileRows * kGemmBK * 2];  // W
  alignas(1024) unsigned char b[kDecStages][kDecKSub][kDecXRows * kGemmBK * 2];     // X
  uint64_t full[kDecStages];
  uint64_t empty[kDecStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int owner_fail;
  int exchange_abort;
  float exchange_part[32];
};

// Uses GemmArArgs: tma_a = X [M, K] with a 32-row box, tma_b = W [N, K] with a 128-row box (or w_packed),
// landing_off = the fp32 product [M][N], flags_off = uint32 [tiles * splits * 4], rows_per_rank = K splits.
template <typename T>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_decode_kernel(const __grid_constant__ GemmArArgs args) {
  extern __shared__ unsigned char smem_raw[];
  DecodeSmem& s = *reinterpret_cast<DecodeSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const RankView& me = args.k.v[blockIdx.y];
  const HeapLayout& lay = args.k.lay;
  const int W = args.local_only ? 1 : me.world;
  const int rank = me.rank;
  const int warp = int(threadIdx.x >> 5);
  const int lane = int(threadIdx.x & 31);
  const int G = int(gridDim.x);
  const int M = args.M, N = args.N, K = args.K;
  const int splits = args.rows_per_rank;
  const int tiles = N / kDecTileRows;
  const int units = tiles * splits;
  const int kb_total = (K + kGemmBK - 1) / kGemmBK;
  int kb_per = (kb_total + splits - 1) / splits;
  kb_per = (kb_per + kDecKSub - 1) / kDecKSub * kDecKSub;
  const uint64_t timeout_ns = me.timeout_ns;
  pdl_launch_dependents();  // the next kernel may set itself up (and prefetch its weights) while this one runs
  constexpr uint32_t kTmemCols = 2 * kDecXRows;
  constexpr uint32_t kSubBytes = uint32_t(kDecTileRows + kDecXRows) * kGemmBK * 2;

  if (threadIdx.x == 0) gemm_trace(me, lay, 0);
  if (threadIdx.x == 0) {
    for (int i = 0; i < kDecStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 4);
    }
    s.abort_flag = 0;
    s.owner_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = s.tmem_base;
  volatile int* abort_flag = &s.abort_flag;
  if (threadIdx.x == 0) gemm_trace(me, lay, 1);

  const CUtensorMap* tx = &args.tma_a[blockIdx.y];
  const CUtensorMap* tw = &args.tma_b[blockIdx.y];
  const char* wp = static_cast<const char*>(args.w_packed[blockIdx.y]);
  constexpr uint32_t kBlk = 64 * kGemmBK * 2;
  auto load_w = [&](int st, int sub, int tile, int kb) {
    if (wp) {
      for (int rb = 0; rb < kDecTileRows / 64; ++rb)
        bulk_load(s.a[st][sub] + rb * kBlk,
                  wp + (size_t(tile * (kDecTileRows / 64) + rb) * size_t(args.packed_kblocks) + size_t(kb)) * kBlk, kBlk, &s.full[st]);
    } else {
      tma_load_2d(s.a[st][sub], tw, &s.full[st], kb * kGemmBK, tile * kDecTileRows);
    }
  };
  // The weights do not depend on the kernel before this one: the producer fills the ring with the W halves of
  // its first stages before it waits for that kernel; the X halves follow after the wait.
  uint32_t npre = 0;
  if (warp == 0 && lane == 0 && int(blockIdx.x) < units) {
    const int u = int(blockIdx.x);
    const int tile = u / splits, ks = u % splits;
    const int kb0 = ks * kb_per;
    int kb1 = kb0 + kb_per;
    if (kb1 > kb_total) kb1 = kb_total;
    for (int kb = kb0; kb < kb1 && npre < uint32_t(kDecStages); kb += kDecKSub, ++npre) {
      const int nsub = (kb1 - kb) < kDecKSub ? (kb1 - kb) : kDecKSub;
      mbar_expect_tx(&s.full[npre], kSubBytes * uint32_t(nsub));
      for (int sub = 0; sub < nsub; ++sub) load_w(int(npre), sub, tile, kb + sub);
    }
  }
  pdl_wait();  // everything below may read what earlier kernels wrote (activations, flags, counters, the fp32 product)
  uint32_t epoch = args.epoch;
  if (me.seq_dev) epoch += ld_volatile_u32(me.seq_dev + kGemmEpochSlot);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int u = int(blockIdx.x); u < units && !*abort_flag; u += G) {
        const int tile = u / splits, ks = u % splits;
        const int kb0 = ks * kb_per;
        int kb1 = kb0 + kb_per;
        if (kb1 > kb_total) kb1 = kb_total;
        for (int kb = kb0; kb < kb1; kb += kDecKSub, ++it) {
          const int st = int(it % kDecStages);
          const uint32_t ph = (it / kDecStages) & 1u;
          const int nsub = (kb1 - kb) < kDecKSub ? (kb1 - kb) : kDecKSub;
          const bool w_done = it < npre;  // this stage's W halves are already on their way
          if (!w_done) {
            if (!mbar_wait(&s.empty[st], ph ^ 1u, abort_flag, timeout_ns)) break;
            mbar_expect_tx(&s.full[st], kSubBytes * uint32_t(nsub));
          }
          for (int sub = 0; sub < nsub; ++sub) {
            tma_load_2d(s.b[st][sub], tx, &s.full[st], (kb + sub) * kGemmBK, 0);
            if (!w_done) load_w(st, sub, tile, kb + sub);
          }
        }
      }
      gemm_trace(me, lay, 2);
      for (uint32_t back = 0; back < uint32_t(kDecStages) && back < it; ++back) {
        const uint32_t j = it - 1 - back;
        mbar_wait(&s.full[j % kDecStages], (j / kDecStages) & 1u, abort_flag, timeout_ns);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc<T>(kDecTileRows, kDecXRows);
      uint32_t it = 0, unit_i = 0;
      for (int u = int(blockIdx.x); u < units && !*abort_flag; u += G, ++unit_i) {
        const int ks = u % splits;
        const int kb0 = ks * kb_per;
        int kb1 = kb0 + kb_per;
        if (kb1 > kb_total) kb1 = kb_total;
        const uint32_t buf = unit_i & 1u;
        const uint32_t use = unit_i >> 1;
        if (!mbar_wait(&s.acc_empty[buf], (use & 1u) ^ 1u, abort_flag, timeout_ns)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kDecXRows;
        bool ok = true;
        bool first = true;
        for (int kb = kb0; kb < kb1; kb += kDecKSub, ++it) {
          const int st = int(it % kDecStages);
          const uint32_t ph = (it / kDecStages) & 1u;
          if (!mbar_wait(&s.full[st], ph, abort_flag, timeout_ns)) { ok = false; break; }
          tc_fence_after_sync();
          const int nsub = (kb1 - kb) < kDecKSub ? (kb1 - kb) : kDecKSub;
          for (int sub = 0; sub < nsub; ++sub) {
            const uint64_t da = make_sw128_kmajor_desc(smem_u32(s.a[st][sub]));
            const uint64_t db = make_sw128_kmajor_desc(smem_u32(s.b[st][sub]));
#pragma unroll
            for (int k = 0; k < kGemmBK / 16; ++k) {
              umma_f16(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, first ? 0u : 1u);
              first = false;
            }
          }
          umma_commit(&s.empty[st]);
        }
        if (!ok) break;
        umma_commit(&s.acc_full[buf]);
      }
      gemm_trace(me, lay, 3);
    }
  } else if (warp < 6) {
    // epilogue: lane = a row of W (an output column), registers = the batch rows
    const int lane_group = warp & 3;
    float* prod = reinterpret_cast<float*>(me.heap + args.landing_off);
    uint32_t* flags = reinterpret_cast<uint32_t*>(me.heap + args.flags_off);
    uint32_t unit_i = 0;
    for (int u = int(blockIdx.x); u < units && !*abort_flag; u += G, ++unit_i) {
      const int tile = u / splits;
      const uint32_t buf = unit_i & 1u;
      const uint32_t use = unit_i >> 1;
      if (!mbar_wait(&s.acc_full[buf], use & 1u, abort_flag, timeout_ns)) break;
      tc_fence_after_sync();
      uint32_t acc[32];
      tmem_ld_32cols(tmem_base + (uint32_t(lane_group * 32) << 16) + buf * kDecXRows, acc);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
      float* col = prod + size_t(tile) * kDecTileRows + size_t(lane_group) * 32 + size_t(lane);
#pragma unroll
      for (int m = 0; m < kDecXRows; ++m)
        if (m < M) asm volatile("red.global.add.f32 [%0], %1;" ::"l"(col + size_t(m) * N), "f"(__uint_as_float(acc[m])) : "memory");
      __syncwarp();  // the release below covers the whole warp's additions
      if (lane_group == 0 && lane == 0) gemm_trace(me, lay, 8);
      if (lane == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flags + size_t(u) * 4 + lane_group), "r"(epoch) : "memory");
      if (lane_group == 0 && lane == 0) gemm_trace(me, lay, 9);
    }
    if (threadIdx.x == 64) gemm_trace(me, lay, 4);
  } else {
    // these warps have nothing to do until the exchange: pull what it will read (residual, gamma) into L2
    // and warm the address translation of what it will write
    const int per = (M + G - 1) / G;
    if (args.with_norm && int(blockIdx.x) * per < M) {
      const int otid = int(threadIdx.x) - (kGemmThreads - kGemmOwnerThreads);
      const size_t row_bytes = size_t(N) * 2;
      for (int rr = 0; rr < per; ++rr) {
        const int row = int(blockIdx.x) * per + rr;
        if (row >= M) break;
        const char* res = static_cast<const char*>(args.residual[blockIdx.y]) + size_t(row) * row_bytes;
        const char* gam = static_cast<const char*>(args.gamma[blockIdx.y]);
        const char* o1 = me.heap + args.out_off + size_t(row) * row_bytes;
        const char* o2 = me.heap + args.res_out_off + size_t(row) * row_bytes;
        for (size_t b = size_t(otid) * 128; b < row_bytes; b += size_t(kGemmOwnerThreads) * 128) {
          // real loads, not prefetches: a prefetch that misses the address translation is dropped
          (void)ld_volatile_u32(res + b);
          (void)ld_volatile_u32(gam + b);
          (void)ld_volatile_u32(o1 + b);
          (void)ld_volatile_u32(o2 + b);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0) gemm_trace(me, lay, 5);
  uint32_t* abort_word = reinterpret_cast<uint32_t*>(me.heap + lay.ctrl_off + kCtrlAbortOff);
  if (*abort_flag) {
    if (threadIdx.x == 0) {
      st_volatile_u32(abort_word, 1u);
      if (claim_status(abort_word, kTimeout)) {
        StatusBlock* sb = me.status;
        sb->rank = uint32_t(rank);
        sb->peer = uint32_t(rank);
        sb->wire = blockIdx.x;
        sb->where = 20;  // a local pipeline wait (TMA / MMA / epilogue hand-over) gave up
        __threadfence_system();
        sb->code = kTimeout;
        __threadfence_system();
      }
    }
    return;
  }

  // ---- every share of the product is in memory: exchange, reduce, normalise ---------------------------
  {
    RowCtx<T> rc;
    rc.me = &me;
    rc.lay = &lay;
    rc.args = &args;
    rc.slot = int(blockIdx.y);
    rc.epoch = epoch;
    rc.m_tiles = 1;
    rc.n_tiles = units * 4;
    rc.fail = &s.owner_fail;
    rc.wait_local_tiles(int(threadIdx.x), int(blockDim.x));
    __syncthreads();
    if (threadIdx.x == 0) gemm_trace(me, lay, 10);
    if (s.owner_fail == 0) {
      FusedOperands op;
      op.in = me.heap + args.landing_off;
      op.out = me.heap + args.out_off;
      op.residual = args.residual[blockIdx.y];
      op.gamma = args.gamma[blockIdx.y];
      op.res_out = me.heap + args.res_out_off;
      op.nelems = uint64_t(M) * uint64_t(N);
      op.hidden = N;
      op.scale_or_eps = args.with_norm ? args.eps : 1.0f;
      op.trace = reinterpret_cast<unsigned long long*>(me.heap + lay.ctrl_off + kGemmTraceOff) + 11;
      op.row_parts = args.with_norm ? args.row_parts : 1;
      op.stat_scratch = reinterpret_cast<unsigned long long*>(me.heap + args.inv_off);
      op.stat_epoch = epoch;
      float* part = s.exchange_part;
      int* ab = &s.exchange_abort;
      if (args.with_norm) {
        switch (W) {
          case 1: oneshot_fused_body<T, T, 1, kEpiNorm, true>(me, lay, op, part, ab, false); break;
          case 2: oneshot_fused_body<T, T, 2, kEpiNorm, true>(me, lay, op, part, ab, false); break;
          case 4: oneshot_fused_body<T, T, 4, kEpiNorm, true>(me, lay, op, part, ab, false); break;
          default: oneshot_fused_body<T, T, 8, kEpiNorm, true>(me, lay, op, part, ab, false); break;
        }
      } else {
        switch (W) {
          case 1: oneshot_fused_body<T, T, 1, kEpiScale, true>(me, lay, op, part, ab, false); break;
          case 2: oneshot_fused_body<T, T, 2, kEpiScale, true>(me, lay, op, part, ab, false); break;
          case 4: oneshot_fused_body<T, T, 4, kEpiScale, true>(me, lay, op, part, ab, false); break;
          default: oneshot_fused_body<T, T, 8, kEpiScale, true>(me, lay, op, part, ab, false); break;
        }
      }
    }
  }
  if (threadIdx.x == 0) gemm_trace(me, lay, 6);
  if (threadIdx.x == 0) gemm_trace(me, lay, 7);
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    unsigned long long* ring = reinterpret_cast<unsigned long long*>(me.heap + lay.ctrl_off + kGemmTraceOff + 128) + (epoch & 15u) * 2;
    ring[0] = reinterpret_cast<unsigned long long*>(me.heap + lay.ctrl_off + kGemmTraceOff)[0];
    ring[1] = globaltimer_ns();
  }
  if (me.seq_dev) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(me.seq_dev + 1, 1u) == gridDim.x - 1) {
        me.seq_dev[1] = 0;
        me.seq_dev[0] += me.seq_step;
        me.seq_dev[kGemmEpochSlot] += 1;
        __threadfence();
      }
    }
  }
}

}  // namespace b200ipc
