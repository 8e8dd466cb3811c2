// All-gather fused with the GEMM that consumes it (column-parallel linear layer with
// row-sharded activations):
//
//     Y_r[M, N_r] = concat over ranks q of X_q[M / world, K]  .  W_r[N_r, K]^T
//
// in ONE kernel per rank.  Every rank first pushes its shard of X into the same rows of a
// symmetric buffer on every rank (plain 16-byte peer stores, one release-add per CTA and
// destination), then runs the tcgen05/TMA GEMM of gemm_ar.cuh over that buffer.  Tiles are
// visited starting with the rank's own rows, and the TMA producer waits - bounded, on a
// counter in its own memory - only for the shards a tile actually needs, so the transfer of
// the remote shards overlaps the math on the rows that are already there.  The remote rows
// are always read from LOCAL memory by non-multicast TMA loads.
//
// The buffer is double-buffered by launch parity: a rank can be at most one launch ahead of
// a peer (it needs the peer's shard of the current launch to finish), so it never overwrites
// rows a peer still reads.  No counterpart in the reference.
#pragma once

#include "gemm_ar.cuh"

namespace b200ipc {

struct AgGemmArgs {
  KArgs k;
  alignas(64) CUtensorMap tma_a[kMaxRanks];  // gathered X [M, K] inside this rank's heap (this launch's buffer)
  alignas(64) CUtensorMap tma_b[kMaxRanks];  // W [N_local, K]
  const void* x_shard[kMaxRanks];            // [rows_per_rank, K] this rank's rows
  void* out[kMaxRanks];                      // [M, N_local]
  int M, N, K;
  int rows_per_rank;
  uint32_t arrive_target;  // value the per-source counters reach when a source's shard is complete
  uint64_t xfull_off;      // heap offset of this launch's gathered-X buffer
};

constexpr size_t kAgCounterOff = kCtrlSeqOff + 64;  // uint32 arrived[kMaxRanks] in the control region

template <typename T, int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1) ag_gemm_kernel(const __grid_constant__ AgGemmArgs args) {
  extern __shared__ unsigned char smem_raw[];
  using Smem = GemmSmem<BN, STAGES, kGemmBM>;
  Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  pdl_launch_dependents();
  pdl_wait();  // activations, flags and counters come from earlier kernels

  const RankView& me = args.k.v[blockIdx.y];
  const HeapLayout& lay = args.k.lay;
  const int W = me.world;
  const int rank = me.rank;
  const int warp = int(threadIdx.x >> 5);
  const int lane = int(threadIdx.x & 31);
  const int G = int(gridDim.x);
  const int M = args.M, N = args.N, K = args.K;
  const int m_tiles = (M + kGemmBM - 1) / kGemmBM;
  const int n_tiles = N / BN;
  const int k_iters = (K + kGemmBK - 1) / kGemmBK;
  const int total_tiles = m_tiles * n_tiles;
  const int rpr = args.rows_per_rank;
  constexpr uint32_t kTmemCols = 2 * BN;
  constexpr uint32_t kStageBytes = uint32_t(kGemmBM + BN) * kGemmBK * 2;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 4);
    }
    s.abort_flag = 0;
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

  // ---- phase 0: push my rows of X to every rank (all-gather by peer stores) -------------------
  {
    int my_rows = M - rank * rpr;
    if (my_rows > rpr) my_rows = rpr;
    if (my_rows < 0) my_rows = 0;
    const int64_t nvec = int64_t(my_rows) * K / 8;  // K % 8 == 0
    const uint4* src = static_cast<const uint4*>(args.x_shard[blockIdx.y]);
    const size_t dst_off = args.xfull_off + size_t(rank) * rpr * size_t(K) * 2;
    if (!(me.flags & kMuteSends)) {
      for (int64_t v = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += int64_t(G) * blockDim.x) {
        const uint4 x = src[v];
        for (int k = 0; k < W; ++k) {
          const int q = (rank + k) % W;
          *reinterpret_cast<uint4*>(me.peer[q] + dst_off + size_t(v) * 16) = x;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x < uint32_t(W) && !(me.flags & kMuteSends)) {
      // one arrival per CTA and destination; the release orders the CTA's stores before it
      red_release_sys_add(reinterpret_cast<uint32_t*>(me.peer[threadIdx.x] + lay.ctrl_off + kAgCounterOff) + rank, 1u);
    }
  }

  // ---- phase 1: GEMM over the gathered rows, own shard first --------------------------------------
  const int first_mt = (rank * rpr) / kGemmBM;
  if (warp == 0) {
    if (lane == 0) {
      const CUtensorMap* ta = &args.tma_a[blockIdx.y];
      const CUtensorMap* tb = &args.tma_b[blockIdx.y];
      const uint32_t* arrived = reinterpret_cast<const uint32_t*>(me.heap + lay.ctrl_off + kAgCounterOff);
      uint32_t* abort_word = reinterpret_cast<uint32_t*>(me.heap + lay.ctrl_off + kCtrlAbortOff);
      uint32_t it = 0;
      for (int t = int(blockIdx.x); t < total_tiles && !*abort_flag; t += G) {
        const int mt = (t / n_tiles + first_mt) % m_tiles, nt = t % n_tiles;
        // shards this tile reads
        int last_row = mt * kGemmBM + kGemmBM - 1;
        if (last_row > M - 1) last_row = M - 1;
        bool ok = true;
        for (int q = (mt * kGemmBM) / rpr; q <= last_row / rpr && ok; ++q) {
          uint32_t spins = 0;
          uint64_t t0 = 0;
          for (;;) {
            const uint32_t seen = ld_acquire_sys_u32(arrived + q);
            if (int32_t(seen - args.arrive_target) >= 0) break;
            if ((++spins & 0x3fu) == 0) {
              if (ld_volatile_u32(abort_word) != 0) {
                note_aborted_by_peer(abort_word, me.status, rank, 30);
                ok = false;
                break;
              }
              const uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              else if (now - t0 > me.timeout_ns) {
                if (claim_status(abort_word, kTimeout)) {
                  StatusBlock* sb = me.status;
                  sb->rank = uint32_t(rank);
                  sb->peer = uint32_t(q);
                  sb->wire = blockIdx.x;
                  sb->expected = args.arrive_target;
                  sb->seen = seen;
                  sb->where = 30;
                  __threadfence_system();
                  sb->code = kTimeout;
                  __threadfence_system();
                }
                for (int p = 0; p < W; ++p)  // own abort word included
                  st_volatile_u32(reinterpret_cast<uint32_t*>(me.peer[p] + lay.ctrl_off + kCtrlAbortOff), 1u);
                ok = false;
                break;
              }
            }
          }
        }
        if (!ok) {
          *abort_flag = 1;
          break;
        }
        // the rows were written by ordinary stores (possibly from another GPU); TMA reads through
        // the asynchronous proxy
        asm volatile("fence.proxy.async;" ::: "memory");
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int st = int(it % STAGES);
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&s.empty[st], ph ^ 1u, abort_flag, me.timeout_ns)) break;
          mbar_expect_tx(&s.full[st], kStageBytes);
          tma_load_2d(s.a[st][0], ta, &s.full[st], kb * kGemmBK, mt * kGemmBM);
          tma_load_2d(s.b[st][0], tb, &s.full[st], kb * kGemmBK, nt * BN);
        }
      }
      for (uint32_t back = 0; back < uint32_t(STAGES) && back < it; ++back) {
        const uint32_t j = it - 1 - back;
        mbar_wait(&s.full[j % STAGES], (j / STAGES) & 1u, abort_flag, me.timeout_ns);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc<T>(kGemmBM, BN);
      uint32_t it = 0, tile_i = 0;
      for (int t = int(blockIdx.x); t < total_tiles && !*abort_flag; t += G, ++tile_i) {
        const uint32_t buf = tile_i & 1u;
        const uint32_t use = tile_i >> 1;
        if (!mbar_wait(&s.acc_empty[buf], (use & 1u) ^ 1u, abort_flag, me.timeout_ns)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        bool ok = true;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int st = int(it % STAGES);
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&s.full[st], ph, abort_flag, me.timeout_ns)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t da = make_sw128_kmajor_desc(smem_u32(s.a[st][0]));
          const uint64_t db = make_sw128_kmajor_desc(smem_u32(s.b[st][0]));
#pragma unroll
          for (int k = 0; k < kGemmBK / 16; ++k)
            umma_f16(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&s.empty[st]);
        }
        if (!ok) break;
        umma_commit(&s.acc_full[buf]);
      }
    }
  } else if (warp < 6) {
    const int lane_group = warp & 3;
    uint32_t tile_i = 0;
    unsigned char* patch = s.epi[lane_group];
    uint16_t* out = static_cast<uint16_t*>(args.out[blockIdx.y]);
    for (int t = int(blockIdx.x); t < total_tiles && !*abort_flag; t += G, ++tile_i) {
      const int mt = (t / n_tiles + first_mt) % m_tiles, nt = t % n_tiles;
      const uint32_t buf = tile_i & 1u;
      const uint32_t use = tile_i >> 1;
      if (!mbar_wait(&s.acc_full[buf], use & 1u, abort_flag, me.timeout_ns)) break;
      tc_fence_after_sync();
#pragma unroll 1
      for (int c = 0; c < BN; c += 64) {
        uint32_t acc[32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          tmem_ld_32cols(tmem_base + (uint32_t(lane_group * 32) << 16) + buf * BN + uint32_t(c + 32 * h), acc);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = Cvt<T>::down(__uint_as_float(acc[8 * v + 0]), __uint_as_float(acc[8 * v + 1]));
            o.y = Cvt<T>::down(__uint_as_float(acc[8 * v + 2]), __uint_as_float(acc[8 * v + 3]));
            o.z = Cvt<T>::down(__uint_as_float(acc[8 * v + 4]), __uint_as_float(acc[8 * v + 5]));
            o.w = Cvt<T>::down(__uint_as_float(acc[8 * v + 6]), __uint_as_float(acc[8 * v + 7]));
            const int chunk = 4 * h + v;
            *reinterpret_cast<uint4*>(patch + lane * 128 + ((chunk ^ (lane & 7)) * 16)) = o;
          }
        }
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int pr = it * 4 + (lane >> 3);
          const int chunk = lane & 7;
          const uint4 o = *reinterpret_cast<const uint4*>(patch + pr * 128 + ((chunk ^ (pr & 7)) * 16));
          const int row = mt * kGemmBM + lane_group * 32 + pr;
          if (row < M)
            *reinterpret_cast<uint4*>(out + size_t(row) * N + size_t(nt) * BN + size_t(c) + size_t(chunk) * 8) = o;
        }
        __syncwarp();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (*abort_flag && threadIdx.x == 0) {
    uint32_t* abort_word = reinterpret_cast<uint32_t*>(me.heap + lay.ctrl_off + kCtrlAbortOff);
    st_volatile_u32(abort_word, 1u);
    if (claim_status(abort_word, kTimeout)) {
      StatusBlock* sb = me.status;
      sb->rank = uint32_t(rank);
      sb->peer = uint32_t(rank);
      sb->wire = blockIdx.x;
      sb->where = 31;
      __threadfence_system();
      sb->code = kTimeout;
      __threadfence_system();
    }
  }
}

}  // namespace b200ipc
