// Row-parallel linear layer fused with its all-reduce and what follows it:
//
//     Y = sum over ranks r of  X_r[M, K] . W_r[N, K]^T          (each rank holds a K-slice)
//     res_out = Y + residual ;  out = RMSNorm(res_out) * gamma   (or out = Y without the norm)
//
// in ONE kernel per rank.  The GEMM runs on the 5th-generation tensor cores: TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast) streams tiles of X and BN x 64 tiles
// of W into a shared-memory ring; one elected thread issues tcgen05.mma (M = 128, N = BN,
// K = 16) into a double-buffered fp32 accumulator in tensor memory; four epilogue warps read
// it back with tcgen05.ld.  The exchange comes in two forms:
//
//   reduce-scatter (any M):  the epilogue rounds each finished tile to 16 bit and stores it
//     straight into the memory of the rank that OWNS those rows (peer stores over NVLink), then
//     releases one flag per (source, tile, 32-row group) - the transfer of tile i overlaps the
//     math of tile i+1.  Six more warps of every CTA are the owner side and run AT THE SAME
//     TIME as the GEMM: they wait for the flags of an owned row, add the world partial copies
//     in rank order in fp32 (+ residual), and push the summed row and its 1/rms to every rank
//     (all-gather by peer stores).  Tiles are visited so that every owner's rows complete at an
//     even pace.  A delivery counter per rank tells when all owners are done; then every rank
//     normalises the rows locally (out = sum * 1/rms * gamma), so only ONE tensor crosses the
//     links in the all-gather.
//   one-shot (M <= 32, decode):  the epilogue keeps the rank's partial product in LOCAL memory
//     (one flag per column tile, device scope); the CTA that holds a row then runs the one-shot
//     flag-in-data exchange of fused/oneshot_fused.cuh on it without leaving the kernel: LL512
//     transactions to every peer (no fence, one NVLink hop), the world copies added in rank order,
//     + residual, RMSNorm.  No owner, no all-gather, no system-scope release on the critical path.
//
// Small M is a weight-streaming problem: the X stage of the ring shrinks to the rows that
// exist, and a stage holds several 64-column sub-tiles, so that every row of W contributes a
// longer contiguous run per stage.  Best of all is a weight PACKED once at load time
// (Communicator.pack_weight): [N/64][K/64 padded][64 rows][64 columns], every 64 x 64 block
// stored exactly as the 128-byte-swizzled shared-memory image the tensor core reads - a stage is
// then one contiguous bulk copy of 8 KiB per sub-tile, which is what HBM likes most (the
// [N, K] layout makes a tile 64 separate short runs, one DRAM page each).
// Every wait is bounded (time limit of the communicator); tensor memory is always returned.
//
// No counterpart in the reference.  Baseline: cuBLAS GEMM + NCCL all-reduce + a fused
// add/normalise kernel.
#pragma once

#include <cuda.h>

#include "../coll/bulk_kernels.cuh"
#include "../proto/dev_backend.cuh"
#include "oneshot_fused.cuh"

namespace b200ipc {

constexpr int kGemmBM = 128;
constexpr int kGemmBK = 64;        // 64 x 2 B = one 128-byte swizzle row
constexpr int kGemmThreads = 384;  // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue, warps 6-11: owner side
constexpr int kGemmOwnerWarps = 6;
constexpr int kGemmOwnerThreads = kGemmOwnerWarps * 32;
constexpr int kGemmModeReduceScatter = 0;
constexpr int kGemmModeOneShot = 1;
constexpr int kGemmOneShotMaxRows = 32;

struct GemmArArgs {
  KArgs k;
  alignas(64) CUtensorMap tma_a[kMaxRanks];  // X  [M, K], K contiguous
  alignas(64) CUtensorMap tma_b[kMaxRanks];  // W  [N, K], K contiguous (nn.Linear layout)
  const void* residual[kMaxRanks];           // [M, N] or nullptr
  const void* gamma[kMaxRanks];              // [N] or nullptr
  const void* w_packed[kMaxRanks];           // W in the tile-packed layout (see below), or nullptr: then tma_b is used
  int packed_kblocks;                        // 64-column blocks per 64-row block in the packed layout
  int M, N, K;
  int rows_per_rank;
  int a_box_rows;        // rows of X one TMA box brings in: 128, or fewer when M is small (the rest of the
                         // 128-row operand tile then holds other data, which only reaches accumulator rows >= M)
  int mode;              // kGemmModeReduceScatter / kGemmModeOneShot
  uint32_t done_target;  // value the local delivery counter reaches when all owners are done (reduce-scatter)
  uint32_t epoch;        // launch number of this kernel family on the communicator: the flag value
  float eps;
  int with_norm;         // 0: out = sum (+ residual if given); 1: RMSNorm as well
  int local_only;        // 1: no exchange at all, out = this rank's own product (decode-sized kernel only)
  int row_parts;         // decode-sized kernel with RMSNorm: CTAs that share one row in the exchange (1, 2, 4 or 8)
  // heap offsets (same on every rank)
  uint64_t landing_off;  // reduce-scatter: [world][rows_per_rank][N] partials from every source; one-shot: [M][N], this rank's own
  uint64_t flags_off;    // reduce-scatter: [world][m_tiles][n_tiles][4]; one-shot: [n_tiles]   uint32
  uint64_t inv_off;      // [M] fp32: 1/rms of every row, written by the row's owner
  uint64_t out_off;      // [M][N]
  uint64_t res_out_off;  // [M][N] (0 = not wanted)
};

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up (and tells the whole CTA through *abort_flag) when the communicator's time
// limit for one wait has passed.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint64_t timeout_ns) {
  uint64_t t0 = 0;
  for (uint32_t n = 0;; ++n) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((n & 1023u) == 1023u) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > timeout_ns) break;
    }
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion counted on an mbarrier.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld_32cols(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 16-bit
// elements) in the 128-byte swizzle TMA writes: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sw128_kmajor_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3ffffu) >> 4);  // start address, 16-byte units
  d |= uint64_t(1) << 16;                      // leading byte offset (unused for swizzled K-major)
  d |= uint64_t(1024 >> 4) << 32;              // stride byte offset between 8-row groups
  d |= uint64_t(1) << 46;                      // descriptor version of this architecture
  d |= uint64_t(2) << 61;                      // 128-byte swizzle
  return d;
}
// Instruction descriptor: 16-bit A and B (K-major), fp32 accumulate, M x N tile.
template <typename T>
__device__ __forceinline__ uint32_t make_idesc(int m, int n) {
  const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Phase time stamps of CTA 0 (global timer, ns), kept in the control region of the heap at
// kGemmTraceOff: [0] entry, [1] set-up done, [2] last TMA issued, [3] last MMA committed,
// [4] last epilogue tile stored, [5] tensor memory returned, [6] all deliveries seen,
// [7] exit, [8] / [9] before / after the flag release of the epilogue warp that holds rows 0..31,
// [10] one-shot: every tile of the local product is there.  Behind them, at +128 bytes, a ring of
// 16 (entry, exit) pairs indexed by the launch number: the spacing of consecutive launches.
// A debugging and tuning aid; costs a handful of timer reads by single threads.
constexpr size_t kGemmTraceOff = 1024;
__device__ __forceinline__ void gemm_trace(const RankView& me, const HeapLayout& lay, int slot) {
  if (blockIdx.x == 0)
    reinterpret_cast<unsigned long long*>(me.heap + lay.ctrl_off + kGemmTraceOff)[slot] = globaltimer_ns();
}

// Offsets (uint32 slots) next to the device-side sequence words in the control region.
constexpr int kGemmDoneTotalSlot = 3;   // device-side running total of expected deliveries (graph-captured launches)
constexpr int kGemmDoneSlot = 4;        // the delivery counter the owners' CTAs add to
constexpr int kGemmEpochSlot = 6;       // device-side running launch number (graph-captured launches)

// A stage of the ring holds KSUB sub-tiles of 64 columns (one 128-byte swizzle row each) of both
// operands: KSUB > 1 makes every row of W contribute KSUB x 128 contiguous bytes per stage, which is
// what a weight-streaming (small M) problem needs from HBM.
template <int BN, int STAGES, int A_ROWS, int KSUB = 1>
struct GemmSmem {
  // The X stages come first: with A_ROWS < 128 the tensor core reads past a sub-tile's rows into the
  // next ones (and, for the last one, into the W stages), never outside this structure.
  alignas(1024) unsigned char a[STAGES][KSUB][A_ROWS * kGemmBK * 2];
  alignas(1024) unsigned char b[STAGES][KSUB][BN * kGemmBK * 2];
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  alignas(16) unsigned char epi[4][32 * 128];  // transpose patch of each epilogue warp
  uint32_t tmem_base;
  int abort_flag;
  int owner_fail;
  int exchange_abort;
  float red[kGemmThreads / 32];
  float exchange_part[32];
};
static_assert(kGemmBM * kGemmBK * 2 <= 4 * 64 * kGemmBK * 2, "the W stages must cover what a short X stage leaves to read");

// Barrier among the owner warps only (warps 6..11); the GEMM warps never join it.
__device__ __forceinline__ void owner_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kGemmOwnerThreads) : "memory"); }

// m-tile visited at position j of the tile order.  When the m-tiles divide evenly over the ranks the
// order interleaves the owners (first tile of every owner, then the second, ...), so that every
// owner's rows complete at an even pace while the GEMM runs; otherwise it is the identity.
__device__ __forceinline__ int gemm_mtile_at(int j, int m_tiles, int world, int rows_per_rank) {
  if (world <= 1 || m_tiles % world != 0 || rows_per_rank % kGemmBM != 0) return j;
  const int per = m_tiles / world;
  return (j % world) * per + j / world;
}

// What a group of threads (`tid` of `nthr`) does for one row: the reduce-scatter owner's side
// (sum of the world landed copies) and the one-shot receiver's side (the same sum, from the
// one-shot landing zone).  A thread touches the same vectors in every pass, so no barrier is
// needed between the passes.
template <typename T>
struct RowCtx {
  const RankView* me;
  const HeapLayout* lay;
  const GemmArArgs* args;
  int slot;  // which of the launch's ranks this block row is
  uint32_t epoch;
  int m_tiles, n_tiles;
  int* fail;  // shared-memory flag of the thread group

  // LOCAL: the flag is raised by a CTA of this GPU (device-scope release): relaxed polls and ONE device-scope
  // fence once the value is there, instead of a system-scope acquire on every poll.
  template <bool LOCAL = false>
  __device__ bool poll_flag(const uint32_t* fp, int src, int nt, int site) const {
    uint32_t* abort_word = reinterpret_cast<uint32_t*>(me->heap + lay->ctrl_off + kCtrlAbortOff);
    uint32_t spins = 0;
    uint64_t t0 = 0;
    for (;;) {
      uint32_t seen;
      if constexpr (LOCAL) {
        seen = ld_volatile_u32(fp);
        if (seen == epoch) {
          asm volatile("fence.acq_rel.gpu;" ::: "memory");
          return true;
        }
      } else {
        seen = ld_acquire_sys_u32(fp);
      }
      if (seen == epoch) return true;
      if ((++spins & 0x3fu) == 0) {
        if (ld_volatile_u32(abort_word) != 0 || *reinterpret_cast<volatile int*>(fail)) {
          if (ld_volatile_u32(abort_word) != 0) note_aborted_by_peer(abort_word, me->status, me->rank, site);
          *fail = 1;
          return false;
        }
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > me->timeout_ns) {
          if (claim_status(abort_word, kTimeout)) {
            StatusBlock* sb = me->status;
            sb->rank = uint32_t(me->rank);
            sb->peer = uint32_t(src);
            sb->wire = blockIdx.x;
            sb->step = uint32_t(nt);
            sb->expected = epoch;
            sb->seen = seen;
            sb->where = uint32_t(site);
            __threadfence_system();
            sb->code = kTimeout;
            __threadfence_system();
          }
          for (int q = 0; q < me->world; ++q)  // own abort word included
            st_volatile_u32(reinterpret_cast<uint32_t*>(me->peer[q] + lay->ctrl_off + kCtrlAbortOff), 1u);
          *fail = 1;
          return false;
        }
      }
    }
  }

  // Reduce-scatter: bounded wait until every source rank has delivered every column tile of this
  // row's 32-row group.
  __device__ bool wait_row_flags(int row, int tid, int nthr) const {
    const int W = me->world;
    const int mt = row / kGemmBM;
    const int grp = (row % kGemmBM) / 32;
    bool ok = true;
    for (int f = tid; f < W * n_tiles && ok; f += nthr) {
      const int src = f / n_tiles, nt = f % n_tiles;
      const uint32_t* fp = reinterpret_cast<const uint32_t*>(me->heap + args->flags_off) +
                           ((size_t(src) * m_tiles + mt) * n_tiles + nt) * 4 + grp;
      ok = poll_flag(fp, src, nt, 21);
    }
    return ok;
  }
  // One-shot: bounded wait until every column tile of this rank's own partial product is in memory.
  __device__ bool wait_local_tiles(int tid, int nthr) const {
    const uint32_t* base = reinterpret_cast<const uint32_t*>(me->heap + args->flags_off);
    bool ok = true;
    for (int f = tid; f < n_tiles && ok; f += nthr) ok = poll_flag<true>(base + f, me->rank, f, 23);
    return ok;
  }

  // Where the summed row lives on every rank: res_out if the caller wants it, else out.
  __device__ size_t sum_off() const { return args->res_out_off ? args->res_out_off : args->out_off; }

  // Sum of the world partial copies of one row in rank order (+ residual), rounded; `copy0` is the
  // row's copy from source rank 0, the other sources are `src_stride` bytes apart.  The rounded row
  // goes to the summed-row buffer of every rank in `dest_mask` (bit q = rank q).  Returns this
  // thread's share of the sum of squares of the rounded values.
  __device__ float sum_row(const char* copy0, size_t src_stride, int row, int tid, int nthr, uint32_t dest_mask) const {
    constexpr int U = 4;
    const int W = me->world, N = args->N;
    const int nvec = N / 8;
    const uint16_t* residual = static_cast<const uint16_t*>(args->residual[slot]);
    const size_t row_off = sum_off() + size_t(row) * N * 2;
    float ss = 0.f;
    for (int v0 = tid; v0 < nvec; v0 += U * nthr) {
      float a[U][8];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int e = 0; e < 8; ++e) a[u][e] = 0.f;
      for (int src = 0; src < W; ++src) {
        const char* base = copy0 + size_t(src) * src_stride;
        uint4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = v0 + u * nthr;
          x[u] = v < nvec ? ld_volatile_u4(base + size_t(v) * 16) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) acc8_add<T>(a[u], x[u]);
      }
      if (residual) {
        uint4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = v0 + u * nthr;
          x[u] = v < nvec ? *reinterpret_cast<const uint4*>(residual + size_t(row) * N + size_t(v) * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) acc8_add<T>(a[u], x[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * nthr;
        if (v >= nvec) continue;
        const uint4 o = acc8_pack<T>(a[u]);
        for (int k = 0; k < W; ++k) {
          const int q = (me->rank + k) % W;
          if (dest_mask & (1u << q)) *reinterpret_cast<uint4*>(me->peer[q] + row_off + size_t(v) * 16) = o;
        }
        float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        acc8_add<T>(b, o);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += b[e] * b[e];
      }
    }
    return ss;
  }

  // out[row] = summed row * inv * gamma (or a plain copy without the norm); everything is local.
  __device__ void finish_row(int row, int tid, int nthr, float inv) const {
    constexpr int U = 4;
    const int N = args->N;
    const int nvec = N / 8;
    const char* src = me->heap + sum_off() + size_t(row) * N * 2;
    char* dst = me->heap + args->out_off + size_t(row) * N * 2;
    if (!args->with_norm && src == dst) return;
    const uint4* gamma = static_cast<const uint4*>(args->gamma[slot]);
    for (int v0 = tid; v0 < nvec; v0 += U * nthr) {
      uint4 x[U], g[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * nthr;
        x[u] = v < nvec ? ld_volatile_u4(src + size_t(v) * 16) : make_uint4(0, 0, 0, 0);
        g[u] = (args->with_norm && v < nvec) ? gamma[v] : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * nthr;
        if (v >= nvec) continue;
        uint4 y = x[u];
        if (args->with_norm) {
          const uint32_t xs[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
          const uint32_t gs[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
          uint32_t ys[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 xf = Cvt<T>::up(xs[e]);
            const float2 gf = Cvt<T>::up(gs[e]);
            ys[e] = Cvt<T>::down(xf.x * inv * gf.x, xf.y * inv * gf.y);
          }
          y = make_uint4(ys[0], ys[1], ys[2], ys[3]);
        }
        *reinterpret_cast<uint4*>(dst + size_t(v) * 16) = y;
      }
    }
  }
};

template <typename T, int BN, int STAGES, int A_ROWS, int KSUB>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_ar_kernel(const __grid_constant__ GemmArArgs args) {
  extern __shared__ unsigned char smem_raw[];
  using Smem = GemmSmem<BN, STAGES, A_ROWS, KSUB>;
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
  const int k_iters = (K + kGemmBK * KSUB - 1) / (kGemmBK * KSUB);  // columns past K read as zeros
  const int total_tiles = m_tiles * n_tiles;
  const int rpr = args.rows_per_rank;
  const bool oneshot = args.mode == kGemmModeOneShot;
  const uint64_t timeout_ns = me.timeout_ns;
  // Graph-captured launches: launch number and delivery total live on the device and
  // args.done_target then holds this launch's increment instead of an absolute value.
  uint32_t epoch = args.epoch;
  uint32_t done_target = args.done_target;
  if (me.seq_dev) {
    epoch += ld_volatile_u32(me.seq_dev + kGemmEpochSlot);
    done_target += ld_volatile_u32(me.seq_dev + kGemmDoneTotalSlot);
  }
  constexpr uint32_t kTmemCols = 2 * BN;
  const uint32_t stage_bytes = uint32_t(args.a_box_rows + BN) * kGemmBK * 2 * KSUB;
  const bool mute = (me.flags & kMuteSends) != 0;

  // ---- set-up ---------------------------------------------------------------------------
  if (threadIdx.x == 0) gemm_trace(me, lay, 0);
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 4);  // one arrival per epilogue warp
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

  RowCtx<T> rc;
  rc.me = &me;
  rc.lay = &lay;
  rc.args = &args;
  rc.slot = int(blockIdx.y);
  rc.epoch = epoch;
  rc.m_tiles = m_tiles;
  rc.n_tiles = n_tiles;
  rc.fail = &s.owner_fail;

  // ---- GEMM + exchange: four roles run side by side ---------------------------------------------
  if (warp == 0) {
    if (lane == 0) {
      const CUtensorMap* ta = &args.tma_a[blockIdx.y];
      const CUtensorMap* tb = &args.tma_b[blockIdx.y];
      const char* wp = static_cast<const char*>(args.w_packed[blockIdx.y]);
      uint32_t it = 0;
      for (int t = int(blockIdx.x); t < total_tiles && !*abort_flag; t += G) {
        const int mt = gemm_mtile_at(t / n_tiles, m_tiles, W, rpr), nt = t % n_tiles;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int st = int(it % STAGES);
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&s.empty[st], ph ^ 1u, abort_flag, timeout_ns)) break;
          mbar_expect_tx(&s.full[st], stage_bytes);
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub)
            tma_load_2d(s.a[st][sub], ta, &s.full[st], (kb * KSUB + sub) * kGemmBK, mt * kGemmBM);
          if (wp) {
            // packed W: block (row block, k block) is 8 KiB; the k blocks of one row block are adjacent
            constexpr uint32_t kBlk = 64 * kGemmBK * 2;
#pragma unroll
            for (int rb = 0; rb < BN / 64; ++rb) {
              const char* src = wp + (size_t(nt * (BN / 64) + rb) * size_t(args.packed_kblocks) + size_t(kb) * KSUB) * kBlk;
              if (BN == 64) {
                bulk_load(s.b[st][0], src, kBlk * KSUB, &s.full[st]);
              } else {
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub) bulk_load(s.b[st][sub] + rb * kBlk, src + sub * kBlk, kBlk, &s.full[st]);
              }
            }
          } else {
#pragma unroll
            for (int sub = 0; sub < KSUB; ++sub)
              tma_load_2d(s.b[st][sub], tb, &s.full[st], (kb * KSUB + sub) * kGemmBK, nt * BN);
          }
        }
      }
      gemm_trace(me, lay, 2);
      // copies in flight land in this CTA's shared memory: wait for the ones still pending
      for (uint32_t back = 0; back < uint32_t(STAGES) && back < it; ++back) {
        const uint32_t j = it - 1 - back;
        mbar_wait(&s.full[j % STAGES], (j / STAGES) & 1u, abort_flag, timeout_ns);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc<T>(kGemmBM, BN);
      uint32_t it = 0, tile_i = 0;
      for (int t = int(blockIdx.x); t < total_tiles && !*abort_flag; t += G, ++tile_i) {
        const uint32_t buf = tile_i & 1u;
        const uint32_t use = tile_i >> 1;  // how often this accumulator buffer has been used before
        if (!mbar_wait(&s.acc_empty[buf], (use & 1u) ^ 1u, abort_flag, timeout_ns)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        bool ok = true;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int st = int(it % STAGES);
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(&s.full[st], ph, abort_flag, timeout_ns)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const uint64_t da = make_sw128_kmajor_desc(smem_u32(s.a[st][sub]));
            const uint64_t db = make_sw128_kmajor_desc(smem_u32(s.b[st][sub]));
#pragma unroll
            for (int k = 0; k < kGemmBK / 16; ++k) {
              // advance 16 elements (32 bytes) along K inside the swizzle atom: +2 in 16-byte units
              umma_f16(d_tmem, da + uint64_t(2 * k), db + uint64_t(2 * k), idesc, (kb > 0 || sub > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(&s.empty[st]);  // the stage may be refilled once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(&s.acc_full[buf]);  // accumulator complete
      }
      gemm_trace(me, lay, 3);
    }
  } else if (warp < 6) {
    // epilogue warps 2..5: warp w may touch tensor-memory lanes 32 * (w % 4) .. + 31
    const int lane_group = warp & 3;
    uint32_t tile_i = 0;
    for (int t = int(blockIdx.x); t < total_tiles && !*abort_flag; t += G, ++tile_i) {
      const int mt = gemm_mtile_at(t / n_tiles, m_tiles, W, rpr), nt = t % n_tiles;
      const uint32_t buf = tile_i & 1u;
      const uint32_t use = tile_i >> 1;
      if (!mbar_wait(&s.acc_full[buf], use & 1u, abort_flag, timeout_ns)) break;
      tc_fence_after_sync();
      const int first_row = mt * kGemmBM + lane_group * 32;
      if (first_row < M) {
        // The accumulator comes out of tensor memory one row per lane.  Written like that, a warp
        // store would be 32 pieces of 16 bytes 2 N bytes apart - poison for NVLink.  So each 64-column
        // chunk is rounded, transposed through a swizzled 4 KiB shared-memory patch and stored with
        // eight lanes per row: every store instruction writes four full 128-byte lines.
        unsigned char* patch = s.epi[lane_group];
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
              const int chunk = 4 * h + v;  // 16-byte chunk of this lane's 128-byte row
              *reinterpret_cast<uint4*>(patch + lane * 128 + ((chunk ^ (lane & 7)) * 16)) = o;
            }
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int pr = it * 4 + (lane >> 3);  // row of the patch this lane stores
            const int chunk = lane & 7;
            const uint4 o = *reinterpret_cast<const uint4*>(patch + pr * 128 + ((chunk ^ (pr & 7)) * 16));
            const int row = first_row + pr;
            if (row < M && (oneshot || !mute)) {
              const size_t col = size_t(nt) * BN + size_t(c) + size_t(chunk) * 8;
              if (oneshot) {
                // the partial product stays here: [row][N]; the exchange that follows reads it
                *reinterpret_cast<uint4*>(me.heap + args.landing_off + (size_t(row) * size_t(N) + col) * 2) = o;
              } else {
                const int owner = row / rpr;
                char* dst = me.peer[owner] + args.landing_off +
                            ((size_t(rank) * rpr + size_t(row - owner * rpr)) * size_t(N) + col) * 2;
                *reinterpret_cast<uint4*>(dst) = o;
              }
            }
          }
          __syncwarp();  // the patch is rewritten by the next chunk
        }
      }
      // accumulator buffer free again
      tc_fence_before_sync();
      __syncwarp();  // also orders this warp's row stores before the flag stores below
      if (lane == 0) mbar_arrive(&s.acc_empty[buf]);
      if (lane_group == 0 && lane == 0) gemm_trace(me, lay, 8);
      if (first_row < M && oneshot) {
        // one local flag per column tile (rows 0..31 are all there is); device scope is enough, the
        // reader is another CTA of this kernel
        if (lane == 0) {
          uint32_t* f = reinterpret_cast<uint32_t*>(me.heap + args.flags_off) + nt;
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
        }
      } else if (first_row < M && !mute) {
        // st.release.sys orders this warp's row stores (made visible to the storing lane by the
        // __syncwarp above) before the flag; no separate fence
        {
          // one flag per (source, tile, 32-row group) on every owner that got rows from this warp:
          // no barrier between the epilogue warps is needed, each warp answers for its own rows
          int last_row = first_row + 31;
          if (last_row > M - 1) last_row = M - 1;
          const int q = first_row / rpr + lane;
          if (q <= last_row / rpr) {
            uint32_t* f = reinterpret_cast<uint32_t*>(me.peer[q] + args.flags_off) +
                          ((size_t(rank) * m_tiles + mt) * n_tiles + nt) * 4 + lane_group;
            st_release_sys_u32(f, epoch);
          }
        }
      }
      if (lane_group == 0 && lane == 0) gemm_trace(me, lay, 9);
    }
    if (threadIdx.x == 64) gemm_trace(me, lay, 4);
  } else if (oneshot) {
    // ---- one-shot: these warps have nothing to do until the exchange; they use the time to pull what the
    // exchange will read (residual row, gamma) into L2 and to warm the address translation of what it
    // will write, so that the first access after the GEMM is not a cold one -------------------------------
    if (args.with_norm && int(blockIdx.x) < M) {
      const int otid = int(threadIdx.x) - (kGemmThreads - kGemmOwnerThreads);
      const int per = (M + G - 1) / G;
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
  } else {
    // ---- owner side (warps 6..11), concurrent with the GEMM: one row at a time per CTA, in the order
    // in which the rows complete ----------------------------------------------------------------------
    const int otid = int(threadIdx.x) - (kGemmThreads - kGemmOwnerThreads);
    const int owarp = otid >> 5;
    const int row0 = rank * rpr;
    int nrows = M - row0;
    if (nrows > rpr) nrows = rpr;
    if (nrows < 0) nrows = 0;
    // owned rows in completion order: the m-tiles of this rank as the tile order visits them
    const int own_tiles = (nrows + kGemmBM - 1) / kGemmBM;
    const bool interleaved = gemm_mtile_at(1, m_tiles, W, rpr) != 1 || m_tiles <= 1;
    (void)interleaved;
    float* inv_all = nullptr;
    for (int i = int(blockIdx.x); i < nrows; i += G) {
      // position i of the owned rows -> row: rows are spread so that consecutive CTAs take rows of the
      // same 32-row group (their flags arrive together)
      const int row = row0 + i;
      (void)own_tiles;
      rc.wait_row_flags(row, otid, kGemmOwnerThreads);
      owner_bar_sync();
      if (s.owner_fail) break;
      const char* copy0 = me.heap + args.landing_off + size_t(i) * size_t(N) * 2;
      float ss = rc.sum_row(copy0, size_t(rpr) * size_t(N) * 2, row, otid, kGemmOwnerThreads, mute ? 0u : ((1u << W) - 1u));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) s.red[owarp] = ss;
      owner_bar_sync();
      if (otid < W && !mute) {
        float tot = 0.f;
        for (int w = 0; w < kGemmOwnerWarps; ++w) tot += s.red[w];
        const float inv = rsqrtf(tot / float(N) + args.eps);
        inv_all = reinterpret_cast<float*>(me.peer[otid] + args.inv_off);
        inv_all[row] = inv;
      }
      owner_bar_sync();  // s.red is reused by the next row
    }
  }

  // ---- everybody meets; tensor memory goes back --------------------------------------------------
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
  const int nthreads = int(blockDim.x);
  const int nwarps = nthreads >> 5;
  bool failed = s.owner_fail != 0;

  if (oneshot) {
    // ---- one-shot: the CTAs that hold rows exchange them with every rank (flag-in-data), add the world
    // copies, the residual, and normalise ------------------------------------------------------------
    if constexpr (A_ROWS <= kGemmOneShotMaxRows) {
      rc.wait_local_tiles(int(threadIdx.x), nthreads);  // every CTA takes a piece of the product
      __syncthreads();
      if (threadIdx.x == 0) gemm_trace(me, lay, 10);
      failed = s.owner_fail != 0;
      if (!failed) {
        FusedOperands op;
        op.in = me.heap + args.landing_off;
        op.out = me.heap + args.out_off;
        op.residual = args.residual[blockIdx.y];
        op.gamma = args.gamma[blockIdx.y];
        op.res_out = me.heap + args.res_out_off;
        op.nelems = uint64_t(M) * uint64_t(N);
        op.hidden = N;
        op.scale_or_eps = args.with_norm ? args.eps : 1.0f;
        float* part = s.exchange_part;
        int* ab = &s.exchange_abort;
        if (args.with_norm) {
          switch (W) {
            case 1: oneshot_fused_body<T, T, 1, kEpiNorm>(me, lay, op, part, ab, false); break;
            case 2: oneshot_fused_body<T, T, 2, kEpiNorm>(me, lay, op, part, ab, false); break;
            case 4: oneshot_fused_body<T, T, 4, kEpiNorm>(me, lay, op, part, ab, false); break;
            default: oneshot_fused_body<T, T, 8, kEpiNorm>(me, lay, op, part, ab, false); break;
          }
        } else {
          switch (W) {
            case 1: oneshot_fused_body<T, T, 1, kEpiScale>(me, lay, op, part, ab, false); break;
            case 2: oneshot_fused_body<T, T, 2, kEpiScale>(me, lay, op, part, ab, false); break;
            case 4: oneshot_fused_body<T, T, 4, kEpiScale>(me, lay, op, part, ab, false); break;
            default: oneshot_fused_body<T, T, 8, kEpiScale>(me, lay, op, part, ab, false); break;
          }
        }
      }
    }
    if (threadIdx.x == 0) gemm_trace(me, lay, 6);
  } else {
    // ---- reduce-scatter: tell everyone this CTA has delivered, wait for all deliveries, then
    // normalise a share of the rows locally ------------------------------------------------------------
    uint32_t* done = reinterpret_cast<uint32_t*>(me.heap + lay.ctrl_off + kCtrlSeqOff) + kGemmDoneSlot;
    if (threadIdx.x < uint32_t(W) && !mute && !failed) {
      // release semantics of the reduction order the CTA's pushes (synchronised by the barrier above) before it
      red_release_sys_add(reinterpret_cast<uint32_t*>(me.peer[threadIdx.x] + lay.ctrl_off + kCtrlSeqOff) + kGemmDoneSlot, 1u);
    }
    if (threadIdx.x == 0 && !failed) {
      uint32_t spins = 0;
      uint64_t t0 = 0;
      for (;;) {
        const uint32_t seen = ld_acquire_sys_u32(done);
        if (int32_t(seen - done_target) >= 0) break;
        if ((++spins & 0x3fu) == 0) {
          if (ld_volatile_u32(abort_word) != 0) {
            note_aborted_by_peer(abort_word, me.status, rank, 22);
            s.owner_fail = 1;
            break;
          }
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > timeout_ns) {
            st_volatile_u32(abort_word, 1u);
            if (claim_status(abort_word, kTimeout)) {
              StatusBlock* sb = me.status;
              sb->rank = uint32_t(rank);
              sb->peer = 0;
              sb->wire = blockIdx.x;
              sb->expected = done_target;
              sb->seen = seen;
              sb->where = 22;
              __threadfence_system();
              sb->code = kTimeout;
              __threadfence_system();
            }
            s.owner_fail = 1;
            break;
          }
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) gemm_trace(me, lay, 6);
    failed = s.owner_fail != 0;
    if (!failed && (args.with_norm || args.res_out_off != 0)) {
      const float* inv = reinterpret_cast<const float*>(me.heap + args.inv_off);
      for (int row = int(blockIdx.x); row < M; row += G) {
        float iv = 1.f;
        if (args.with_norm) iv = __uint_as_float(ld_volatile_u32(inv + row));
        rc.finish_row(row, int(threadIdx.x), nthreads, iv);
      }
    }
  }
  if (threadIdx.x == 0) gemm_trace(me, lay, 7);
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    unsigned long long* ring = reinterpret_cast<unsigned long long*>(me.heap + lay.ctrl_off + kGemmTraceOff + 128) + (epoch & 15u) * 2;
    ring[0] = reinterpret_cast<unsigned long long*>(me.heap + lay.ctrl_off + kGemmTraceOff)[0];
    ring[1] = globaltimer_ns();
  }
  if (me.seq_dev) {
    // the last CTA to leave advances the device-side launch number and delivery total
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(me.seq_dev + 1, 1u) == gridDim.x - 1) {
        me.seq_dev[1] = 0;
        me.seq_dev[0] += me.seq_step;  // the one-shot exchange used flag-in-data sequence numbers
        me.seq_dev[kGemmEpochSlot] += 1;
        me.seq_dev[kGemmDoneTotalSlot] += args.done_target;
        __threadfence();
      }
    }
  }
}

}  // namespace b200ipc
