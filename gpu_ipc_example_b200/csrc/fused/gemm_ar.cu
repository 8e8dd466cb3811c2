#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <set>
#include <tuple>

#include "../common/check.h"
#include "../common/cu_driver.h"
#include "fused_ops.h"
#include "ag_gemm.cuh"
#include "gemm_ar.cuh"
#include "gemm_decode.cuh"

namespace b200ipc {
namespace {

constexpr int kStages256 = 4;   // 4 x (16 KiB + 32 KiB) = 192 KiB of the 227 KiB a CTA may use
constexpr int kStages128 = 6;   // 6 x (16 KiB + 16 KiB) = 192 KiB
constexpr int kStages64 = 8;    // 8 x (16 KiB +  8 KiB) = 192 KiB
constexpr int kStagesDecode = 16;  // 16 x (4 KiB + 8 KiB) = 192 KiB: M <= 32, the X stage holds 32 rows
constexpr int kDecodeRows = 32;
constexpr int kDecodeMaxSplits = 8;

template <typename T, int BN, int STAGES, int A_ROWS, int KSUB = 1>
const void* kernel_ptr() {
  return reinterpret_cast<const void*>(&gemm_ar_kernel<T, BN, STAGES, A_ROWS, KSUB>);
}

// Tensor maps depend only on (pointer, extents, box, type): weights and activation buffers are
// reused call after call, so encoding is done once per distinct operand.  The cache is bounded: when
// it is full the oldest entry makes room (never a wholesale clear in the middle of serving).
using MapKey = std::tuple<const void*, uint64_t, uint64_t, uint32_t, int>;
constexpr size_t kMaxCachedMaps = 4096;
std::mutex g_map_mu;
std::map<MapKey, CUtensorMap> g_maps;
std::deque<MapKey> g_map_order;
std::set<const void*> g_attr_done;

void encode_2d(CUtensorMap* map, DType t, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  const MapKey key(base, rows, cols, box_rows, int(t));
  {
    std::lock_guard<std::mutex> lk(g_map_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
      *map = it->second;
      return;
    }
  }
  B200_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "GEMM operands must be 16-byte aligned");
  B200_REQUIRE((cols * 2) % 16 == 0, "the K extent must be a multiple of 8 elements");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {uint32_t(kGemmBK), box_rows};
  cuuint32_t estr[2] = {1, 1};
  B200_CU_CHECK(cu().TensorMapEncodeTiled(map, t == DType::F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                          2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  std::lock_guard<std::mutex> lk(g_map_mu);
  if (g_maps.emplace(key, *map).second) {
    g_map_order.push_back(key);
    if (g_map_order.size() > kMaxCachedMaps) {
      g_maps.erase(g_map_order.front());
      g_map_order.pop_front();
    }
  }
}

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

// Which exchange a problem uses: one-shot for decode-sized M (every rank gets every partial, one NVLink
// hop), reduce-scatter + all-gather otherwise.  B200IPC_GEMM_MODE=rs|oneshot overrides (oneshot only
// where M allows it).
int gemm_mode_for(int64_t M, bool with_norm, bool has_residual) {
  // the one-shot form computes either the plain sum or sum + residual followed by RMSNorm
  int mode = (M <= kGemmOneShotMaxRows && with_norm == has_residual) ? kGemmModeOneShot : kGemmModeReduceScatter;
  if (const char* e = std::getenv("B200IPC_GEMM_MODE")) {
    if (std::strcmp(e, "rs") == 0) mode = kGemmModeReduceScatter;
  }
  return mode;
}

}  // namespace

GemmArWorkspace gemm_ar_workspace(int world, int64_t M, int64_t N) {
  GemmArWorkspace w;
  const int64_t rpr = (M + world - 1) / world;
  const int64_t m_tiles = (M + kGemmBM - 1) / kGemmBM;
  // room for either form of the exchange, so that the choice can change between calls
  const size_t rs_landing = size_t(world) * size_t(rpr) * size_t(N) * 2;
  const size_t os_landing = M <= kGemmOneShotMaxRows ? size_t(M) * size_t(N) * 4 : 0;  // the decode kernel keeps an fp32 product
  w.landing_bytes = up256(std::max(rs_landing, os_landing));
  const size_t rs_flags = size_t(world) * size_t(m_tiles) * size_t(N / 64) * 4 * sizeof(uint32_t);
  const size_t os_flags = size_t(N / 64) * 4 * kDecodeMaxSplits * sizeof(uint32_t);
  w.flags_bytes = up256(std::max(rs_flags, os_flags));
  // [M] fp32 (reduce-scatter form), or [M][8] 8-byte words: the row-statistic hand-over of the decode-sized form
  w.inv_bytes = up256(std::max(size_t(M) * sizeof(float), size_t(std::min<int64_t>(M, 32)) * 8 * sizeof(uint64_t)));
  return w;
}

// Decode sizes (M <= 32, N a multiple of 128): the swapped-operand, split-K kernel of gemm_decode.cuh.
static CollInfo fused_gemm_decode(Comm& comm, DType t, const GemmArPtrs* ptrs, int64_t M, int64_t N, int64_t K, float eps,
                                  bool with_norm, int ctas_req, cudaStream_t stream, bool local_only) {
  const int W = comm.world();
  const void* fn = t == DType::F16 ? reinterpret_cast<const void*>(&gemm_decode_kernel<__half>)
                                   : reinterpret_cast<const void*>(&gemm_decode_kernel<__nv_bfloat16>);
  const size_t smem = sizeof(DecodeSmem) + 1024;
  {
    std::lock_guard<std::mutex> lk(g_map_mu);
    if (!g_attr_done.count(fn)) {
      B200_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
      g_attr_done.insert(fn);
    }
  }
  int cap = comm.resident_ctas(reinterpret_cast<KernelFn>(const_cast<void*>(fn)), kGemmThreads, smem);
  B200_REQUIRE(cap >= 1, "GEMM kernel does not fit on the device");
  cap = std::min<int>(cap, kMaxOneShotWires / (kGemmThreads / 32));
  const int64_t tiles = N / kDecTileRows;
  const int64_t kb_total = (K + kGemmBK - 1) / kGemmBK;
  // split K until the tiles x splits fill the GPU (every split keeps at least two stages of work)
  int64_t splits = std::max<int64_t>(1, cap / tiles);
  splits = std::min<int64_t>(splits, std::min<int64_t>(kDecodeMaxSplits, std::max<int64_t>(1, kb_total / (2 * kDecKSub))));
  const int64_t units = tiles * splits;
  int ctas = ctas_req > 0 ? ctas_req : int(std::min<int64_t>(cap, std::max<int64_t>(units, M)));
  B200_REQUIRE(ctas <= cap, "requested " << ctas << " CTAs, only " << cap << " can run at once");

  GemmArArgs args;
  std::memset(&args, 0, sizeof(args));
  args.mode = kGemmModeOneShot;
  std::vector<const void*> ins(size_t(comm.nlocal()), nullptr);
  std::vector<void*> outs(size_t(comm.nlocal()), nullptr);
  comm.fill_views(&args.k, ins.data(), outs.data(), size_t(M * N), 0);
  const GemmArWorkspace ws = gemm_ar_workspace(W, M, N);
  size_t landing_off = SIZE_MAX, out_off = SIZE_MAX, res_off = 0;
  for (int i = 0; i < comm.nlocal(); ++i) {
    const GemmArPtrs& p = ptrs[i];
    const size_t lo = comm.sym_offset_of(p.workspace, i);
    const size_t oo = comm.sym_offset_of(p.out, i);
    const size_t ro = p.res_out ? comm.sym_offset_of(p.res_out, i) : 0;
    B200_REQUIRE(lo != SIZE_MAX && oo != SIZE_MAX && ro != SIZE_MAX,
                 "workspace, out and res_out must be tensors from the symmetric heap (Communicator.empty)");
    if (i == 0) {
      landing_off = lo;
      out_off = oo;
      res_off = ro;
    }
    B200_REQUIRE(lo == landing_off && oo == out_off && ro == res_off, "symmetric tensors must sit at the same offset on every rank");
    B200_REQUIRE(lo % 256 == 0 && oo % 16 == 0 && ro % 16 == 0, "symmetric tensors must be 16-byte aligned");
    if (with_norm) B200_REQUIRE(p.gamma != nullptr && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0, "RMSNorm needs gamma and an aligned residual");
    encode_2d(&args.tma_a[i], t, p.x, uint64_t(M), uint64_t(K), uint32_t(kDecXRows));
    if (p.packed_kblocks > 0) {
      B200_REQUIRE(p.packed_kblocks == ptrs[0].packed_kblocks && int64_t(p.packed_kblocks) * 64 >= K,
                   "packed weight does not match K (pack it with Communicator.pack_weight)");
      args.w_packed[i] = p.w;
      args.packed_kblocks = p.packed_kblocks;
    } else {
      B200_REQUIRE(ptrs[0].packed_kblocks == 0, "either every rank's weight is packed or none");
      encode_2d(&args.tma_b[i], t, p.w, uint64_t(N), uint64_t(K), uint32_t(kDecTileRows));
    }
    args.residual[i] = p.residual;
    args.gamma[i] = p.gamma;
  }
  args.M = int(M);
  args.N = int(N);
  args.K = int(K);
  args.rows_per_rank = int(splits);
  args.eps = eps;
  args.with_norm = with_norm ? 1 : 0;
  args.local_only = local_only ? 1 : 0;
  // few rows, many CTAs: several CTAs share a row in the exchange, so that its transactions leave from many SMs
  int parts = 1;
  if (with_norm && !local_only && std::getenv("B200IPC_GEMM_ROW_PARTS_OFF") == nullptr)  // also without an exchange: 4x the CTAs per row
    while (parts < 8 && M * parts * 2 <= ctas && (N / 2) % (parts * 2 * 4) == 0) parts *= 2;
  args.row_parts = parts;
  args.landing_off = landing_off;
  args.flags_off = landing_off + ws.landing_bytes;
  args.inv_off = args.flags_off + ws.flags_bytes;
  args.out_off = out_off;
  args.res_out_off = res_off;
  args.epoch = comm.take_gemm_epoch();
  const int64_t per = (M + ctas - 1) / ctas;
  const int64_t steps = ceil_div64(ceil_div64(per * (N / 2), 120), kGemmThreads / 32);
  const uint32_t adv = uint32_t(steps + 1);
  const uint32_t first = comm.take_seq(adv);
  for (int i = 0; i < comm.nlocal(); ++i) {
    args.k.v[i].seq = first;
    args.k.v[i].seq_step = adv;
  }
  void* params[] = {&args};
  comm.launch_raw(fn, ctas, kGemmThreads, params, smem, stream, true);
  CollInfo info;
  info.sched = SchedKind::OneShot;
  info.proto = ProtoKind::LL512;
  info.ctas = ctas;
  info.warps = kGemmThreads / 32;
  info.nwires = ctas * kGemmThreads / 32;
  info.steps = (units + ctas - 1) / ctas;
  info.first_flag = args.epoch;
  info.launches = 1;
  return info;
}

CollInfo fused_gemm_allreduce(Comm& comm, DType t, const GemmArPtrs* ptrs, int64_t M, int64_t N, int64_t K, float eps,
                              bool with_norm, int ctas_req, cudaStream_t stream, bool local_only) {
  const int W = comm.world();
  B200_REQUIRE(M > 0 && N > 0 && K > 0, "empty GEMM");
  B200_REQUIRE(N % 64 == 0, "N must be a multiple of 64");
  B200_REQUIRE(K % 8 == 0, "K must be a multiple of 8");
  B200_REQUIRE(W == 1 || W == 2 || W == 4 || W == 8, "world size must be 1, 2, 4 or 8");
  B200_CUDA_CHECK(cudaSetDevice(comm.device()));
  const int mode = gemm_mode_for(M, with_norm, ptrs[0].residual != nullptr && ptrs[0].res_out != nullptr);
  if (local_only) {
    B200_REQUIRE(M <= kDecXRows && N % kDecTileRows == 0 && !with_norm && ptrs[0].residual == nullptr,
                 "the local (no exchange) form takes M <= " << kDecXRows << " rows, N a multiple of " << kDecTileRows
                                                           << ", no residual and no norm");
    return fused_gemm_decode(comm, t, ptrs, M, N, K, eps, false, ctas_req, stream, true);
  }
  if (mode == kGemmModeOneShot && N % kDecTileRows == 0 && std::getenv("B200IPC_GEMM_NO_SWAP") == nullptr)
    return fused_gemm_decode(comm, t, ptrs, M, N, K, eps, with_norm, ctas_req, stream, false);
  // Tile width: narrow tiles give small-M problems enough CTAs to stream the weight; wide tiles
  // cut the operand traffic per FLOP for large M.
  int BN = (M <= 128 || N % 128 != 0) ? 64 : ((M >= 512 && N % 256 == 0) ? 256 : 128);
  if (const char* e = std::getenv("B200IPC_GEMM_BN")) {  // experiments: force the tile width
    const int v = std::atoi(e);
    if ((v == 64 || v == 128 || v == 256) && N % v == 0) BN = v;
  }
  const bool decode = BN == 64 && M <= kDecodeRows;  // short X stage, deep ring
  const void* fn;
  size_t smem;
  const bool h = t == DType::F16;
  if (decode) {
    // sub-tiles per stage (contiguous bytes per weight row and stage = 128 x this); the ring always holds 192 KiB
    int ksub = 4;
    if (const char* e = std::getenv("B200IPC_GEMM_KSUB")) ksub = std::atoi(e);
    if (ksub == 4) {
      fn = h ? kernel_ptr<__half, 64, kStagesDecode / 4, kDecodeRows, 4>() : kernel_ptr<__nv_bfloat16, 64, kStagesDecode / 4, kDecodeRows, 4>();
      smem = sizeof(GemmSmem<64, kStagesDecode / 4, kDecodeRows, 4>) + 1024;
    } else if (ksub == 1) {
      fn = h ? kernel_ptr<__half, 64, kStagesDecode, kDecodeRows, 1>() : kernel_ptr<__nv_bfloat16, 64, kStagesDecode, kDecodeRows, 1>();
      smem = sizeof(GemmSmem<64, kStagesDecode, kDecodeRows, 1>) + 1024;
    } else {
      fn = h ? kernel_ptr<__half, 64, kStagesDecode / 2, kDecodeRows, 2>() : kernel_ptr<__nv_bfloat16, 64, kStagesDecode / 2, kDecodeRows, 2>();
      smem = sizeof(GemmSmem<64, kStagesDecode / 2, kDecodeRows, 2>) + 1024;
    }
  } else if (BN == 64) {
    fn = h ? kernel_ptr<__half, 64, kStages64, kGemmBM>() : kernel_ptr<__nv_bfloat16, 64, kStages64, kGemmBM>();
    smem = sizeof(GemmSmem<64, kStages64, kGemmBM>) + 1024;
  } else if (BN == 128) {
    fn = h ? kernel_ptr<__half, 128, kStages128, kGemmBM>() : kernel_ptr<__nv_bfloat16, 128, kStages128, kGemmBM>();
    smem = sizeof(GemmSmem<128, kStages128, kGemmBM>) + 1024;
  } else {
    fn = h ? kernel_ptr<__half, 256, kStages256, kGemmBM>() : kernel_ptr<__nv_bfloat16, 256, kStages256, kGemmBM>();
    smem = sizeof(GemmSmem<256, kStages256, kGemmBM>) + 1024;
  }
  {
    std::lock_guard<std::mutex> lk(g_map_mu);
    if (!g_attr_done.count(fn)) {
      B200_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
      g_attr_done.insert(fn);
    }
  }

  const int64_t rpr = (M + W - 1) / W;
  const int64_t m_tiles = (M + kGemmBM - 1) / kGemmBM;
  const int64_t n_tiles = N / BN;
  const int64_t total_tiles = m_tiles * n_tiles;
  int cap = comm.resident_ctas(reinterpret_cast<KernelFn>(const_cast<void*>(fn)), kGemmThreads, smem);
  B200_REQUIRE(cap >= 1, "GEMM kernel does not fit on the device");
  // enough CTAs for the tiles, and for the rows of the phase that follows (one row per CTA at a time)
  const int64_t rows_after = mode == kGemmModeOneShot ? M : rpr;
  int ctas = ctas_req > 0 ? ctas_req : int(std::min<int64_t>(cap, std::max<int64_t>(total_tiles, std::min<int64_t>(rows_after, cap))));
  B200_REQUIRE(ctas <= cap, "requested " << ctas << " CTAs, only " << cap << " can run at once");

  int a_box = kGemmBM;
  if (M < kGemmBM) {
    a_box = 8;
    while (a_box < M) a_box *= 2;
  }
  GemmArArgs args;
  std::memset(&args, 0, sizeof(args));
  args.a_box_rows = a_box;
  args.mode = mode;
  std::vector<const void*> ins(size_t(comm.nlocal()), nullptr);
  std::vector<void*> outs(size_t(comm.nlocal()), nullptr);
  comm.fill_views(&args.k, ins.data(), outs.data(), size_t(M * N), 0);
  const GemmArWorkspace ws = gemm_ar_workspace(W, M, N);
  size_t landing_off = SIZE_MAX, out_off = SIZE_MAX, res_off = 0;
  for (int i = 0; i < comm.nlocal(); ++i) {
    const GemmArPtrs& p = ptrs[i];
    const size_t lo = comm.sym_offset_of(p.workspace, i);
    const size_t oo = comm.sym_offset_of(p.out, i);
    const size_t ro = p.res_out ? comm.sym_offset_of(p.res_out, i) : 0;
    B200_REQUIRE(lo != SIZE_MAX && oo != SIZE_MAX && ro != SIZE_MAX,
                 "workspace, out and res_out must be tensors from the symmetric heap (Communicator.empty)");
    if (i == 0) {
      landing_off = lo;
      out_off = oo;
      res_off = ro;
    }
    B200_REQUIRE(lo == landing_off && oo == out_off && ro == res_off, "symmetric tensors must sit at the same offset on every rank");
    B200_REQUIRE(lo % 256 == 0 && oo % 16 == 0 && ro % 16 == 0, "symmetric tensors must be 16-byte aligned");
    if (with_norm) B200_REQUIRE(p.gamma != nullptr, "RMSNorm needs gamma");
    encode_2d(&args.tma_a[i], t, p.x, uint64_t(M), uint64_t(K), uint32_t(a_box));
    if (p.packed_kblocks > 0) {
      B200_REQUIRE(p.packed_kblocks == ptrs[0].packed_kblocks && p.packed_kblocks % 4 == 0 && int64_t(p.packed_kblocks) * 64 >= K,
                   "packed weight does not match K (pack it with Communicator.pack_weight)");
      B200_REQUIRE((reinterpret_cast<uintptr_t>(p.w) & 15) == 0, "packed weight must be 16-byte aligned");
      args.w_packed[i] = p.w;
      args.packed_kblocks = p.packed_kblocks;
    } else {
      B200_REQUIRE(ptrs[0].packed_kblocks == 0, "either every rank's weight is packed or none");
      encode_2d(&args.tma_b[i], t, p.w, uint64_t(N), uint64_t(K), uint32_t(BN));
    }
    args.residual[i] = p.residual;
    args.gamma[i] = p.gamma;
  }
  args.M = int(M);
  args.N = int(N);
  args.K = int(K);
  args.rows_per_rank = int(rpr);
  args.eps = eps;
  args.with_norm = with_norm ? 1 : 0;
  args.landing_off = landing_off;
  args.flags_off = landing_off + ws.landing_bytes;
  args.inv_off = args.flags_off + ws.flags_bytes;
  args.out_off = out_off;
  args.res_out_off = res_off;
  args.epoch = comm.take_gemm_epoch();
  if (mode == kGemmModeReduceScatter) {
    const uint32_t deliveries = uint32_t(W) * uint32_t(ctas);
    args.done_target = comm.device_seq() ? deliveries : comm.take_done(deliveries);
  } else {
    // flag-in-data sequence numbers of the exchange: a CTA's warps share the transactions of its rows
    B200_REQUIRE(N % 8 == 0 && int64_t(ctas) * (kGemmThreads / 32) <= kMaxOneShotWires, "too many CTAs for the one-shot exchange");
    const int64_t per = (M + ctas - 1) / ctas;
    const int64_t steps = ceil_div64(ceil_div64(per * (N / 2), 120), kGemmThreads / 32);
    const uint32_t adv = uint32_t(steps + 1);
    const uint32_t first = comm.take_seq(adv);
    for (int i = 0; i < comm.nlocal(); ++i) {
      args.k.v[i].seq = first;
      args.k.v[i].seq_step = adv;
      B200_REQUIRE(!with_norm || (reinterpret_cast<uintptr_t>(ptrs[i].residual) & 15) == 0, "residual must be 16-byte aligned");
    }
  }

  void* params[] = {&args};
  comm.launch_raw(fn, ctas, kGemmThreads, params, smem, stream, true);

  CollInfo info;
  info.sched = mode == kGemmModeOneShot ? SchedKind::OneShot : SchedKind::Bulk;
  info.proto = ProtoKind::LL512;
  info.ctas = ctas;
  info.warps = kGemmThreads / 32;
  info.nwires = ctas * kGemmThreads / 32;
  info.steps = (total_tiles + ctas - 1) / ctas;
  info.first_flag = args.epoch;
  info.launches = 1;
  return info;
}

namespace {
template <typename T, int BN, int STAGES>
const void* ag_kernel_ptr() {
  return reinterpret_cast<const void*>(&ag_gemm_kernel<T, BN, STAGES>);
}
}  // namespace

CollInfo fused_allgather_gemm(Comm& comm, DType t, const AgGemmPtrs* ptrs, int64_t M, int64_t N, int64_t K, int ctas_req,
                              cudaStream_t stream) {
  const int W = comm.world();
  B200_REQUIRE(M > 0 && N > 0 && K > 0, "empty GEMM");
  B200_REQUIRE(N % 64 == 0 && K % 8 == 0, "N must be a multiple of 64 and K of 8");
  B200_REQUIRE(M % W == 0, "the rows of X must divide evenly over the ranks");
  B200_REQUIRE(!comm.device_seq(), "the all-gather + GEMM kernel keeps its counters on the host");
  B200_CUDA_CHECK(cudaSetDevice(comm.device()));
  int BN = (M <= 128 || N % 128 != 0) ? 64 : ((M >= 512 && N % 256 == 0) ? 256 : 128);
  if (const char* e = std::getenv("B200IPC_GEMM_BN")) {  // experiments: force the tile width
    const int v = std::atoi(e);
    if ((v == 64 || v == 128 || v == 256) && N % v == 0) BN = v;
  }
  const void* fn;
  size_t smem;
  const bool h = t == DType::F16;
  if (BN == 64) {
    fn = h ? ag_kernel_ptr<__half, 64, kStages64>() : ag_kernel_ptr<__nv_bfloat16, 64, kStages64>();
    smem = sizeof(GemmSmem<64, kStages64, kGemmBM>) + 1024;
  } else if (BN == 128) {
    fn = h ? ag_kernel_ptr<__half, 128, kStages128>() : ag_kernel_ptr<__nv_bfloat16, 128, kStages128>();
    smem = sizeof(GemmSmem<128, kStages128, kGemmBM>) + 1024;
  } else {
    fn = h ? ag_kernel_ptr<__half, 256, kStages256>() : ag_kernel_ptr<__nv_bfloat16, 256, kStages256>();
    smem = sizeof(GemmSmem<256, kStages256, kGemmBM>) + 1024;
  }
  {
    std::lock_guard<std::mutex> lk(g_map_mu);
    if (!g_attr_done.count(fn)) {
      B200_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
      g_attr_done.insert(fn);
    }
  }
  const int64_t m_tiles = (M + kGemmBM - 1) / kGemmBM;
  const int64_t total_tiles = m_tiles * (N / BN);
  int cap = comm.resident_ctas(reinterpret_cast<KernelFn>(const_cast<void*>(fn)), kGemmThreads, smem);
  B200_REQUIRE(cap >= 1, "GEMM kernel does not fit on the device");
  int ctas = ctas_req > 0 ? ctas_req : int(std::min<int64_t>(cap, total_tiles));
  B200_REQUIRE(ctas <= cap, "requested " << ctas << " CTAs, only " << cap << " can run at once");

  AgGemmArgs args;
  std::memset(&args, 0, sizeof(args));
  std::vector<const void*> ins(size_t(comm.nlocal()), nullptr);
  std::vector<void*> outs(size_t(comm.nlocal()), nullptr);
  comm.fill_views(&args.k, ins.data(), outs.data(), size_t(M * N), 0);
  int parity = 0;
  args.arrive_target = comm.take_arrivals(uint32_t(ctas), &parity);
  const size_t buf_bytes = (size_t(M) * size_t(K) * 2 + 255) / 256 * 256;
  size_t ws_off = SIZE_MAX;
  for (int i = 0; i < comm.nlocal(); ++i) {
    const AgGemmPtrs& p = ptrs[i];
    const size_t off = comm.sym_offset_of(p.workspace, i);
    B200_REQUIRE(off != SIZE_MAX && off % 256 == 0, "the workspace must be a tensor from the symmetric heap (Communicator.empty)");
    if (i == 0) ws_off = off;
    B200_REQUIRE(off == ws_off, "the workspace must sit at the same offset on every rank");
    B200_REQUIRE((reinterpret_cast<uintptr_t>(p.x_shard) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0,
                 "x and out must be 16-byte aligned");
    const size_t xfull_off = ws_off + size_t(parity) * buf_bytes;
    encode_2d(&args.tma_a[i], t, comm.sym_ptr(xfull_off, i), uint64_t(M), uint64_t(K), kGemmBM);
    encode_2d(&args.tma_b[i], t, p.w, uint64_t(N), uint64_t(K), uint32_t(BN));
    args.x_shard[i] = p.x_shard;
    args.out[i] = p.out;
    args.xfull_off = xfull_off;
  }
  args.M = int(M);
  args.N = int(N);
  args.K = int(K);
  args.rows_per_rank = int(M / W);
  void* params[] = {&args};
  comm.launch_raw(fn, ctas, kGemmThreads, params, smem, stream, true);
  CollInfo info;
  info.sched = SchedKind::Bulk;
  info.proto = ProtoKind::LL512;
  info.ctas = ctas;
  info.warps = kGemmThreads / 32;
  info.nwires = ctas * kGemmThreads / 32;
  info.steps = (total_tiles + ctas - 1) / ctas;
  info.first_flag = args.arrive_target;
  info.launches = 1;
  return info;
}

}  // namespace b200ipc
