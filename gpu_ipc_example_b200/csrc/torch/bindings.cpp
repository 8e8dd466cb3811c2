// PyTorch binding: custom ops in the `b200ipc` namespace that run the
// collectives on the current CUDA stream of the tensors' device, plus plain
// pybind functions for communicator life-cycle and introspection.
//
// Capability parity: the reference's framework smoke test drives an all-reduce
// of fp16 activations through a torch process group (script/gpu_inference_test.py:
// 21-45); here the same call lands in this library's kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <sys/mman.h>
#include <unistd.h>

#include <map>
#include <memory>
#include <mutex>
#include <tuple>

#include "../mem/device_registry.h"
#include "../proto/wire_format.h"

#include "../bootstrap/unix_mesh.h"
#include "../coll/comm.h"
#include "../common/check.h"
#include "../fused/fused_ops.h"
#include "../model/decode_ops.h"

namespace {

using namespace b200ipc;

struct Entry {
  std::unique_ptr<UnixMesh> mesh;
  std::unique_ptr<Comm> comm;
};

std::mutex g_mu;
std::map<int64_t, Entry> g_comms;
int64_t g_next_id = 1;

Comm& get(int64_t id) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_comms.find(id);
  TORCH_CHECK(it != g_comms.end(), "b200ipc: unknown communicator id ", id);
  return *it->second.comm;
}

HeapBacking parse_backing(const std::string& s) {
  if (s == "auto") return HeapBacking::Auto;
  if (s == "vmm-fd" || s == "vmm") return HeapBacking::VmmFd;
  if (s == "cuda-ipc" || s == "ipc") return HeapBacking::CudaIpc;
  if (s == "host-shm" || s == "host") return HeapBacking::HostShm;
  TORCH_CHECK(false, "b200ipc: unknown backing '", s, "'");
}

CommOptions make_options(int64_t staging_bytes, bool nvls, int64_t timeout_ms, const std::string& backing,
                         bool device_seq, int64_t first_seq, int64_t max_ctas) {
  CommOptions o;
  o.heap.staging_bytes = size_t(staging_bytes);
  o.heap.nvls = nvls;
  o.heap.backing = parse_backing(backing);
  o.timeout_ms = uint64_t(timeout_ms);
  o.device_seq = device_seq;
  o.first_seq = uint32_t(first_seq);
  o.max_ctas = int(max_ctas);
  return o;
}

int64_t comm_create(int64_t rank, int64_t world, int64_t device, const std::string& job_id, int64_t instance,
                    int64_t staging_bytes, bool nvls, int64_t timeout_ms, const std::string& backing, bool device_seq,
                    int64_t first_seq, int64_t max_ctas, int64_t bootstrap_timeout_ms) {
  Entry e;
  MeshOptions mo;
  mo.job_id = job_id;
  mo.instance = int(instance);
  mo.timeout_ms = int(bootstrap_timeout_ms);
  e.mesh = std::make_unique<UnixMesh>(int(rank), int(world), mo);
  e.comm = Comm::create(*e.mesh, int(device),
                        make_options(staging_bytes, nvls, timeout_ms, backing, device_seq, first_seq, max_ctas));
  std::lock_guard<std::mutex> lk(g_mu);
  int64_t id = g_next_id++;
  g_comms[id] = std::move(e);
  return id;
}

int64_t comm_create_virtual(int64_t world, int64_t device, int64_t staging_bytes, int64_t timeout_ms, bool device_seq,
                            int64_t first_seq, int64_t max_ctas) {
  Entry e;
  e.comm = Comm::create_virtual(int(world), int(device),
                                make_options(staging_bytes, false, timeout_ms, "auto", device_seq, first_seq, max_ctas));
  std::lock_guard<std::mutex> lk(g_mu);
  int64_t id = g_next_id++;
  g_comms[id] = std::move(e);
  return id;
}

void comm_destroy(int64_t id) {
  Entry e;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_comms.find(id);
    if (it == g_comms.end()) return;
    e = std::move(it->second);
    g_comms.erase(it);
  }
  e.comm->finalize();
  e.comm.reset();
  e.mesh.reset();
}

DType dtype_of(const at::Tensor& t) {
  if (t.scalar_type() == at::kHalf) return DType::F16;
  if (t.scalar_type() == at::kBFloat16) return DType::BF16;
  TORCH_CHECK(false, "b200ipc: only float16 and bfloat16 tensors are supported, got ", t.scalar_type());
}

void check_tensors(Comm& c, const std::vector<at::Tensor>& ts, const char* what) {
  TORCH_CHECK(int(ts.size()) == c.nlocal(), "b200ipc: expected ", c.nlocal(), " ", what, " tensor(s), got ", ts.size());
  for (const auto& t : ts) {
    TORCH_CHECK(t.is_cuda() && t.get_device() == c.device(), "b200ipc: ", what, " must live on cuda:", c.device());
    TORCH_CHECK(t.is_contiguous(), "b200ipc: ", what, " must be contiguous");
  }
}

AlgoSpec algo_or_throw(const std::string& name, bool want_allgather) {
  AlgoSpec a;
  bool ag = false;
  TORCH_CHECK(parse_algo(name, &a, &ag), "b200ipc: unknown algorithm '", name, "'. Known: ", algo_names_help());
  if (a.automatic) return a;
  TORCH_CHECK(ag == want_allgather || a.sched == SchedKind::Bulk || a.sched == SchedKind::Nvls,
              "b200ipc: algorithm '", name, "' is for ", ag ? "all-gather" : "all-reduce");
  return a;
}

std::vector<int64_t> info_vec(const CollInfo& i) {
  return {int64_t(i.sched), int64_t(i.proto), i.ctas, i.warps, i.nwires, i.steps, int64_t(i.first_flag), i.launches,
          int64_t(i.staged)};
}

std::vector<int64_t> all_reduce(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, int64_t comm_id,
                                const std::string& algo, int64_t ctas, int64_t warps, int64_t flags) {
  Comm& c = get(comm_id);
  check_tensors(c, ins, "input");
  check_tensors(c, outs, "output");
  std::vector<const void*> ip;
  std::vector<void*> op;
  for (int i = 0; i < c.nlocal(); ++i) {
    TORCH_CHECK(ins[i].numel() == ins[0].numel() && outs[i].numel() == ins[0].numel(), "b200ipc: size mismatch");
    TORCH_CHECK(ins[i].scalar_type() == outs[i].scalar_type(), "b200ipc: dtype mismatch");
    ip.push_back(ins[i].data_ptr());
    op.push_back(outs[i].data_ptr());
  }
  c10::cuda::CUDAGuard guard(c.device());
  LaunchGeom g{int(ctas), int(warps)};
  CollInfo info = c.all_reduce(algo_or_throw(algo, false), dtype_of(ins[0]), ip.data(), op.data(), size_t(ins[0].numel()), g,
                               at::cuda::getCurrentCUDAStream(c.device()), uint32_t(flags));
  return info_vec(info);
}

std::vector<int64_t> all_gather(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, int64_t comm_id,
                                const std::string& algo, int64_t ctas, int64_t warps, int64_t flags) {
  Comm& c = get(comm_id);
  check_tensors(c, ins, "input");
  check_tensors(c, outs, "output");
  std::vector<const void*> ip;
  std::vector<void*> op;
  for (int i = 0; i < c.nlocal(); ++i) {
    TORCH_CHECK(outs[i].numel() == ins[i].numel() * c.world(), "b200ipc: output must hold world * input elements");
    ip.push_back(ins[i].data_ptr());
    op.push_back(outs[i].data_ptr());
  }
  c10::cuda::CUDAGuard guard(c.device());
  LaunchGeom g{int(ctas), int(warps)};
  CollInfo info = c.all_gather(algo_or_throw(algo, true), dtype_of(ins[0]), ip.data(), op.data(), size_t(ins[0].numel()), g,
                               at::cuda::getCurrentCUDAStream(c.device()), uint32_t(flags));
  return info_vec(info);
}

std::vector<int64_t> reduce_scatter(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, int64_t comm_id,
                                    const std::string& algo, int64_t ctas, int64_t flags) {
  Comm& c = get(comm_id);
  check_tensors(c, ins, "input");
  check_tensors(c, outs, "output");
  std::vector<const void*> ip;
  std::vector<void*> op;
  for (int i = 0; i < c.nlocal(); ++i) {
    TORCH_CHECK(ins[i].numel() == outs[i].numel() * c.world(), "b200ipc: input must hold world * output elements");
    ip.push_back(ins[i].data_ptr());
    op.push_back(outs[i].data_ptr());
  }
  c10::cuda::CUDAGuard guard(c.device());
  LaunchGeom g{int(ctas), 0};
  AlgoSpec a = algo_or_throw(algo, false);
  CollInfo info = c.reduce_scatter(a, dtype_of(ins[0]), ip.data(), op.data(), size_t(ins[0].numel()), g,
                                   at::cuda::getCurrentCUDAStream(c.device()), uint32_t(flags));
  return info_vec(info);
}

// In-place single-tensor form, the shape `dist.all_reduce(t)` has.
at::Tensor all_reduce_(at::Tensor t, int64_t comm_id, const std::string& algo) {
  all_reduce({t}, {t}, comm_id, algo, 0, 0, 0);
  return t;
}

at::Tensor sym_empty(int64_t comm_id, std::vector<int64_t> shape, at::ScalarType dtype, int64_t local) {
  Comm& c = get(comm_id);
  int64_t n = 1;
  for (int64_t s : shape) n *= s;
  size_t bytes = size_t(n) * c10::elementSize(dtype);
  size_t off;
  if (local == 0) {
    off = c.sym_alloc(bytes);
    // remember for the other local ranks of a virtual world
    c.set_last_sym_offset(off);
  } else {
    off = c.last_sym_offset();
  }
  auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, c.device());
  return at::from_blob(c.sym_ptr(off, int(local)), shape, opts);
}

std::vector<int64_t> fused_ar_rmsnorm(std::vector<at::Tensor> ins, std::vector<at::Tensor> residuals,
                                      std::vector<at::Tensor> gammas, std::vector<at::Tensor> outs,
                                      std::vector<at::Tensor> res_outs, double eps, int64_t comm_id, int64_t ctas) {
  Comm& c = get(comm_id);
  check_tensors(c, ins, "input");
  check_tensors(c, outs, "output");
  check_tensors(c, residuals, "residual");
  check_tensors(c, gammas, "gamma");
  check_tensors(c, res_outs, "residual output");
  TORCH_CHECK(ins[0].dim() == 2, "b200ipc: fused all-reduce + RMSNorm takes [rows, hidden] tensors");
  const int64_t rows = ins[0].size(0), hidden = ins[0].size(1);
  std::vector<FusedNormPtrs> p(size_t(c.nlocal()));
  for (int i = 0; i < c.nlocal(); ++i) {
    TORCH_CHECK(ins[i].sizes() == ins[0].sizes() && outs[i].sizes() == ins[0].sizes() &&
                    residuals[i].sizes() == ins[0].sizes() && res_outs[i].sizes() == ins[0].sizes() &&
                    gammas[i].numel() == hidden,
                "b200ipc: shape mismatch");
    p[size_t(i)] = {ins[i].data_ptr(), residuals[i].data_ptr(), gammas[i].data_ptr(), outs[i].data_ptr(),
                    res_outs[i].data_ptr()};
  }
  c10::cuda::CUDAGuard guard(c.device());
  CollInfo info = fused_allreduce_residual_rmsnorm(c, dtype_of(ins[0]), p.data(), rows, hidden, float(eps), int(ctas),
                                                   at::cuda::getCurrentCUDAStream(c.device()));
  return info_vec(info);
}

std::vector<int64_t> fused_ar_scale_cast(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, double scale,
                                         int64_t comm_id, int64_t ctas) {
  Comm& c = get(comm_id);
  check_tensors(c, ins, "input");
  check_tensors(c, outs, "output");
  std::vector<const void*> ip;
  std::vector<void*> op;
  for (int i = 0; i < c.nlocal(); ++i) {
    TORCH_CHECK(ins[i].numel() == outs[i].numel(), "b200ipc: size mismatch");
    ip.push_back(ins[i].data_ptr());
    op.push_back(outs[i].data_ptr());
  }
  c10::cuda::CUDAGuard guard(c.device());
  CollInfo info = fused_allreduce_scale_cast(c, dtype_of(ins[0]), dtype_of(outs[0]), ip.data(), op.data(),
                                             size_t(ins[0].numel()), float(scale), int(ctas),
                                             at::cuda::getCurrentCUDAStream(c.device()));
  return info_vec(info);
}

// Row-parallel linear + all-reduce (+ residual + RMSNorm).  xs: [M, K] per rank, ws: [N, K] per rank
// (nn.Linear layout); outs / res_outs / workspaces are symmetric tensors.  residuals / gammas /
// res_outs may be empty lists.
std::vector<int64_t> fused_gemm_ar(std::vector<at::Tensor> xs, std::vector<at::Tensor> ws, std::vector<at::Tensor> residuals,
                                   std::vector<at::Tensor> gammas, std::vector<at::Tensor> outs,
                                   std::vector<at::Tensor> res_outs, std::vector<at::Tensor> workspaces, double eps,
                                   bool with_norm, int64_t comm_id, int64_t ctas, bool local_only) {
  Comm& c = get(comm_id);
  check_tensors(c, xs, "x");
  check_tensors(c, ws, "weight");
  check_tensors(c, outs, "output");
  check_tensors(c, workspaces, "workspace");
  if (!residuals.empty()) check_tensors(c, residuals, "residual");
  if (!gammas.empty()) check_tensors(c, gammas, "gamma");
  if (!res_outs.empty()) check_tensors(c, res_outs, "residual output");
  // weight: [N, K], or packed by pack_weight as [N / 64, K blocks, 64, 64]
  const bool packed = ws[0].dim() == 4;
  TORCH_CHECK(xs[0].dim() == 2 && (ws[0].dim() == 2 || packed), "b200ipc: x must be [M, K] and weight [N, K] (or packed)");
  const int64_t M = xs[0].size(0), K = xs[0].size(1), N = packed ? ws[0].size(0) * 64 : ws[0].size(0);
  if (packed) {
    TORCH_CHECK(ws[0].size(2) == 64 && ws[0].size(3) == 64 && ws[0].size(1) * 64 >= K && ws[0].size(1) % 4 == 0,
                "b200ipc: packed weight must be [N / 64, K blocks, 64, 64] covering K");
  } else {
    TORCH_CHECK(ws[0].size(1) == K, "b200ipc: weight must be [N, K] with the same K as x");
  }
  GemmArWorkspace need = gemm_ar_workspace(c.world(), M, N);
  std::vector<GemmArPtrs> p(size_t(c.nlocal()));
  for (int i = 0; i < c.nlocal(); ++i) {
    TORCH_CHECK(xs[i].sizes() == xs[0].sizes() && ws[i].sizes() == ws[0].sizes() && outs[i].numel() == M * N,
                "b200ipc: shape mismatch between ranks");
    TORCH_CHECK(xs[i].scalar_type() == ws[i].scalar_type() && xs[i].scalar_type() == outs[i].scalar_type(), "b200ipc: dtype mismatch");
    TORCH_CHECK(size_t(workspaces[i].numel() * workspaces[i].element_size()) >= need.total(), "b200ipc: workspace too small, need ",
                need.total(), " bytes");
    p[size_t(i)].x = xs[i].data_ptr();
    p[size_t(i)].w = ws[i].data_ptr();
    p[size_t(i)].residual = residuals.empty() ? nullptr : residuals[i].data_ptr();
    p[size_t(i)].gamma = gammas.empty() ? nullptr : gammas[i].data_ptr();
    p[size_t(i)].out = outs[i].data_ptr();
    p[size_t(i)].res_out = res_outs.empty() ? nullptr : res_outs[i].data_ptr();
    p[size_t(i)].workspace = workspaces[i].data_ptr();
    p[size_t(i)].packed_kblocks = packed ? int(ws[i].size(1)) : 0;
  }
  c10::cuda::CUDAGuard guard(c.device());
  CollInfo info = fused_gemm_allreduce(c, dtype_of(xs[0]), p.data(), M, N, K, float(eps), with_norm, int(ctas),
                                       at::cuda::getCurrentCUDAStream(c.device()), local_only);
  return info_vec(info);
}

// All-gather of row-sharded activations + column-parallel linear.  xs: [M / world, K] per rank, ws: [N_local, K],
// outs: [M, N_local]; workspaces: symmetric tensors of at least 2 * M * K elements.
std::vector<int64_t> fused_ag_gemm(std::vector<at::Tensor> xs, std::vector<at::Tensor> ws, std::vector<at::Tensor> outs,
                                   std::vector<at::Tensor> workspaces, int64_t comm_id, int64_t ctas) {
  Comm& c = get(comm_id);
  check_tensors(c, xs, "x");
  check_tensors(c, ws, "weight");
  check_tensors(c, outs, "output");
  check_tensors(c, workspaces, "workspace");
  TORCH_CHECK(xs[0].dim() == 2 && ws[0].dim() == 2, "b200ipc: x must be [M / world, K] and weight [N, K]");
  const int64_t M = xs[0].size(0) * c.world(), K = xs[0].size(1), N = ws[0].size(0);
  TORCH_CHECK(ws[0].size(1) == K, "b200ipc: weight must be [N, K] with the same K as x");
  std::vector<AgGemmPtrs> p(size_t(c.nlocal()));
  for (int i = 0; i < c.nlocal(); ++i) {
    TORCH_CHECK(xs[i].sizes() == xs[0].sizes() && ws[i].sizes() == ws[0].sizes() && outs[i].numel() == M * N,
                "b200ipc: shape mismatch between ranks");
    TORCH_CHECK(xs[i].scalar_type() == ws[i].scalar_type() && xs[i].scalar_type() == outs[i].scalar_type(), "b200ipc: dtype mismatch");
    TORCH_CHECK(workspaces[i].numel() * workspaces[i].element_size() >= 2 * (M * K * 2 + 256), "b200ipc: workspace too small");
    p[size_t(i)] = {xs[i].data_ptr(), ws[i].data_ptr(), outs[i].data_ptr(), workspaces[i].data_ptr()};
  }
  c10::cuda::CUDAGuard guard(c.device());
  CollInfo info = fused_allgather_gemm(c, dtype_of(xs[0]), p.data(), M, N, K, int(ctas), at::cuda::getCurrentCUDAStream(c.device()));
  return info_vec(info);
}

// ---- decode-step kernels (model/decode_ops.cu) --------------------------------------------------------
int sm_count_of(int device) {
  int n = 0;
  B200_CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device));
  return n;
}

// qkv [B, (hq + 2 hkv) * D] (q rotated in place), caches [B, hkv, max_ctx, D] (k, v of `pos` written).
void rope_kv_append_op(at::Tensor qkv, at::Tensor kcache, at::Tensor vcache, int64_t hq, int64_t hkv, int64_t pos, double theta) {
  TORCH_CHECK(qkv.is_cuda() && qkv.is_contiguous() && kcache.is_contiguous() && vcache.is_contiguous() && kcache.dim() == 4,
              "b200ipc: rope_kv_append takes contiguous CUDA tensors, caches [B, hkv, max_ctx, D]");
  const int64_t B = qkv.size(0), D = kcache.size(3);
  TORCH_CHECK(qkv.size(1) == (hq + 2 * hkv) * D && kcache.size(0) == B && kcache.size(1) == hkv && vcache.sizes() == kcache.sizes(),
              "b200ipc: rope_kv_append shape mismatch");
  c10::cuda::CUDAGuard guard(qkv.device());
  rope_kv_append(dtype_of(qkv), qkv.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), int(B), int(hq), int(hkv), int(D),
                 int(kcache.size(2)), int(pos), float(theta), at::cuda::getCurrentCUDAStream(qkv.get_device()));
}

int64_t attention_splits(int64_t batch, int64_t hkv, int64_t ctx, int64_t device) {
  return decode_attention_splits(int(batch), int(hkv), int(ctx), sm_count_of(int(device)));
}
int64_t attention_workspace_bytes(int64_t batch, int64_t hq, int64_t hkv, int64_t splits) {
  return int64_t(decode_attention_workspace_bytes(int(batch), int(hq), int(hkv), int(splits)));
}

// q = the first hq * D columns of qkv [B, (hq + 2 hkv) * D]; returns [B, hq * D].
at::Tensor decode_attention_op(at::Tensor qkv, at::Tensor kcache, at::Tensor vcache, at::Tensor workspace, int64_t hq, int64_t hkv,
                               int64_t ctx, int64_t splits) {
  TORCH_CHECK(qkv.is_cuda() && qkv.is_contiguous() && kcache.is_contiguous() && vcache.is_contiguous() && kcache.dim() == 4,
              "b200ipc: decode_attention takes contiguous CUDA tensors, caches [B, hkv, max_ctx, D]");
  const int64_t B = qkv.size(0), D = kcache.size(3);
  TORCH_CHECK(int64_t(workspace.numel() * workspace.element_size()) >= attention_workspace_bytes(B, hq, hkv, splits),
              "b200ipc: attention workspace too small");
  at::Tensor out = at::empty({B, hq * D}, qkv.options());
  c10::cuda::CUDAGuard guard(qkv.device());
  decode_attention(dtype_of(qkv), qkv.data_ptr(), int(qkv.size(1)), kcache.data_ptr(), vcache.data_ptr(), out.data_ptr(),
                   workspace.data_ptr(), int(B), int(hq), int(hkv), int(D), int(kcache.size(2)), int(ctx), int(splits),
                   at::cuda::getCurrentCUDAStream(qkv.get_device()));
  return out;
}

// (RMSNorm(x + residual) * gamma, x + residual) for [rows, hidden] tensors
std::vector<at::Tensor> add_rmsnorm_op(at::Tensor x, at::Tensor residual, at::Tensor gamma, double eps) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && residual.is_contiguous() && gamma.is_contiguous() && x.dim() == 2 &&
                  residual.sizes() == x.sizes() && gamma.numel() == x.size(1) && x.size(1) % 8 == 0,
              "b200ipc: add_rmsnorm takes contiguous [rows, hidden] tensors, hidden a multiple of 8");
  at::Tensor out = at::empty_like(x), res_out = at::empty_like(x);
  c10::cuda::CUDAGuard guard(x.device());
  add_rmsnorm(dtype_of(x), x.data_ptr(), residual.data_ptr(), gamma.data_ptr(), out.data_ptr(), res_out.data_ptr(), x.size(0),
              int(x.size(1)), float(eps), at::cuda::getCurrentCUDAStream(x.get_device()));
  return {out, res_out};
}

// [rows, 2 F] -> [rows, F]: silu(first half) * second half
at::Tensor silu_mul_op(at::Tensor gate_up) {
  TORCH_CHECK(gate_up.is_cuda() && gate_up.is_contiguous() && gate_up.dim() == 2 && gate_up.size(1) % 16 == 0,
              "b200ipc: silu_mul takes a contiguous [rows, 2 F] CUDA tensor, F a multiple of 8");
  const int64_t rows = gate_up.size(0), F = gate_up.size(1) / 2;
  at::Tensor act = at::empty({rows, F}, gate_up.options());
  c10::cuda::CUDAGuard guard(gate_up.device());
  silu_mul(dtype_of(gate_up), gate_up.data_ptr(), act.data_ptr(), rows, int(F), sm_count_of(gate_up.get_device()),
           at::cuda::getCurrentCUDAStream(gate_up.get_device()));
  return act;
}

int64_t gemm_ar_workspace_bytes(int64_t world, int64_t M, int64_t N) { return int64_t(gemm_ar_workspace(int(world), M, N).total()); }

}  // namespace

TORCH_LIBRARY(b200ipc, m) {
  m.def("fused_ag_gemm(Tensor[] xs, Tensor[] ws, Tensor[] outs, Tensor[] workspaces, int comm, int ctas) -> int[]", &fused_ag_gemm);
  m.def(
      "fused_gemm_ar(Tensor[] xs, Tensor[] ws, Tensor[] residuals, Tensor[] gammas, Tensor[] outs, Tensor[] res_outs, "
      "Tensor[] workspaces, float eps, bool with_norm, int comm, int ctas, bool local_only) -> int[]",
      &fused_gemm_ar);
  m.def("all_reduce(Tensor[] ins, Tensor[] outs, int comm, str algo, int ctas, int warps, int flags) -> int[]", &all_reduce);
  m.def("all_gather(Tensor[] ins, Tensor[] outs, int comm, str algo, int ctas, int warps, int flags) -> int[]", &all_gather);
  m.def("reduce_scatter(Tensor[] ins, Tensor[] outs, int comm, str algo, int ctas, int flags) -> int[]", &reduce_scatter);
  m.def("all_reduce_(Tensor(a!) t, int comm, str algo) -> Tensor(a!)", &all_reduce_);
  m.def(
      "fused_ar_rmsnorm(Tensor[] ins, Tensor[] residuals, Tensor[] gammas, Tensor[] outs, Tensor[] res_outs, float eps, "
      "int comm, int ctas) -> int[]",
      &fused_ar_rmsnorm);
  m.def("fused_ar_scale_cast(Tensor[] ins, Tensor[] outs, float scale, int comm, int ctas) -> int[]", &fused_ar_scale_cast);
  m.def("rope_kv_append(Tensor(a!) qkv, Tensor(b!) kcache, Tensor(c!) vcache, int hq, int hkv, int pos, float theta) -> ()", &rope_kv_append_op);
  m.def("decode_attention(Tensor qkv, Tensor kcache, Tensor vcache, Tensor(a!) workspace, int hq, int hkv, int ctx, int splits) -> Tensor",
        &decode_attention_op);
  m.def("silu_mul(Tensor gate_up) -> Tensor", &silu_mul_op);
  m.def("add_rmsnorm(Tensor x, Tensor residual, Tensor gamma, float eps) -> Tensor[]", &add_rmsnorm_op);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "b200ipc native extension";
  m.def("comm_create", &comm_create);
  m.def("comm_create_virtual", &comm_create_virtual);
  m.def("comm_destroy", &comm_destroy);
  m.def("sym_empty", &sym_empty);
  m.def("sym_free_all", [](int64_t id) { get(id).sym_free_all(); });
  m.def("world", [](int64_t id) { return get(id).world(); });
  m.def("nlocal", [](int64_t id) { return get(id).nlocal(); });
  m.def("rank", [](int64_t id, int64_t local) { return get(id).rank(int(local)); });
  m.def("has_nvls", [](int64_t id) { return get(id).has_nvls(); });
  m.def("nvls_note", [](int64_t id) { return get(id).heap(0).nvls_note(); });
  m.def("backing", [](int64_t id) { return std::string(backing_name(get(id).heap(0).backing())); });
  m.def("launches", [](int64_t id) { return get(id).launches(); });
  m.def("seq", [](int64_t id) { return int64_t(get(id).seq()); });
  m.def("set_seq", [](int64_t id, int64_t s) { get(id).set_seq(uint32_t(s)); });
  m.def("set_timeout_ms", [](int64_t id, int64_t ms) { get(id).set_timeout_ms(uint64_t(ms)); });
  m.def("set_thresholds", [](int64_t id, int64_t a, int64_t b) { get(id).set_thresholds(size_t(a), size_t(b)); });
  m.def("host_barrier", [](int64_t id) { get(id).host_barrier(); });
  m.def("reset", [](int64_t id) { get(id).reset(); });
  m.def("raise_if_failed", [](int64_t id) { get(id).raise_if_failed(); });
  m.def("status", [](int64_t id, int64_t local) {
    StatusBlock s = get(id).status(int(local));
    return std::vector<int64_t>{s.code, s.rank, s.peer, s.wire, s.step, s.expected, s.seen, s.where};
  });
  m.def("dump_heap", [](int64_t id, int64_t local, int64_t offset, int64_t bytes) {
    at::Tensor t = at::empty({bytes}, at::TensorOptions().dtype(at::kByte));
    get(id).heap(int(local)).dump(size_t(offset), size_t(bytes), t.data_ptr());
    return t;
  });
  m.def("set_safe_protos", [](int64_t id, bool on) { get(id).set_safe_protos(on); });
  m.def("safe_protos", [](int64_t id) { return get(id).safe_protos(); });
  m.def("set_trace_wires", [](int64_t id, bool on) { get(id).set_trace_wires(on); });
  m.def("trace_wires", [](int64_t id) { return get(id).trace_wires(); });
  // (offset of the trace ring inside the heap, number of records it holds, bytes per record)
  m.def("trace_ring", [](int64_t id) {
    const HeapLayout& l = get(id).heap(0).layout();
    return std::vector<int64_t>{int64_t(l.ctrl_off + kCtrlTraceOff), int64_t(kTraceEntries), int64_t(sizeof(TraceRecord))};
  });
  m.def("heap_layout", [](int64_t id) {
    const HeapLayout& l = get(id).heap(0).layout();
    return std::vector<int64_t>{int64_t(l.ctrl_off),     int64_t(l.half_off[0]),  int64_t(l.half_off[1]),
                                int64_t(l.half_bytes),   int64_t(l.oneshot_off),  int64_t(l.oneshot_bytes),
                                int64_t(l.staging_off),  int64_t(l.staging_bytes), int64_t(l.total_bytes)};
  });
  m.def("gemm_ar_workspace_bytes", &gemm_ar_workspace_bytes);
  m.def("attention_splits", &attention_splits);
  m.def("attention_workspace_bytes", &attention_workspace_bytes);
  m.def("algo_names", &algo_names_help);
  // Parses an algorithm name: (known, is_allgather, automatic, schedule, proto, direct).
  m.def("parse_algo", [](const std::string& name) {
    AlgoSpec a;
    bool ag = false;
    bool ok = parse_algo(name, &a, &ag);
    return std::make_tuple(ok, ag, a.automatic, std::string(sched_name(a.sched)), std::string(proto_name(a.proto)),
                           a.direct_allgather);
  });
  // Exercises the bootstrap mesh without a GPU: all-gathers a blob, passes a memfd
  // whose content is the sender's rank (SCM_RIGHTS), runs a barrier and a max-reduce.
  // Returns (gathered bytes, ranks read back through the received descriptors, max).
  m.def("mesh_selftest", [](int64_t rank, int64_t world, const std::string& job, int64_t instance, int64_t timeout_ms,
                            const std::string& blob) {
    MeshOptions mo;
    mo.job_id = job;
    mo.instance = int(instance);
    mo.timeout_ms = int(timeout_ms);
    UnixMesh mesh(int(rank), int(world), mo);
    std::string all(blob.size() * size_t(world), '\0');
    mesh.allgather(blob.data(), blob.size(), all.data());
    int fd = ::memfd_create("b200ipc-selftest", 0);
    B200_SYS_CHECK(fd);
    int32_t me = int32_t(rank);
    B200_SYS_CHECK(::write(fd, &me, sizeof(me)));
    std::vector<int> fds = mesh.allgather_fds(fd);
    ::close(fd);
    std::vector<int64_t> seen;
    for (int f : fds) {
      int32_t v = -1;
      B200_SYS_CHECK(::pread(f, &v, sizeof(v), 0));
      ::close(f);
      seen.push_back(v);
    }
    mesh.barrier();
    int64_t mx = mesh.allreduce_max(rank * 10);
    return std::make_tuple(py::bytes(all), seen, mx);
  });
  m.def("rank_env", []() {
    RankEnv e = rank_env_from_environment();
    return std::make_tuple(e.found, e.rank, e.world, e.local_rank, e.job_id);
  });
  m.def("device_for_rank", [](const std::string& list, int64_t rank, int64_t ndev) {
    return device_for_rank(list, int(rank), int(ndev));
  });
  m.def("describe_devices", &describe_devices);
  m.def("socket_name", [](const std::string& job, int64_t instance, int64_t rank) {
    MeshOptions mo;
    mo.job_id = job;
    mo.instance = int(instance);
    return UnixMesh::socket_name(mo, int(rank));
  });
}
