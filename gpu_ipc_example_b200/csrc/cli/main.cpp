// Benchmark / verification driver.
//
// Keeps the reference CLI's letters (main.cpp:177-198): -n elements (K/M/G
// suffix), -g CTAs ("groups"), -w warps per CTA ("sub-groups"), -f first flag,
// -s SIMD width (a warp: 32), -v verify, -a algorithm, -i instance, -l device
// list, -p host-memory scratch.  Flow as there (main.cpp:47-168): run once;
// with -v compare against the CPU oracle; otherwise two more warm-ups, a host
// barrier and a timed run whose device time is printed per rank.  Additions:
// the maximum over ranks and bandwidths, a non-zero exit code on a mismatch,
// --sweep, bf16 or fp16 by option instead of a compile-time typedef, and three
// ways to get ranks: a launcher's environment (torchrun, mpirun, srun), --np N
// (fork here) or --virtual N (all ranks emulated on one GPU).
#include <getopt.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include "../bootstrap/unix_mesh.h"
#include "../coll/comm.h"
#include "../coll/oracle.h"
#include "../common/check.h"
#include "../mem/device_registry.h"
#include "../proto/wire_format.h"
#include "nccl_baseline.h"

using namespace b200ipc;

namespace {

struct Options {
  std::string nelems = "8M";
  int groups = 0;     // 0 = derive from the message size
  int subgroups = 0;  // 0 = derive
  uint32_t flag = 0xe00f100fu;
  int simd = 32;
  bool verify = false;
  std::string algo = "small";
  int instance = 0;
  std::string devices = "012345678";
  bool pcie = false;
  // additions
  std::string dtype = "half";
  bool out_of_place = false;
  int iters = 1;
  int np = 0;
  int virt = 0;
  bool nvls = false;
  bool ref_accum = false;
  std::string sweep;  // "lo:hi" log2 of the element count
  uint64_t timeout_ms = 2000;
  size_t staging_mb = 256;
  bool random = false;
  std::string backing = "auto";
  std::string baseline;  // "nccl": time NCCL instead of this library
  bool symmetric = false;
};

// "8M" -> 8 * 1024 * 1024 elements (main.cpp:17-34; a trailing B as in the default "8MB" is accepted).
size_t parse_nelems(const std::string& s) {
  size_t mult = 1;
  if (s.find('K') != std::string::npos || s.find('k') != std::string::npos) mult = 1024ull;
  else if (s.find('M') != std::string::npos || s.find('m') != std::string::npos) mult = 1024ull * 1024;
  else if (s.find('G') != std::string::npos || s.find('g') != std::string::npos) mult = 1024ull * 1024 * 1024;
  return std::stoull(s) * mult;
}

void usage() {
  std::printf(
      "b200ipc main - single-kernel all-reduce / all-gather over NVLink peer memory\n"
      "  -n, --nelems N      elements per rank, K/M/G suffix (default 8M)\n"
      "  -g, --groups G      CTAs per rank (default: from the message size)\n"
      "  -w, --subgroups W   warps per CTA (default: from the message size)\n"
      "  -f, --flag F        first sequence flag (default 0xe00f100f)\n"
      "  -s, --simd S        lanes per wire; only 32 exists on this hardware\n"
      "  -v, --verify        check against the CPU oracle instead of timing\n"
      "  -a, --algo NAME     %s\n"
      "  -i, --instance I    namespace for several jobs on one node\n"
      "  -l, --devices LIST  device per rank, one digit each or comma separated (default 012345678)\n"
      "  -p, --pcie          scratch in shared pinned host memory instead of device memory\n"
      "  -t, --dtype T       half | bf16 (default half)\n"
      "  -o, --out-of-place  write to a separate output buffer\n"
      "      --iters K       timed launches (default 1)\n"
      "      --np N          fork N ranks from this process\n"
      "      --virtual N     emulate N ranks on one GPU (one cooperative launch)\n"
      "      --nvls          set up the NVSwitch multicast mapping\n"
      "      --ref-accum     round to the element type after every add, like the reference\n"
      "      --random        N(0,1) / U(-1,1) data instead of the (i%%32)*(rank+1) pattern\n"
      "      --sweep LO:HI   time 2^LO .. 2^HI elements\n"
      "      --timeout-ms T  time limit of one device-side wait (default 2000)\n"
      "      --staging-mb M  staging region of the heap (default 256)\n"
      "      --backing B     auto | vmm-fd | cuda-ipc | host-shm\n"
      "      --symmetric     buffers inside the symmetric heap (zero-copy for bulk / nvls)\n"
      "      --baseline nccl time ncclAllReduce / ncclAllGather on the same buffers instead\n",
      algo_names_help().c_str());
}

bool parse(int argc, char** argv, Options* o) {
  static option longopts[] = {{"nelems", required_argument, nullptr, 'n'},
                              {"groups", required_argument, nullptr, 'g'},
                              {"subgroups", required_argument, nullptr, 'w'},
                              {"flag", required_argument, nullptr, 'f'},
                              {"simd", required_argument, nullptr, 's'},
                              {"verify", no_argument, nullptr, 'v'},
                              {"algo", required_argument, nullptr, 'a'},
                              {"instance", required_argument, nullptr, 'i'},
                              {"devices", required_argument, nullptr, 'l'},
                              {"pcie", no_argument, nullptr, 'p'},
                              {"dtype", required_argument, nullptr, 't'},
                              {"out-of-place", no_argument, nullptr, 'o'},
                              {"iters", required_argument, nullptr, 1000},
                              {"np", required_argument, nullptr, 1001},
                              {"virtual", required_argument, nullptr, 1002},
                              {"nvls", no_argument, nullptr, 1003},
                              {"ref-accum", no_argument, nullptr, 1004},
                              {"sweep", required_argument, nullptr, 1005},
                              {"timeout-ms", required_argument, nullptr, 1006},
                              {"staging-mb", required_argument, nullptr, 1007},
                              {"random", no_argument, nullptr, 1008},
                              {"backing", required_argument, nullptr, 1009},
                              {"baseline", required_argument, nullptr, 1010},
                              {"symmetric", no_argument, nullptr, 1011},
                              {"help", no_argument, nullptr, 'h'},
                              {nullptr, 0, nullptr, 0}};
  opterr = 0;  // unknown options are ignored, as in the reference (main.cpp:176)
  int c;
  while ((c = getopt_long(argc, argv, "n:g:w:f:s:va:i:l:pt:oh", longopts, nullptr)) != -1) {
    switch (c) {
      case 'n': o->nelems = optarg; break;
      case 'g': o->groups = std::atoi(optarg); break;
      case 'w': o->subgroups = std::atoi(optarg); break;
      case 'f': o->flag = uint32_t(std::strtoull(optarg, nullptr, 0)); break;
      case 's': o->simd = std::atoi(optarg); break;
      case 'v': o->verify = true; break;
      case 'a': o->algo = optarg; break;
      case 'i': o->instance = std::atoi(optarg); break;
      case 'l': o->devices = optarg; break;
      case 'p': o->pcie = true; break;
      case 't': o->dtype = optarg; break;
      case 'o': o->out_of_place = true; break;
      case 1000: o->iters = std::max(1, std::atoi(optarg)); break;
      case 1001: o->np = std::atoi(optarg); break;
      case 1002: o->virt = std::atoi(optarg); break;
      case 1003: o->nvls = true; break;
      case 1004: o->ref_accum = true; break;
      case 1005: o->sweep = optarg; break;
      case 1006: o->timeout_ms = std::strtoull(optarg, nullptr, 0); break;
      case 1007: o->staging_mb = std::strtoull(optarg, nullptr, 0); break;
      case 1008: o->random = true; break;
      case 1009: o->backing = optarg; break;
      case 1010: o->baseline = optarg; break;
      case 1011: o->symmetric = true; break;
      case 'h': usage(); return false;
      default: break;
    }
  }
  return true;
}

struct Buffers {
  std::vector<void*> in, out;  // device, one per local rank
};

struct RunResult {
  double ns_max = 0;    // slowest rank, mean over the timed launches
  double ns_local = 0;  // this process
  size_t mismatches = 0;
};

int run_rank(int rank, int world, const Options& opt, UnixMesh* mesh) {
  AlgoSpec algo;
  bool is_ag = false;
  if (!parse_algo(opt.algo, &algo, &is_ag)) {
    // with --baseline nccl the -a value only says which collective: anything naming "allgather" is one
    if (opt.baseline.empty()) {
      std::fprintf(stderr, "unknown algorithm '%s'\nknown: %s\n", opt.algo.c_str(), algo_names_help().c_str());
      return 2;
    }
    is_ag = opt.algo.find("allgather") != std::string::npos;
  }
  B200_REQUIRE(opt.simd == 32, "-s " << opt.simd << ": a wire is one warp of 32 lanes on this hardware");
  const DType dt = (opt.dtype == "bf16" || opt.dtype == "bfloat16") ? DType::BF16 : DType::F16;

  int ndev = 0;
  B200_CUDA_CHECK(cudaGetDeviceCount(&ndev));
  const bool virt = opt.virt > 0;
  const int device = device_for_rank(opt.devices, virt ? 0 : rank, ndev);
  B200_CUDA_CHECK(cudaSetDevice(device));

  std::vector<size_t> sizes;
  if (!opt.sweep.empty()) {
    int lo = 10, hi = 24;
    if (std::sscanf(opt.sweep.c_str(), "%d:%d", &lo, &hi) != 2) B200_REQUIRE(false, "--sweep wants LO:HI");
    for (int e = lo; e <= hi; ++e) sizes.push_back(size_t(1) << e);
    if (opt.iters == 1) const_cast<Options&>(opt).iters = 20;
  } else {
    sizes.push_back(parse_nelems(opt.nelems));
  }
  const size_t max_n = *std::max_element(sizes.begin(), sizes.end());
  const size_t in_elems = max_n;
  const size_t out_elems = is_ag ? max_n * size_t(world) : max_n;

  CommOptions co;
  co.heap.staging_bytes = opt.staging_mb << 20;
  // room for the symmetric buffers and for staging the largest message
  const size_t want_staging = (in_elems + out_elems) * 2 * (opt.symmetric ? 2 : 1) + (size_t(64) << 20);
  if (co.heap.staging_bytes < want_staging) co.heap.staging_bytes = want_staging;
  co.heap.nvls = opt.nvls;
  co.timeout_ms = opt.timeout_ms;
  co.first_seq = opt.flag;
  if (opt.pcie) co.heap.backing = HeapBacking::HostShm;
  else if (opt.backing == "vmm-fd") co.heap.backing = HeapBacking::VmmFd;
  else if (opt.backing == "cuda-ipc") co.heap.backing = HeapBacking::CudaIpc;
  else if (opt.backing == "host-shm") co.heap.backing = HeapBacking::HostShm;

  std::unique_ptr<Comm> comm = virt ? Comm::create_virtual(world, device, co) : Comm::create(*mesh, device, co);
  if (rank == 0) {
    std::printf("# world %d%s, backing %s, nvls %s, dtype %s, algo %s\n", world, virt ? " (virtual, one GPU)" : "",
                backing_name(comm->heap(0).backing()), comm->has_nvls() ? "on" : (opt.nvls ? comm->heap(0).nvls_note().c_str() : "off"),
                dt == DType::F16 ? "half" : "bf16", opt.algo.c_str());
  }
  std::unique_ptr<NcclBaseline> nccl;
  if (opt.baseline == "nccl") {
    B200_REQUIRE(mesh != nullptr && world > 1, "--baseline nccl needs a multi-process world");
    nccl = std::make_unique<NcclBaseline>(*mesh, device);
    if (rank == 0) std::printf("# baseline: NCCL %d\n", nccl->version());
  }
  const int nlocal = comm->nlocal();
  const uint32_t flags = opt.ref_accum ? uint32_t(kRoundEachAdd) : 0u;
  cudaStream_t stream;
  B200_CUDA_CHECK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  cudaEvent_t ev0, ev1;
  B200_CUDA_CHECK(cudaEventCreate(&ev0));
  B200_CUDA_CHECK(cudaEventCreate(&ev1));

  Buffers buf;
  std::vector<std::vector<uint16_t>> host_in(static_cast<size_t>(world));
  // --symmetric: the buffers live in the heap at the same offset on every rank, so the
  // large-message kernels work on them in place (no staging copies).
  size_t sym_in_off = 0, sym_out_off = 0;
  if (opt.symmetric) {
    sym_in_off = comm->sym_alloc(in_elems * 2);
    if (is_ag || opt.out_of_place) sym_out_off = comm->sym_alloc(out_elems * 2);
  }
  for (int i = 0; i < nlocal; ++i) {
    void *a = nullptr, *b = nullptr;
    if (opt.symmetric) a = comm->sym_ptr(sym_in_off, i);
    else B200_CUDA_CHECK(cudaMalloc(&a, in_elems * 2));
    buf.in.push_back(a);
    if (is_ag || opt.out_of_place) {
      if (opt.symmetric) b = comm->sym_ptr(sym_out_off, i);
      else B200_CUDA_CHECK(cudaMalloc(&b, out_elems * 2));
      B200_CUDA_CHECK(cudaMemset(b, 1, out_elems * 2));
      buf.out.push_back(b);
    } else {
      buf.out.push_back(a);
    }
  }
  auto cleanup = make_guard([&] {
    cudaDeviceSynchronize();
    for (int i = 0; i < nlocal && !opt.symmetric; ++i) {
      if (buf.out[size_t(i)] != buf.in[size_t(i)]) cudaFree(buf.out[size_t(i)]);
      cudaFree(buf.in[size_t(i)]);
    }
    cudaEventDestroy(ev0);
    cudaEventDestroy(ev1);
    cudaStreamDestroy(stream);
  });

  int exit_code = 0;
  if (rank == 0 && !opt.verify)
    std::printf("# %12s %10s %6s %6s %12s %10s %10s\n", "elements", "bytes", "ctas", "warps", "time_us(max)", "algbw_GBs", "busbw_GBs");

  for (size_t n : sizes) {
    auto fill_inputs = [&] {
      for (int r = 0; r < world; ++r) {
        host_in[size_t(r)].resize(n);
        if (opt.random) fill_random(dt, host_in[size_t(r)].data(), r, n, is_ag);
        else fill_pattern(dt, host_in[size_t(r)].data(), r, n);
      }
      for (int i = 0; i < nlocal; ++i)
        B200_CUDA_CHECK(cudaMemcpy(buf.in[size_t(i)], host_in[size_t(comm->rank(i))].data(), n * 2, cudaMemcpyHostToDevice));
    };
    auto launch_once = [&]() -> CollInfo {
      std::vector<const void*> ins(buf.in.begin(), buf.in.end());
      LaunchGeom g{opt.groups, opt.subgroups};
      if (nccl) {
        if (is_ag) nccl->all_gather(ins[0], buf.out[0], n, dt == DType::F16 ? 0 : 1, stream);
        else nccl->all_reduce(ins[0], buf.out[0], n, dt == DType::F16 ? 0 : 1, stream);
        return CollInfo{};
      }
      if (is_ag) return comm->all_gather(algo, dt, ins.data(), buf.out.data(), n, g, stream, flags);
      return comm->all_reduce(algo, dt, ins.data(), buf.out.data(), n, g, stream, flags);
    };

    fill_inputs();
    comm->host_barrier();
    CollInfo info = launch_once();
    B200_CUDA_CHECK(cudaStreamSynchronize(stream));
    comm->raise_if_failed();

    if (opt.verify) {
      // expected result on the CPU, from regenerated inputs of every rank
      std::vector<const uint16_t*> all;
      for (int r = 0; r < world; ++r) all.push_back(host_in[size_t(r)].data());
      const size_t out_n = is_ag ? n * size_t(world) : n;
      std::vector<uint16_t> want(out_n), got(out_n);
      if (is_ag) cpu_all_gather(all, want.data(), n);
      else cpu_all_reduce(dt, all, want.data(), n, opt.ref_accum);
      const bool exact = is_ag || (!opt.random && dt == DType::F16);
      size_t bad = 0;
      for (int i = 0; i < nlocal; ++i) {
        B200_CUDA_CHECK(cudaMemcpy(got.data(), buf.out[size_t(i)], out_n * 2, cudaMemcpyDeviceToHost));
        VerifyReport rep = verify_buffer(dt, got.data(), want.data(), out_n, exact, dt == DType::F16 ? 2e-2f : 1.5e-1f,
                                         dt == DType::F16 ? 4e-3f : 3e-2f);
        if (rep.mismatches) {
          std::printf("[%d] Error Compare! %zu of %zu elements differ; first at %zu: expected %g, got %g\n", comm->rank(i),
                      rep.mismatches, out_n, rep.first_index, double(rep.first_expected), double(rep.first_got));
        }
        bad += rep.mismatches;
      }
      int64_t worst = int64_t(bad);
      if (mesh) worst = mesh->allreduce_max(worst);
      if (rank == 0)
        std::printf("verify %-16s n=%zu world=%d ctas=%d warps=%d steps=%lld : %s\n", opt.algo.c_str(), n, world, info.ctas,
                    info.warps, static_cast<long long>(info.steps), worst ? "FAILED" : "ok");
      if (worst) exit_code = 1;
      continue;
    }

    // two more warm-ups, then the timed launches (main.cpp:86-108)
    for (int k = 0; k < 2; ++k) {
      if (!is_ag && !opt.out_of_place) fill_inputs();  // in place: start from fresh data
      launch_once();
    }
    B200_CUDA_CHECK(cudaStreamSynchronize(stream));
    if (rank == 0 && sizes.size() == 1) std::printf("---------last run------------------\n");
    comm->host_barrier();
    B200_CUDA_CHECK(cudaEventRecord(ev0, stream));
    for (int k = 0; k < opt.iters; ++k) info = launch_once();
    B200_CUDA_CHECK(cudaEventRecord(ev1, stream));
    B200_CUDA_CHECK(cudaStreamSynchronize(stream));
    comm->raise_if_failed();
    float ms = 0;
    B200_CUDA_CHECK(cudaEventElapsedTime(&ms, ev0, ev1));
    const double ns_local = double(ms) * 1e6 / opt.iters;
    double ns_max = ns_local;
    if (mesh) ns_max = double(mesh->allreduce_max(int64_t(ns_local)));
    if (sizes.size() == 1) {
      for (int i = 0; i < nlocal; ++i) std::printf("[%d] Running time: %lldns\n", comm->rank(i), static_cast<long long>(ns_local));
      std::fflush(stdout);
      comm->host_barrier();
    }
    if (rank == 0) {
      const double bytes = double(n) * 2;
      const double algbw = (is_ag ? bytes * world : bytes) / ns_max;  // GB/s
      const double busbw = is_ag ? algbw * (world - 1) / world : algbw * 2 * (world - 1) / world;
      std::printf("  %12zu %10.0f %6d %6d %12.2f %10.2f %10.2f\n", n, bytes, info.ctas, info.warps, ns_max / 1e3, algbw, busbw);
      std::fflush(stdout);
    }
  }
  B200_CUDA_CHECK(cudaDeviceSynchronize());
  comm->host_barrier();
  comm->finalize();
  return exit_code;
}

struct ForkArg {
  const Options* opt;
};

int forked_main(int rank, int world, void* arg) {
  const Options& opt = *static_cast<ForkArg*>(arg)->opt;
  RankEnv env = rank_env_from_environment();
  MeshOptions mo;
  mo.job_id = env.job_id;
  mo.instance = opt.instance;
  UnixMesh mesh(rank, world, mo);
  return run_rank(rank, world, opt, &mesh);
}

}  // namespace

int main(int argc, char** argv) {
  Options opt;
  if (!parse(argc, argv, &opt)) return 0;
  try {
    if (opt.virt > 0) return run_rank(0, opt.virt, opt, nullptr);
    if (opt.np > 1) {
      // fork before anything touches CUDA
      ForkArg arg{&opt};
      return fork_ranks(opt.np, &forked_main, &arg);
    }
    RankEnv env = rank_env_from_environment();
    MeshOptions mo;
    mo.job_id = env.job_id;
    mo.instance = opt.instance;
    UnixMesh mesh(env.rank, env.world, mo);
    return run_rank(env.rank, env.world, opt, &mesh);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "%s\n", e.what());
    return 1;
  }
}
