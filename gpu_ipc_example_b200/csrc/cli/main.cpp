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
// (fork here) or --virtual N (all ranks emulated on one GPU).  -a takes a comma
// separated list (the pseudo algorithms `nccl` / `nccl_allgather` time NCCL on the
// same buffers); timed runs rotate over buffers that together exceed L2, refill
// in-place inputs before every sample and report min / median / max over samples,
// optionally from CUDA-graph replays (--graph) and as JSON or CSV rows.
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
  int samples = 0;        // timed batches per size (0: 1 for a single size, 5 for a sweep)
  bool graph = false;     // time replays of a CUDA graph holding the batch
  bool no_rotate = false; // one buffer instead of a rotating set larger than L2
  std::string json_path, csv_path;
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
      "      --baseline nccl time ncclAllReduce / ncclAllGather on the same buffers instead\n"
      "      --samples S     timed batches per size; min / median / max are reported (default 5 in a sweep)\n"
      "      --graph         time replays of a CUDA graph of the batch (device time without host launch cost)\n"
      "      --no-rotate     reuse one buffer (default: rotate over buffers that together exceed L2)\n"
      "      --json FILE     append one JSON object per (algorithm, size) row\n"
      "      --csv FILE      append one CSV line per row\n"
      "  -a also takes a comma separated list; `nccl`, `nccl_allgather` and `nccl_reduce_scatter` in it\n"
      "  time NCCL; `reduce_scatter` (auto) and `reduce_scatter:<parallel:ll512|bulk|nvls|...>` time the\n"
      "  reduce-scatter (-n then counts the whole input)\n",
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
                              {"samples", required_argument, nullptr, 1012},
                              {"graph", no_argument, nullptr, 1013},
                              {"no-rotate", no_argument, nullptr, 1014},
                              {"json", required_argument, nullptr, 1015},
                              {"csv", required_argument, nullptr, 1016},
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
      case 1012: o->samples = std::max(1, std::atoi(optarg)); break;
      case 1013: o->graph = true; break;
      case 1014: o->no_rotate = true; break;
      case 1015: o->json_path = optarg; break;
      case 1016: o->csv_path = optarg; break;
      case 'h': usage(); return false;
      default: break;
    }
  }
  return true;
}

struct AlgoEntry {
  std::string name;
  AlgoSpec spec;
  bool is_ag = false;
  bool is_rs = false;  // reduce-scatter: `elements` counts the whole input, every rank keeps 1/world of the sum
  bool nccl = false;
};

std::vector<std::string> split_commas(const std::string& s) {
  std::vector<std::string> out;
  std::stringstream ss(s);
  std::string item;
  while (std::getline(ss, item, ','))
    if (!item.empty()) out.push_back(item);
  return out;
}

constexpr size_t kL2Bytes = size_t(126) << 20;
constexpr size_t kSeedElems = size_t(1) << 20;

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int run_rank(int rank, int world, const Options& opt_in, UnixMesh* mesh) {
  Options opt = opt_in;
  B200_REQUIRE(opt.simd == 32, "-s " << opt.simd << ": a wire is one warp of 32 lanes on this hardware");
  const DType dt = (opt.dtype == "bf16" || opt.dtype == "bfloat16") ? DType::BF16 : DType::F16;

  // ---- which algorithms ------------------------------------------------------------------
  std::vector<AlgoEntry> algos;
  bool any_nccl = false, any_ag = false, any_ar = false, any_rs = false;
  for (const std::string& name : split_commas(opt.algo)) {
    AlgoEntry e;
    e.name = name;
    if (name == "nccl" || name == "nccl_allgather" || name == "nccl_reduce_scatter") {
      e.nccl = true;
      e.is_ag = name == "nccl_allgather";
      e.is_rs = name == "nccl_reduce_scatter";
    } else if (name.rfind("reduce_scatter", 0) == 0) {
      // "reduce_scatter" (auto) or "reduce_scatter:<parallel:ll512|simple_pcie_p|bulk|nvls|...>"
      e.is_rs = true;
      bool ag = false;
      const std::string rest = name.size() > 15 ? name.substr(15) : std::string("auto");
      if (!parse_algo(rest, &e.spec, &ag) || ag) {
        std::fprintf(stderr, "unknown reduce-scatter algorithm '%s'\n", name.c_str());
        return 2;
      }
    } else if (!parse_algo(name, &e.spec, &e.is_ag)) {
      // with --baseline nccl the -a value only says which collective: anything naming "allgather" is one
      if (opt.baseline != "nccl") {
        std::fprintf(stderr, "unknown algorithm '%s'\nknown: %s reduce_scatter[:<algo>] nccl nccl_allgather nccl_reduce_scatter\n", name.c_str(), algo_names_help().c_str());
        return 2;
      }
      e.is_ag = name.find("allgather") != std::string::npos;
    }
    if (opt.baseline == "nccl") e.nccl = true;
    any_nccl |= e.nccl;
    (e.is_ag ? any_ag : any_ar) = true;
    any_rs |= e.is_rs;
    algos.push_back(e);
  }
  B200_REQUIRE(!algos.empty(), "no algorithm given");

  int ndev = 0;
  B200_CUDA_CHECK(cudaGetDeviceCount(&ndev));
  const bool virt = opt.virt > 0;
  const int device = device_for_rank(opt.devices, virt ? 0 : rank, ndev);
  B200_CUDA_CHECK(cudaSetDevice(device));

  std::vector<size_t> sizes;
  const bool sweeping = !opt.sweep.empty();
  if (sweeping) {
    int lo = 10, hi = 24;
    if (std::sscanf(opt.sweep.c_str(), "%d:%d", &lo, &hi) != 2) B200_REQUIRE(false, "--sweep wants LO:HI");
    for (int e = lo; e <= hi; ++e) sizes.push_back(size_t(1) << e);
    if (opt.iters == 1) opt.iters = 20;
  } else {
    sizes.push_back(parse_nelems(opt.nelems));
  }
  if (opt.samples == 0) opt.samples = sweeping ? 5 : 1;
  const size_t max_n = *std::max_element(sizes.begin(), sizes.end());

  // ---- buffer pools: a rotating set per size, carved out of one pool ----------------------------
  auto in_bytes = [&](size_t n) { return round_up(n * 2, 256); };
  auto out_bytes = [&](size_t n) { return round_up(n * 2 * (any_ag ? size_t(world) : 1), 256); };
  const bool separate_out = any_ag || any_rs || opt.out_of_place;
  auto nbuf_for = [&](size_t n) -> int {
    if (opt.verify || opt.no_rotate) return 1;
    const size_t set = in_bytes(n) + (separate_out ? out_bytes(n) : 0);
    size_t k = (2 * kL2Bytes + set - 1) / set;
    k = std::min<size_t>(std::max<size_t>(k, 2), 16);
    while (k > 2 && k * set > (size_t(3) << 30)) --k;  // cap the pool at 3 GiB
    return int(k);
  };
  size_t pool_in = 0, pool_out = 0;
  for (size_t n : sizes) {
    pool_in = std::max(pool_in, size_t(nbuf_for(n)) * in_bytes(n));
    pool_out = std::max(pool_out, size_t(nbuf_for(n)) * out_bytes(n));
  }
  if (!separate_out) pool_out = 0;

  CommOptions co;
  co.heap.staging_bytes = opt.staging_mb << 20;
  // room for the symmetric buffers and for staging the largest message
  const size_t want_staging =
      (opt.symmetric ? pool_in + pool_out : 0) + (in_bytes(max_n) + out_bytes(max_n)) + (size_t(64) << 20);
  if (co.heap.staging_bytes < want_staging) co.heap.staging_bytes = want_staging;
  co.heap.nvls = opt.nvls;
  co.timeout_ms = opt.timeout_ms;
  co.first_seq = opt.flag;
  co.device_seq = opt.graph;
  if (opt.pcie) co.heap.backing = HeapBacking::HostShm;
  else if (opt.backing == "vmm-fd") co.heap.backing = HeapBacking::VmmFd;
  else if (opt.backing == "cuda-ipc") co.heap.backing = HeapBacking::CudaIpc;
  else if (opt.backing == "host-shm") co.heap.backing = HeapBacking::HostShm;

  std::unique_ptr<Comm> comm = virt ? Comm::create_virtual(world, device, co) : Comm::create(*mesh, device, co);
  if (rank == 0) {
    std::printf("# world %d%s, backing %s, nvls %s, dtype %s, algo %s%s%s\n", world, virt ? " (virtual, one GPU)" : "",
                backing_name(comm->heap(0).backing()), comm->has_nvls() ? "on" : (opt.nvls ? comm->heap(0).nvls_note().c_str() : "off"),
                dt == DType::F16 ? "half" : "bf16", opt.algo.c_str(), opt.graph ? ", CUDA-graph replays" : "",
                opt.out_of_place ? ", out of place" : "");
  }
  std::unique_ptr<NcclBaseline> nccl;
  if (any_nccl) {
    B200_REQUIRE(mesh != nullptr && world > 1, "NCCL rows need a multi-process world");
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

  // --symmetric: the pools live in the heap at the same offset on every rank, so the
  // large-message kernels work on them in place (no staging copies).
  std::vector<char*> in_pool(size_t(nlocal), nullptr), out_pool(size_t(nlocal), nullptr);
  void* seed = nullptr;  // device copy of the first kSeedElems input elements, for refills
  {
    size_t sym_in = 0, sym_out = 0;
    if (opt.symmetric) {
      sym_in = comm->sym_alloc(pool_in);
      if (separate_out) sym_out = comm->sym_alloc(pool_out);
    }
    for (int i = 0; i < nlocal; ++i) {
      void *a = nullptr, *b = nullptr;
      if (opt.symmetric) a = comm->sym_ptr(sym_in, i);
      else B200_CUDA_CHECK(cudaMalloc(&a, pool_in));
      in_pool[size_t(i)] = static_cast<char*>(a);
      if (separate_out) {
        if (opt.symmetric) b = comm->sym_ptr(sym_out, i);
        else B200_CUDA_CHECK(cudaMalloc(&b, pool_out));
        B200_CUDA_CHECK(cudaMemset(b, 1, pool_out));
        out_pool[size_t(i)] = static_cast<char*>(b);
      }
    }
    B200_CUDA_CHECK(cudaMalloc(&seed, kSeedElems * 2 * size_t(nlocal)));
  }
  auto cleanup = make_guard([&] {
    cudaDeviceSynchronize();
    for (int i = 0; i < nlocal && !opt.symmetric; ++i) {
      if (out_pool[size_t(i)]) cudaFree(out_pool[size_t(i)]);
      cudaFree(in_pool[size_t(i)]);
    }
    cudaFree(seed);
    cudaEventDestroy(ev0);
    cudaEventDestroy(ev1);
    cudaStreamDestroy(stream);
  });

  FILE* json = nullptr;
  FILE* csv = nullptr;
  if (rank == 0 && !opt.json_path.empty()) json = std::fopen(opt.json_path.c_str(), "a");
  if (rank == 0 && !opt.csv_path.empty()) {
    csv = std::fopen(opt.csv_path.c_str(), "a");
    if (csv && std::ftell(csv) == 0)
      std::fprintf(csv, "collective,algo,world,dtype,placement,timing,elements,bytes,ctas,warps,us_min,us_median,us_max,algbw_GBs,busbw_GBs\n");
  }
  auto close_files = make_guard([&] {
    if (json) std::fclose(json);
    if (csv) std::fclose(csv);
  });

  int exit_code = 0;
  std::vector<std::vector<uint16_t>> host_in(static_cast<size_t>(world));

  for (const AlgoEntry& algo : algos) {
    const bool is_ag = algo.is_ag;
    const bool is_rs = algo.is_rs;
    if (rank == 0 && !opt.verify) {
      std::printf("# algo %s\n", algo.name.c_str());
      std::printf("# %12s %10s %6s %6s %12s %12s %12s %10s %10s\n", "elements", "bytes", "ctas", "warps", "us_min(max)", "us_median",
                  "us_max", "algbw_GBs", "busbw_GBs");
    }
    for (size_t n : sizes) {
      const int nbuf = nbuf_for(n);
      if (is_rs && n % (8 * size_t(world)) != 0) continue;
      const size_t out_n = is_ag ? n * size_t(world) : (is_rs ? n / size_t(world) : n);
      auto in_ptr = [&](int i, int k) { return static_cast<void*>(in_pool[size_t(i)] + size_t(k) * in_bytes(n)); };
      auto out_ptr = [&](int i, int k) {
        return separate_out ? static_cast<void*>(out_pool[size_t(i)] + size_t(k) * out_bytes(n)) : in_ptr(i, k);
      };
      // Exact inputs of every rank on the host (verification), or only the first kSeedElems of the
      // local ranks (timing: the buffers are filled by tiling that piece).
      auto fill_inputs = [&](bool first) {
        const size_t host_n = opt.verify ? n : std::min(n, kSeedElems);
        if (first) {
          for (int r = 0; r < world; ++r) {
            host_in[size_t(r)].resize(host_n);
            if (opt.random || !opt.verify) fill_random(dt, host_in[size_t(r)].data(), r, host_n, is_ag);
            else fill_pattern(dt, host_in[size_t(r)].data(), r, host_n);
          }
          for (int i = 0; i < nlocal; ++i)
            B200_CUDA_CHECK(cudaMemcpy(static_cast<char*>(seed) + size_t(i) * kSeedElems * 2, host_in[size_t(comm->rank(i))].data(),
                                       std::min(host_n, kSeedElems) * 2, cudaMemcpyHostToDevice));
        }
        for (int i = 0; i < nlocal; ++i) {
          if (opt.verify) {
            B200_CUDA_CHECK(cudaMemcpy(in_ptr(i, 0), host_in[size_t(comm->rank(i))].data(), n * 2, cudaMemcpyHostToDevice));
            continue;
          }
          for (int k = 0; k < nbuf; ++k)
            for (size_t off = 0; off < n; off += kSeedElems)
              B200_CUDA_CHECK(cudaMemcpyAsync(static_cast<char*>(in_ptr(i, k)) + off * 2,
                                              static_cast<char*>(seed) + size_t(i) * kSeedElems * 2,
                                              std::min(kSeedElems, n - off) * 2, cudaMemcpyDeviceToDevice, stream));
        }
        B200_CUDA_CHECK(cudaStreamSynchronize(stream));
      };
      auto launch_once = [&](int k) -> CollInfo {
        std::vector<const void*> ins(static_cast<size_t>(nlocal));
        std::vector<void*> outs(static_cast<size_t>(nlocal));
        for (int i = 0; i < nlocal; ++i) {
          ins[size_t(i)] = in_ptr(i, k % nbuf);
          outs[size_t(i)] = out_ptr(i, k % nbuf);
        }
        LaunchGeom g{opt.groups, opt.subgroups};
        if (algo.nccl) {
          if (is_ag) nccl->all_gather(ins[0], outs[0], n, dt == DType::F16 ? 0 : 1, stream);
          else if (is_rs) nccl->reduce_scatter(ins[0], outs[0], n / size_t(world), dt == DType::F16 ? 0 : 1, stream);
          else nccl->all_reduce(ins[0], outs[0], n, dt == DType::F16 ? 0 : 1, stream);
          return CollInfo{};
        }
        if (is_ag) return comm->all_gather(algo.spec, dt, ins.data(), outs.data(), n, g, stream, flags);
        if (is_rs) return comm->reduce_scatter(algo.spec, dt, ins.data(), outs.data(), n, g, stream, flags);
        return comm->all_reduce(algo.spec, dt, ins.data(), outs.data(), n, g, stream, flags);
      };

      fill_inputs(true);
      comm->host_barrier();
      CollInfo info;
      try {
        info = launch_once(0);
      } catch (const std::exception& e) {
        // a geometry this algorithm does not take at this size: the check runs on the host before anything is
        // launched and depends on nothing but the size, so every rank skips the same rows
        if (opt.verify || !sweeping) throw;  // only a sweep skips sizes; a single run or a verification fails
        if (rank == 0) std::printf("# skipped %zu elements: %s\n", n, e.what());
        cudaGetLastError();
        continue;
      }
      B200_CUDA_CHECK(cudaStreamSynchronize(stream));
      comm->raise_if_failed();

      if (opt.verify) {
        // expected result on the CPU, from regenerated inputs of every rank
        std::vector<const uint16_t*> all;
        for (int r = 0; r < world; ++r) all.push_back(host_in[size_t(r)].data());
        std::vector<uint16_t> want(is_rs ? n : out_n), got(out_n);
        if (is_ag) cpu_all_gather(all, want.data(), n);
        else cpu_all_reduce(dt, all, want.data(), n, opt.ref_accum);
        const bool exact = is_ag || (!opt.random && dt == DType::F16);
        size_t bad = 0;
        for (int i = 0; i < nlocal; ++i) {
          B200_CUDA_CHECK(cudaMemcpy(got.data(), out_ptr(i, 0), out_n * 2, cudaMemcpyDeviceToHost));
          const uint16_t* want_i = want.data() + (is_rs ? size_t(comm->rank(i)) * out_n : 0);
          VerifyReport rep = verify_buffer(dt, got.data(), want_i, out_n, exact, dt == DType::F16 ? 2e-2f : 1.5e-1f,
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
          std::printf("verify %-16s n=%zu world=%d ctas=%d warps=%d steps=%lld : %s\n", algo.name.c_str(), n, world, info.ctas,
                      info.warps, static_cast<long long>(info.steps), worst ? "FAILED" : "ok");
        if (worst) exit_code = 1;
        continue;
      }

      // two more warm-ups, then the timed batches (main.cpp:86-108)
      for (int k = 1; k <= 2; ++k) info = launch_once(k);
      B200_CUDA_CHECK(cudaStreamSynchronize(stream));
      comm->raise_if_failed();
      if (rank == 0 && !sweeping && algos.size() == 1) std::printf("---------last run------------------\n");

      // --graph: the batch becomes one CUDA graph; a sample is one replay
      cudaGraphExec_t exec = nullptr;
      if (opt.graph && !virt) {
        cudaGraph_t graph = nullptr;
        B200_CUDA_CHECK(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
        for (int k = 0; k < opt.iters; ++k) info = launch_once(k);
        B200_CUDA_CHECK(cudaStreamEndCapture(stream, &graph));
        B200_CUDA_CHECK(cudaGraphInstantiate(&exec, graph, 0));
        B200_CUDA_CHECK(cudaGraphDestroy(graph));
        B200_CUDA_CHECK(cudaGraphLaunch(exec, stream));  // untimed first replay
        B200_CUDA_CHECK(cudaStreamSynchronize(stream));
      }
      std::vector<double> sample_ns;
      double ns_local_last = 0;
      for (int sidx = 0; sidx < opt.samples; ++sidx) {
        if (!is_ag && !is_rs && !opt.out_of_place) fill_inputs(false);  // in place: every sample starts from fresh data
        comm->host_barrier();
        B200_CUDA_CHECK(cudaEventRecord(ev0, stream));
        if (exec) {
          B200_CUDA_CHECK(cudaGraphLaunch(exec, stream));
        } else {
          for (int k = 0; k < opt.iters; ++k) info = launch_once(k);
        }
        B200_CUDA_CHECK(cudaEventRecord(ev1, stream));
        B200_CUDA_CHECK(cudaStreamSynchronize(stream));
        comm->raise_if_failed();
        float ms = 0;
        B200_CUDA_CHECK(cudaEventElapsedTime(&ms, ev0, ev1));
        ns_local_last = double(ms) * 1e6 / opt.iters;
        double ns_max = ns_local_last;
        if (mesh) ns_max = double(mesh->allreduce_max(int64_t(ns_local_last)));
        sample_ns.push_back(ns_max);
      }
      if (exec) B200_CUDA_CHECK(cudaGraphExecDestroy(exec));
      std::sort(sample_ns.begin(), sample_ns.end());
      const double ns_min = sample_ns.front(), ns_med = sample_ns[sample_ns.size() / 2], ns_hi = sample_ns.back();
      if (!sweeping && algos.size() == 1) {
        for (int i = 0; i < nlocal; ++i) std::printf("[%d] Running time: %lldns\n", comm->rank(i), static_cast<long long>(ns_local_last));
        std::fflush(stdout);
        comm->host_barrier();
      }
      if (rank == 0) {
        const double bytes = double(n) * 2;
        const double algbw = (is_ag ? bytes * world : bytes) / ns_med;  // GB/s
        const double busbw = (is_ag || is_rs) ? algbw * (world - 1) / world : algbw * 2 * (world - 1) / world;
        std::printf("  %12zu %10.0f %6d %6d %12.2f %12.2f %12.2f %10.2f %10.2f\n", n, bytes, info.ctas, info.warps, ns_min / 1e3,
                    ns_med / 1e3, ns_hi / 1e3, algbw, busbw);
        std::fflush(stdout);
        const char* coll = is_ag ? "all_gather" : (is_rs ? "reduce_scatter" : "all_reduce");
        const char* place = (is_ag || is_rs) ? "out_of_place" : (opt.out_of_place ? "out_of_place" : "in_place");
        const char* timing = exec ? "graph_replay" : "launch_loop";
        const char* dname = dt == DType::F16 ? "fp16" : "bf16";
        if (json) {
          std::fprintf(json,
                       "{\"collective\": \"%s\", \"algo\": \"%s\", \"world\": %d, \"dtype\": \"%s\", \"placement\": \"%s\", "
                       "\"symmetric\": %s, \"timing\": \"%s\", \"iters\": %d, \"samples\": %d, \"buffers\": %d, \"elements\": %zu, "
                       "\"bytes\": %.0f, \"ctas\": %d, \"warps\": %d, \"us_min\": %.3f, \"us_median\": %.3f, \"us_max\": %.3f, "
                       "\"algbw_GBs\": %.3f, \"busbw_GBs\": %.3f}\n",
                       coll, algo.name.c_str(), world, dname, place, opt.symmetric ? "true" : "false", timing, opt.iters, opt.samples,
                       nbuf, n, bytes, info.ctas, info.warps, ns_min / 1e3, ns_med / 1e3, ns_hi / 1e3, algbw, busbw);
          std::fflush(json);
        }
        if (csv) {
          std::fprintf(csv, "%s,%s,%d,%s,%s,%s,%zu,%.0f,%d,%d,%.3f,%.3f,%.3f,%.3f,%.3f\n", coll, algo.name.c_str(), world, dname, place,
                       timing, n, bytes, info.ctas, info.warps, ns_min / 1e3, ns_med / 1e3, ns_hi / 1e3, algbw, busbw);
          std::fflush(csv);
        }
      }
    }
  }
  B200_CUDA_CHECK(cudaDeviceSynchronize());
  comm->host_barrier();
  nccl.reset();
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
