// NCCL as the comparison baseline of the CLI (--baseline nccl): loaded with dlopen
// at run time so that nothing links against it; the unique id travels over the same
// Unix-socket mesh as the memory handles.  NCCL is what this library is measured
// against, never a path of the library itself.
#pragma once

#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <string>

#include <cuda_runtime_api.h>

#include "../bootstrap/unix_mesh.h"
#include "../common/check.h"

namespace b200ipc {

class NcclBaseline {
 public:
  struct UniqueId { char internal[128]; };
  using Comm = void*;

  NcclBaseline(UnixMesh& mesh, int device) {
    const char* path = std::getenv("B200IPC_NCCL_LIB");
    lib_ = ::dlopen(path ? path : "libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    B200_REQUIRE(lib_ != nullptr, "cannot load NCCL (" << (path ? path : "libnccl.so.2") << "): " << ::dlerror());
    get_unique_id_ = sym<int (*)(UniqueId*)>("ncclGetUniqueId");
    init_rank_ = sym<int (*)(Comm*, int, UniqueId, int)>("ncclCommInitRank");
    all_reduce_ = sym<int (*)(const void*, void*, size_t, int, int, Comm, cudaStream_t)>("ncclAllReduce");
    all_gather_ = sym<int (*)(const void*, void*, size_t, int, Comm, cudaStream_t)>("ncclAllGather");
    reduce_scatter_ = sym<int (*)(const void*, void*, size_t, int, int, Comm, cudaStream_t)>("ncclReduceScatter");
    destroy_ = sym<int (*)(Comm)>("ncclCommDestroy");
    get_version_ = sym<int (*)(int*)>("ncclGetVersion");
    B200_CUDA_CHECK(cudaSetDevice(device));
    UniqueId id;
    std::memset(&id, 0, sizeof(id));
    if (mesh.rank() == 0) check(get_unique_id_(&id), "ncclGetUniqueId");
    std::vector<UniqueId> all(static_cast<size_t>(mesh.world()));
    mesh.allgather(&id, sizeof(id), all.data());
    check(init_rank_(&comm_, mesh.world(), all[0], mesh.rank()), "ncclCommInitRank");
  }
  ~NcclBaseline() {
    if (comm_) destroy_(comm_);
    if (lib_) ::dlclose(lib_);
  }
  int version() const {
    int v = 0;
    get_version_(&v);
    return v;
  }
  // dtype: 0 = fp16, 1 = bf16
  void all_reduce(const void* in, void* out, size_t n, int dtype, cudaStream_t s) {
    check(all_reduce_(in, out, n, dtype == 0 ? 6 : 9, 0 /* sum */, comm_, s), "ncclAllReduce");
  }
  void all_gather(const void* in, void* out, size_t n, int dtype, cudaStream_t s) {
    check(all_gather_(in, out, n, dtype == 0 ? 6 : 9, comm_, s), "ncclAllGather");
  }
  // n: elements every rank receives
  void reduce_scatter(const void* in, void* out, size_t n, int dtype, cudaStream_t s) {
    check(reduce_scatter_(in, out, n, dtype == 0 ? 6 : 9, 0 /* sum */, comm_, s), "ncclReduceScatter");
  }

 private:
  template <typename F>
  F sym(const char* name) {
    void* p = ::dlsym(lib_, name);
    B200_REQUIRE(p != nullptr, "NCCL symbol " << name << " not found");
    return reinterpret_cast<F>(p);
  }
  static void check(int rc, const char* what) { B200_REQUIRE(rc == 0, what << " failed with NCCL error " << rc); }

  void* lib_ = nullptr;
  Comm comm_ = nullptr;
  int (*get_unique_id_)(UniqueId*) = nullptr;
  int (*init_rank_)(Comm*, int, UniqueId, int) = nullptr;
  int (*all_reduce_)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*all_gather_)(const void*, void*, size_t, int, Comm, cudaStream_t) = nullptr;
  int (*reduce_scatter_)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*destroy_)(Comm) = nullptr;
  int (*get_version_)(int*) = nullptr;
};

}  // namespace b200ipc
