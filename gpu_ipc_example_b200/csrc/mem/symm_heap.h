// The symmetric heap: one allocation per rank with the same layout everywhere,
// mapped into every rank's address space so that kernels can store into (and
// load from) a peer's memory directly over NVLink.
//
// Backings, tried in this order under HeapBacking::Auto:
//   VmmFd    cuMemCreate + POSIX file-descriptor export; descriptors travel over
//            the Unix-socket mesh (SCM_RIGHTS); peers cuMemImport + cuMemMap.
//            Needed for NVLS (the multicast object binds VMM allocations).
//   CudaIpc  cudaMalloc + cudaIpcGetMemHandle; the 64-byte handles travel as bytes.
//   HostShm  pinned host memory shared through a memfd; used when peers cannot
//            address each other (no P2P) or when forced (the CLI's -p): the same
//            kernels then run over PCIe.
//   Local    plain cudaMalloc, for the single-GPU emulation of a world.
//
// Capability parity: open_all_ipc_mems (ipc_exchange.cpp:267-313), host-memory
// scratch when P2P is missing or -p is given (main.cpp:236-242), mmap_host debug
// view (ipc_exchange.cpp:340-354; here: dump()), canAccessPeer
// (ipc_exchange.cpp:315-338).
#pragma once

#include <memory>
#include <string>
#include <vector>

#include <cuda.h>

#include "../bootstrap/unix_mesh.h"
#include "../common/heap_layout.h"
#include "../common/types.h"

namespace b200ipc {

enum class HeapBacking : int { Auto = 0, VmmFd = 1, CudaIpc = 2, HostShm = 3, Local = 4 };
const char* backing_name(HeapBacking b);

struct HeapOptions {
  size_t staging_bytes = size_t(256) << 20;
  HeapBacking backing = HeapBacking::Auto;
  bool nvls = false;  // also create and map an NVSwitch multicast object over the heap
};


// True when every pair of the listed devices can address each other's memory.
bool all_peers_accessible(const std::vector<int>& devices);

class SymmHeap {
 public:
  // Collective over the mesh: every rank calls it with its own device.
  SymmHeap(UnixMesh& mesh, int device, const HeapOptions& opt);
  // Single-process world of n ranks on one device (backing Local).
  static std::vector<std::unique_ptr<SymmHeap>> make_virtual(int n, int device, const HeapOptions& opt);
  ~SymmHeap();
  SymmHeap(const SymmHeap&) = delete;
  SymmHeap& operator=(const SymmHeap&) = delete;

  int rank() const { return rank_; }
  int world() const { return world_; }
  int device() const { return device_; }
  const HeapLayout& layout() const { return lay_; }
  HeapBacking backing() const { return backing_; }
  char* base() const { return peer_[size_t(rank_)]; }
  char* peer(int r) const { return peer_[size_t(r)]; }
  char* multicast() const { return mc_ptr_; }  // nullptr without NVLS
  const std::string& nvls_note() const { return nvls_note_; }

  // Copies [offset, offset+bytes) of this rank's heap to host memory (debug view).
  void dump(size_t offset, size_t bytes, void* host_dst) const;
  // Zeroes this rank's heap (all regions but staging unless told otherwise).
  void clear(bool include_staging) const;
  // Unbinds the multicast object; collective, must run on every rank before exit.
  void release_multicast(UnixMesh* mesh);

 private:
  SymmHeap() = default;
  void init_vmm(UnixMesh& mesh, const HeapOptions& opt);
  void init_cuda_ipc(UnixMesh& mesh);
  void init_host_shm(UnixMesh& mesh);
  void init_nvls(UnixMesh& mesh);

  int rank_ = 0;
  int world_ = 1;
  int device_ = 0;
  HeapLayout lay_{};
  HeapBacking backing_ = HeapBacking::Local;
  std::vector<char*> peer_;
  size_t mapped_bytes_ = 0;

  // VmmFd
  std::vector<CUmemGenericAllocationHandle> handles_;
  // CudaIpc / Local
  void* owned_dev_ptr_ = nullptr;
  // HostShm
  std::vector<void*> host_maps_;
  // NVLS
  CUmemGenericAllocationHandle mc_handle_ = 0;
  bool mc_bound_ = false;
  char* mc_ptr_ = nullptr;
  std::string nvls_note_;
};

}  // namespace b200ipc
