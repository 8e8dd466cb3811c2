#include "symm_heap.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>

#include <cuda_runtime_api.h>

#include "../coll/schedules.h"
#include "../common/check.h"
#include "../common/cu_driver.h"
#include "../common/heap_layout.h"

namespace b200ipc {

const char* backing_name(HeapBacking b) {
  switch (b) {
    case HeapBacking::Auto: return "auto";
    case HeapBacking::VmmFd: return "vmm-fd";
    case HeapBacking::CudaIpc: return "cuda-ipc";
    case HeapBacking::HostShm: return "host-shm";
    default: return "local";
  }
}

namespace {
constexpr size_t kAlign = size_t(2) << 20;
size_t up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}  // namespace

bool all_peers_accessible(const std::vector<int>& devices) {
  for (int a : devices)
    for (int b : devices) {
      if (a == b) continue;
      int ok = 0;
      B200_CUDA_CHECK(cudaDeviceCanAccessPeer(&ok, a, b));
      if (!ok) return false;
    }
  return true;
}

SymmHeap::SymmHeap(UnixMesh& mesh, int device, const HeapOptions& opt) {
  rank_ = mesh.rank();
  world_ = mesh.world();
  device_ = device;
  lay_ = make_heap_layout(opt.staging_bytes);
  peer_.assign(size_t(kMaxRanks), nullptr);
  B200_CUDA_CHECK(cudaSetDevice(device));
  B200_CUDA_CHECK(cudaFree(nullptr));  // make the primary context current for driver calls

  // Agree on what every rank can do before choosing.
  std::vector<int32_t> devs(static_cast<size_t>(world_), 0);
  int32_t mydev = device;
  mesh.allgather(&mydev, sizeof(mydev), devs.data());
  std::vector<int> devlist(devs.begin(), devs.end());
  bool same_device_twice = false;
  for (int i = 0; i < world_; ++i)
    for (int j = i + 1; j < world_; ++j) same_device_twice |= (devlist[size_t(i)] == devlist[size_t(j)]);
  // Kernels of different ranks wait on one another; two of them sharing a device are
  // not guaranteed to run at the same time.  The virtual world covers that case.
  B200_REQUIRE(!same_device_twice,
               "two ranks were given the same device; run an emulated world on one GPU with make_virtual()");
  int64_t no_p2p = all_peers_accessible(devlist) ? 0 : 1;
  no_p2p = mesh.allreduce_max(no_p2p);

  HeapBacking want = opt.backing;
  if (want == HeapBacking::Auto) want = no_p2p ? HeapBacking::HostShm : HeapBacking::VmmFd;
  B200_REQUIRE(!(no_p2p && (want == HeapBacking::VmmFd || want == HeapBacking::CudaIpc)),
               "peer access between the chosen devices is not available; use host-shm backing");

  if (want == HeapBacking::VmmFd) {
    // A rank whose driver refuses fd export makes everyone fall back together.
    int64_t failed = 0;
    std::string why;
    try {
      int supported = 0;
      CUdevice cudev;
      B200_CU_CHECK(cu().DeviceGet(&cudev, device));
      B200_CU_CHECK(cu().DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cudev));
      if (!supported) failed = 1;
    } catch (const std::exception& e) {
      failed = 1;
      why = e.what();
    }
    failed = mesh.allreduce_max(failed);
    if (failed) {
      B200_REQUIRE(opt.backing == HeapBacking::Auto, "vmm-fd backing is not available here: " << why);
      want = HeapBacking::CudaIpc;
    }
  }

  backing_ = want;
  switch (want) {
    case HeapBacking::VmmFd: init_vmm(mesh, opt); break;
    case HeapBacking::CudaIpc: init_cuda_ipc(mesh); break;
    case HeapBacking::HostShm: init_host_shm(mesh); break;
    default: B200_REQUIRE(false, "backing " << backing_name(want) << " needs make_virtual()");
  }
  clear(/*include_staging=*/false);
  B200_CUDA_CHECK(cudaDeviceSynchronize());
  mesh.barrier();

  if (opt.nvls) {
    if (backing_ == HeapBacking::VmmFd) {
      init_nvls(mesh);
    } else {
      nvls_note_ = std::string("NVLS needs vmm-fd backing, have ") + backing_name(backing_);
    }
  }
}

std::vector<std::unique_ptr<SymmHeap>> SymmHeap::make_virtual(int n, int device, const HeapOptions& opt) {
  B200_REQUIRE(n >= 1 && n <= kMaxRanks, "virtual world of " << n << " ranks");
  B200_CUDA_CHECK(cudaSetDevice(device));
  std::vector<std::unique_ptr<SymmHeap>> v;
  std::vector<char*> bases;
  HeapLayout lay = make_heap_layout(opt.staging_bytes);
  for (int r = 0; r < n; ++r) {
    std::unique_ptr<SymmHeap> h(new SymmHeap());
    h->rank_ = r;
    h->world_ = n;
    h->device_ = device;
    h->lay_ = lay;
    h->backing_ = HeapBacking::Local;
    h->mapped_bytes_ = lay.total_bytes;
    B200_CUDA_CHECK(cudaMalloc(&h->owned_dev_ptr_, lay.total_bytes));
    bases.push_back(static_cast<char*>(h->owned_dev_ptr_));
    v.push_back(std::move(h));
  }
  for (auto& h : v) {
    h->peer_.assign(size_t(kMaxRanks), nullptr);
    for (int r = 0; r < n; ++r) h->peer_[size_t(r)] = bases[size_t(r)];
    h->clear(false);
  }
  B200_CUDA_CHECK(cudaDeviceSynchronize());
  return v;
}

void SymmHeap::init_vmm(UnixMesh& mesh, const HeapOptions& opt) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  B200_CU_CHECK(cu().MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  size_t mgran = 0;
  if (opt.nvls) {
    CUmulticastObjectProp mp{};
    mp.numDevices = unsigned(world_);
    mp.size = lay_.total_bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    if (cu().MulticastGetGranularity(&mgran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) mgran = 0;
  }
  // All ranks must map the same size: take the largest granularity anyone reports.
  int64_t g = int64_t(std::max(gran, mgran));
  g = mesh.allreduce_max(g);
  mapped_bytes_ = up(lay_.total_bytes, size_t(g));

  handles_.assign(size_t(world_), 0);
  CUmemGenericAllocationHandle mine = 0;
  B200_CU_CHECK(cu().MemCreate(&mine, mapped_bytes_, &prop, 0));
  handles_[size_t(rank_)] = mine;
  int fd = -1;
  B200_CU_CHECK(cu().MemExportToShareableHandle(&fd, mine, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  std::vector<int> fds = mesh.allgather_fds(fd);
  ::close(fd);
  auto close_fds = make_guard([&] {
    for (int f : fds)
      if (f >= 0) ::close(f);
  });

  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int r = 0; r < world_; ++r) {
    if (r != rank_) {
      B200_CU_CHECK(cu().MemImportFromShareableHandle(&handles_[size_t(r)], reinterpret_cast<void*>(uintptr_t(fds[size_t(r)])),
                                                   CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    }
    CUdeviceptr va = 0;
    B200_CU_CHECK(cu().MemAddressReserve(&va, mapped_bytes_, size_t(g), 0, 0));
    B200_CU_CHECK(cu().MemMap(va, mapped_bytes_, 0, handles_[size_t(r)], 0));
    B200_CU_CHECK(cu().MemSetAccess(va, mapped_bytes_, &access, 1));
    peer_[size_t(r)] = reinterpret_cast<char*>(va);
  }
}

void SymmHeap::init_cuda_ipc(UnixMesh& mesh) {
  mapped_bytes_ = lay_.total_bytes;
  B200_CUDA_CHECK(cudaMalloc(&owned_dev_ptr_, mapped_bytes_));
  cudaIpcMemHandle_t mine;
  B200_CUDA_CHECK(cudaIpcGetMemHandle(&mine, owned_dev_ptr_));
  std::vector<cudaIpcMemHandle_t> all(static_cast<size_t>(world_));
  mesh.allgather(&mine, sizeof(mine), all.data());
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) {
      peer_[size_t(r)] = static_cast<char*>(owned_dev_ptr_);
    } else {
      void* p = nullptr;
      B200_CUDA_CHECK(cudaIpcOpenMemHandle(&p, all[size_t(r)], cudaIpcMemLazyEnablePeerAccess));
      peer_[size_t(r)] = static_cast<char*>(p);
    }
  }
}

void SymmHeap::init_host_shm(UnixMesh& mesh) {
  mapped_bytes_ = lay_.total_bytes;
  int fd = ::memfd_create("b200ipc-heap", MFD_CLOEXEC);
  B200_SYS_CHECK(fd);
  B200_SYS_CHECK(::ftruncate(fd, off_t(mapped_bytes_)));
  std::vector<int> fds = mesh.allgather_fds(fd);
  ::close(fd);
  host_maps_.assign(size_t(world_), nullptr);
  for (int r = 0; r < world_; ++r) {
    void* p = ::mmap(nullptr, mapped_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fds[size_t(r)], 0);
    ::close(fds[size_t(r)]);
    B200_REQUIRE(p != MAP_FAILED, "mmap of rank " << r << "'s host heap failed: " << std::strerror(errno));
    host_maps_[size_t(r)] = p;
    B200_CUDA_CHECK(cudaHostRegister(p, mapped_bytes_, cudaHostRegisterMapped | cudaHostRegisterPortable));
    void* d = nullptr;
    B200_CUDA_CHECK(cudaHostGetDevicePointer(&d, p, 0));
    peer_[size_t(r)] = static_cast<char*>(d);
  }
}

void SymmHeap::init_nvls(UnixMesh& mesh) {
  CUdevice cudev;
  B200_CU_CHECK(cu().DeviceGet(&cudev, device_));
  int supported = 0;
  if (cu().DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev) != CUDA_SUCCESS) supported = 0;
  int64_t missing = mesh.allreduce_max(supported ? 0 : 1);
  if (missing) {
    nvls_note_ = "multicast is not supported on at least one device";
    return;
  }
  CUmulticastObjectProp mp{};
  mp.numDevices = unsigned(world_);
  mp.size = mapped_bytes_;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  mp.flags = 0;

  // Rank 0 creates the object; a failure there is shared before anyone blocks on a descriptor.
  int fd = -1;
  int64_t create_failed = 0;
  if (rank_ == 0) {
    CUresult rc = cu().MulticastCreate(&mc_handle_, &mp);
    if (rc == CUDA_SUCCESS) rc = cu().MemExportToShareableHandle(&fd, mc_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (rc != CUDA_SUCCESS) {
      create_failed = 1;
      nvls_note_ = "cuMulticastCreate/export failed: " + cu_error_string(rc);
      if (mc_handle_) cu().MemRelease(mc_handle_);
      mc_handle_ = 0;
    }
  }
  create_failed = mesh.allreduce_max(create_failed);
  if (create_failed) {
    if (nvls_note_.empty()) nvls_note_ = "rank 0 could not create the multicast object";
    return;
  }
  int local_fd = mesh.broadcast_fd(0, fd);
  if (rank_ == 0) ::close(fd);
  if (rank_ != 0) {
    B200_CU_CHECK(cu().MemImportFromShareableHandle(&mc_handle_, reinterpret_cast<void*>(uintptr_t(local_fd)),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  }
  ::close(local_fd);
  B200_CU_CHECK(cu().MulticastAddDevice(mc_handle_, cudev));
  mesh.barrier();  // every device must be added before any memory is bound
  B200_CU_CHECK(cu().MulticastBindMem(mc_handle_, 0, handles_[size_t(rank_)], 0, mapped_bytes_, 0));
  mc_bound_ = true;
  mesh.barrier();

  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  size_t mgran = 0;
  B200_CU_CHECK(cu().MulticastGetGranularity(&mgran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
  CUdeviceptr va = 0;
  B200_CU_CHECK(cu().MemAddressReserve(&va, mapped_bytes_, mgran, 0, 0));
  B200_CU_CHECK(cu().MemMap(va, mapped_bytes_, 0, mc_handle_, 0));
  B200_CU_CHECK(cu().MemSetAccess(va, mapped_bytes_, &access, 1));
  mc_ptr_ = reinterpret_cast<char*>(va);
  nvls_note_ = "ok";
  mesh.barrier();
}

void SymmHeap::release_multicast(UnixMesh* mesh) {
  if (!mc_handle_) return;
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  if (mesh) mesh->barrier();  // nobody may still be issuing multimem traffic
  if (mc_ptr_) {
    cu().MemUnmap(reinterpret_cast<CUdeviceptr>(mc_ptr_), mapped_bytes_);
    cu().MemAddressFree(reinterpret_cast<CUdeviceptr>(mc_ptr_), mapped_bytes_);
    mc_ptr_ = nullptr;
  }
  if (mc_bound_) {
    CUdevice cudev;
    if (cu().DeviceGet(&cudev, device_) == CUDA_SUCCESS) cu().MulticastUnbind(mc_handle_, cudev, 0, mapped_bytes_);
    mc_bound_ = false;
  }
  if (mesh) mesh->barrier();
  cu().MemRelease(mc_handle_);
  mc_handle_ = 0;
}

void SymmHeap::dump(size_t offset, size_t bytes, void* host_dst) const {
  B200_REQUIRE(offset + bytes <= lay_.total_bytes, "dump range outside the heap");
  B200_CUDA_CHECK(cudaSetDevice(device_));
  B200_CUDA_CHECK(cudaMemcpy(host_dst, base() + offset, bytes, cudaMemcpyDeviceToHost));
}

void SymmHeap::clear(bool include_staging) const {
  B200_CUDA_CHECK(cudaSetDevice(device_));
  size_t bytes = include_staging ? lay_.total_bytes : lay_.staging_off;
  B200_CUDA_CHECK(cudaMemset(base(), 0, bytes));
}

SymmHeap::~SymmHeap() {
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  release_multicast(nullptr);
  switch (backing_) {
    case HeapBacking::VmmFd:
      for (int r = 0; r < world_; ++r) {
        if (peer_[size_t(r)]) {
          cu().MemUnmap(reinterpret_cast<CUdeviceptr>(peer_[size_t(r)]), mapped_bytes_);
          cu().MemAddressFree(reinterpret_cast<CUdeviceptr>(peer_[size_t(r)]), mapped_bytes_);
        }
        if (size_t(r) < handles_.size() && handles_[size_t(r)]) cu().MemRelease(handles_[size_t(r)]);
      }
      break;
    case HeapBacking::CudaIpc:
      for (int r = 0; r < world_; ++r)
        if (r != rank_ && peer_[size_t(r)]) cudaIpcCloseMemHandle(peer_[size_t(r)]);
      if (owned_dev_ptr_) cudaFree(owned_dev_ptr_);
      break;
    case HeapBacking::HostShm:
      for (void* p : host_maps_)
        if (p) {
          cudaHostUnregister(p);
          ::munmap(p, mapped_bytes_);
        }
      break;
    default:
      if (owned_dev_ptr_) cudaFree(owned_dev_ptr_);
      break;
  }
}

}  // namespace b200ipc
