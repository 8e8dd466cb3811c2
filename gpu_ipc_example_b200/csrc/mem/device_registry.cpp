#include "device_registry.h"

#include <sstream>

#include <cuda.h>
#include <cuda_runtime_api.h>

#include "../common/check.h"
#include "../common/cu_driver.h"

namespace b200ipc {

std::vector<DeviceInfo> list_devices() {
  int n = 0;
  B200_CUDA_CHECK(cudaGetDeviceCount(&n));
  std::vector<DeviceInfo> out;
  for (int i = 0; i < n; ++i) {
    cudaDeviceProp p;
    B200_CUDA_CHECK(cudaGetDeviceProperties(&p, i));
    DeviceInfo d;
    d.index = i;
    d.name = p.name;
    d.sm_major = p.major;
    d.sm_minor = p.minor;
    d.sm_count = p.multiProcessorCount;
    d.total_mem = p.totalGlobalMem;
    d.l2_bytes = size_t(p.l2CacheSize);
    d.max_smem_per_block = int(p.sharedMemPerBlockOptin);
    char bus[32] = {0};
    if (cudaDeviceGetPCIBusId(bus, sizeof(bus), i) == cudaSuccess) d.pci_bus_id = bus;
    CUdevice dev;
    if (driver_available() && cu().DeviceGet(&dev, i) == CUDA_SUCCESS) {
      int v = 0;
      if (cu().DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS) d.multicast = v != 0;
      v = 0;
      if (cu().DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev) == CUDA_SUCCESS)
        d.posix_fd_handles = v != 0;
    }
    out.push_back(d);
  }
  return out;
}

std::vector<std::vector<int>> peer_matrix() {
  int n = 0;
  B200_CUDA_CHECK(cudaGetDeviceCount(&n));
  std::vector<std::vector<int>> m(static_cast<size_t>(n), std::vector<int>(static_cast<size_t>(n), 0));
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) {
      if (i == j) {
        m[size_t(i)][size_t(j)] = 1;
        continue;
      }
      int ok = 0;
      B200_CUDA_CHECK(cudaDeviceCanAccessPeer(&ok, i, j));
      m[size_t(i)][size_t(j)] = ok;
    }
  return m;
}

std::string describe_devices() {
  std::ostringstream os;
  auto devs = list_devices();
  for (const DeviceInfo& d : devs) {
    os << "[" << d.index << "] " << d.name << "  sm_" << d.sm_major << d.sm_minor << "  " << d.sm_count << " SMs  "
       << (d.total_mem >> 20) << " MiB  L2 " << (d.l2_bytes >> 20) << " MiB  smem/CTA " << (d.max_smem_per_block >> 10)
       << " KiB  multicast " << (d.multicast ? "yes" : "no") << "  fd-handles " << (d.posix_fd_handles ? "yes" : "no")
       << "  " << d.pci_bus_id << "\n";
  }
  if (devs.size() > 1) {
    os << "peer access:\n";
    auto m = peer_matrix();
    for (size_t i = 0; i < m.size(); ++i) {
      os << "  " << i << ":";
      for (int v : m[i]) os << " " << v;
      os << "\n";
    }
  }
  return os.str();
}

int device_for_rank(const std::string& device_list, int rank, int device_count) {
  std::vector<int> ids;
  if (device_list.find(',') != std::string::npos) {
    std::stringstream ss(device_list);
    std::string tok;
    while (std::getline(ss, tok, ',')) {
      B200_REQUIRE(!tok.empty(), "empty entry in device list '" << device_list << "'");
      ids.push_back(std::stoi(tok));
    }
  } else {
    for (char c : device_list) {
      B200_REQUIRE(c >= '0' && c <= '9', "device list '" << device_list << "' must be digits");
      ids.push_back(c - '0');
    }
  }
  B200_REQUIRE(rank >= 0 && size_t(rank) < ids.size(), "device list '" << device_list << "' has no entry for rank " << rank);
  int d = ids[size_t(rank)];
  B200_REQUIRE(d >= 0 && d < device_count, "rank " << rank << " was assigned device " << d << " but only " << device_count
                                                   << " device(s) are visible");
  return d;
}

}  // namespace b200ipc
