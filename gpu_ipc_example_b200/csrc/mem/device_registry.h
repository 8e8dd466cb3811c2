// Device selection and inventory.
//
// Capability parity: the per-tile queue registry and the -l device string
// (sycl_misc.hpp:6-40, sycl_misc.cpp:3-54, main.cpp:226-227) and the device
// lister (list_device.cpp:1-14).  On CUDA a rank's "queue" is simply a device
// ordinal plus the caller's stream, so the registry reduces to the mapping
// rank -> device and a description of what is installed.
#pragma once

#include <string>
#include <vector>

namespace b200ipc {

struct DeviceInfo {
  int index = 0;
  std::string name;
  int sm_major = 0, sm_minor = 0;
  int sm_count = 0;
  size_t total_mem = 0;
  size_t l2_bytes = 0;
  int max_smem_per_block = 0;
  bool multicast = false;       // NVLS capable
  bool posix_fd_handles = false;
  std::string pci_bus_id;
};

std::vector<DeviceInfo> list_devices();
// peer[i][j] != 0 when device i can address device j's memory.
std::vector<std::vector<int>> peer_matrix();
std::string describe_devices();

// The -l option: one decimal digit per rank ("012345678" by default, as in the
// reference).  A longer form "0,1,2,3" is accepted too.  Throws when the rank has
// no entry or the device does not exist.
int device_for_rank(const std::string& device_list, int rank, int device_count);

}  // namespace b200ipc
