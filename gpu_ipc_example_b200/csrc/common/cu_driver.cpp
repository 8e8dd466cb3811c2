#include "cu_driver.h"

#include <mutex>
#include <string>

#include <cuda_runtime_api.h>

#include "check.h"

namespace b200ipc {
namespace {

DriverApi g_api{};
bool g_ok = false;
std::string g_why;
std::once_flag g_once;

template <typename Fn>
bool resolve(const char* name, Fn* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || p == nullptr || q != cudaDriverEntryPointSuccess) {
    cudaGetLastError();
    if (g_why.empty()) g_why = std::string("driver entry point ") + name + " not available";
    return false;
  }
  *out = reinterpret_cast<Fn>(p);
  return true;
}

void load_all() {
  bool ok = true;
#define B200_RESOLVE(field, sym) ok = resolve(sym, &g_api.field) && ok
  B200_RESOLVE(GetErrorName, "cuGetErrorName");
  B200_RESOLVE(GetErrorString, "cuGetErrorString");
  B200_RESOLVE(DeviceGet, "cuDeviceGet");
  B200_RESOLVE(DeviceGetAttribute, "cuDeviceGetAttribute");
  B200_RESOLVE(MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
  B200_RESOLVE(MemCreate, "cuMemCreate");
  B200_RESOLVE(MemRelease, "cuMemRelease");
  B200_RESOLVE(MemExportToShareableHandle, "cuMemExportToShareableHandle");
  B200_RESOLVE(MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
  B200_RESOLVE(MemAddressReserve, "cuMemAddressReserve");
  B200_RESOLVE(MemAddressFree, "cuMemAddressFree");
  B200_RESOLVE(MemMap, "cuMemMap");
  B200_RESOLVE(MemUnmap, "cuMemUnmap");
  B200_RESOLVE(MemSetAccess, "cuMemSetAccess");
  B200_RESOLVE(MulticastCreate, "cuMulticastCreate");
  B200_RESOLVE(MulticastAddDevice, "cuMulticastAddDevice");
  B200_RESOLVE(MulticastBindMem, "cuMulticastBindMem");
  B200_RESOLVE(MulticastUnbind, "cuMulticastUnbind");
  B200_RESOLVE(MulticastGetGranularity, "cuMulticastGetGranularity");
  B200_RESOLVE(TensorMapEncodeTiled, "cuTensorMapEncodeTiled");
#undef B200_RESOLVE
  g_ok = ok;
}

}  // namespace

bool driver_available() {
  std::call_once(g_once, load_all);
  return g_ok;
}

const DriverApi& cu() {
  std::call_once(g_once, load_all);
  if (!g_ok) throw Error("[b200ipc] CUDA driver not usable: " + g_why);
  return g_api;
}

std::string cu_error_string(CUresult r) {
  const char* name = nullptr;
  const char* desc = nullptr;
  if (driver_available()) {
    g_api.GetErrorName(r, &name);
    g_api.GetErrorString(r, &desc);
  }
  std::ostringstream os;
  os << (name ? name : "CUDA_ERROR_?") << " (" << static_cast<int>(r) << "): " << (desc ? desc : "");
  return os.str();
}

}  // namespace b200ipc
