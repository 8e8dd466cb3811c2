// Prints the visible GPUs, what they support and who can address whom.
// Capability parity: list_device.cpp:1-14.
#include <cstdio>
#include <exception>

#include "../mem/device_registry.h"

int main() {
  try {
    std::fputs(b200ipc::describe_devices().c_str(), stdout);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "%s\n", e.what());
    return 1;
  }
  return 0;
}
