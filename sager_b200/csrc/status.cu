// status.cu - the library's device status word and version query.
#include "api_util.cuh"
#include "q4k_common.cuh"

namespace sgr {
namespace {
__device__ int g_status;
constexpr int kMaxDevices = 64;
int* g_status_addr[kMaxDevices];
}  // namespace

int* status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_status_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status) != cudaSuccess) return nullptr;
    g_status_addr[dev] = static_cast<int*>(p);
  }
  return g_status_addr[dev];
}
}  // namespace sgr

// Reads (and clears when `clear` != 0) the status word of the current device.
// 0 = no device-side wait ever gave up. Synchronises the device: diagnostics
// only, never on the hot path.
SGR_API int sgr_status(int clear) {
  int v = 0;
  int* p = sgr::status_word();
  if (p == nullptr) return -1;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (clear && v != 0) {
    const int z = 0;
    cudaMemcpy(p, &z, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}

SGR_API int sgr_abi_version(void) { return 4; }
