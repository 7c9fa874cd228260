// Error reporting and the device status word of the C ABI.

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "vx_common.cuh"

namespace vx {
namespace {

thread_local char g_last_error[512] = "";

// One status word per device context; kernels report expired bounded waits here.
__device__ int g_device_status = 0;

}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("VELOX_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

int* device_status_ptr() {
  // cudaGetSymbolAddress answers for the CURRENT device; looked up once per device.
  static int* cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
  if (dev >= 0 && cache[dev]) return cache[dev];
  int* p = nullptr;
  if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_device_status) != cudaSuccess) return nullptr;
  if (dev >= 0) cache[dev] = p;
  return p;
}

}  // namespace vx

extern "C" {

const char* vx_last_error(void) { return vx::g_last_error; }

int vx_abi_version(void) { return VX_ABI_VERSION; }

int vx_device_status(int* status_out) {
  if (!status_out) return vx::fail(-1, "status_out must not be NULL");
  VX_CUDA_OK(cudaDeviceSynchronize());
  int* p = vx::device_status_ptr();
  if (!p) return vx::fail(-2, "device status word unavailable");
  VX_CUDA_OK(cudaMemcpy(status_out, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status_out != 0) {
    int zero = 0;
    VX_CUDA_OK(cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice));
  }
  return 0;
}

}  // extern "C"
