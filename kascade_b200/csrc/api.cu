// Library-level entry points: init, error text, ABI version.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace kb200 {

static thread_local char g_err[1024] = "";
static int g_sm_count = 0;
static int g_device = -1;

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int sm_count() { return g_sm_count > 0 ? g_sm_count : 148; }

bool initialised(int* device_out) {
  if (device_out) *device_out = g_device;
  return g_device >= 0;
}

}  // namespace kb200

extern "C" int kb200_abi_version(void) { return 1; }

extern "C" const char* kb200_last_error(void) { return kb200::g_err; }

extern "C" int kb200_init(int device) {
  cudaDeviceProp prop;
  KB_CUDA(cudaGetDeviceProperties(&prop, device));
  KB_REQUIRE(prop.major == 10, "device %d is sm_%d%d; this library contains sm_100a code only",
             device, prop.major, prop.minor);
  KB_CUDA(cudaSetDevice(device));
  kb200::g_sm_count = prop.multiProcessorCount;
  if (kb200::init_decode() != 0) return -1;
  if (kb200::init_prefill() != 0) return -1;
  if (kb200::init_selftest() != 0) return -1;
  kb200::g_device = device;
  return 0;
}
