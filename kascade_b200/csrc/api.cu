// Library-level entry points: init, error text, ABI version.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace kb200 {

static thread_local char g_err[1024] = "";
// per-device state, indexed by the CUDA ordinal: a process may drive several GPUs
constexpr int kMaxDevices = 64;
static int g_sm_count[kMaxDevices] = {};
static bool g_inited[kMaxDevices] = {};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  return (dev >= 0 && dev < kMaxDevices) ? dev : -1;
}

int sm_count() {
  const int dev = current_device();
  return (dev >= 0 && g_sm_count[dev] > 0) ? g_sm_count[dev] : 148;
}

// true when kb200_init has run for the device that is current in the calling thread
bool initialised(int* device_out) {
  const int dev = current_device();
  if (device_out) *device_out = dev;
  return dev >= 0 && g_inited[dev];
}

// Rejects a pointer that belongs to another GPU than the current one: launching on device X with
// device-Y pointers is an illegal-address fault (or, with peer access on, silently slow).
int check_on_current_device(const void* ptr, const char* what) {
  if (!ptr) return 0;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
    cudaGetLastError();
    return 0;                                            // not a CUDA allocation the runtime knows: let the launch decide
  }
  if (attr.type != cudaMemoryTypeDevice) return 0;
  const int dev = current_device();
  KB_REQUIRE(attr.device == dev,
             "%s lives on device %d but the calling thread's current device is %d; make the tensors' device current "
             "(cudaSetDevice) before the call", what, attr.device, dev);
  return 0;
}

}  // namespace kb200

extern "C" int kb200_abi_version(void) { return 2; }

extern "C" const char* kb200_last_error(void) { return kb200::g_err; }

extern "C" int kb200_init(int device) {
  cudaDeviceProp prop;
  KB_CUDA(cudaGetDeviceProperties(&prop, device));
  KB_REQUIRE(prop.major == 10, "device %d is sm_%d%d; this library contains sm_100a code only",
             device, prop.major, prop.minor);
  KB_REQUIRE(device >= 0 && device < kb200::kMaxDevices, "device ordinal %d out of range", device);
  // the per-kernel attributes are set for the device that is current: switch, set, switch back
  int prev = -1;
  KB_CUDA(cudaGetDevice(&prev));
  KB_CUDA(cudaSetDevice(device));
  int rc = 0;
  if (kb200::init_decode() != 0 || kb200::init_prefill() != 0 || kb200::init_selftest() != 0) rc = -1;
  if (prev != device) cudaSetDevice(prev);
  if (rc != 0) return -1;
  kb200::g_sm_count[device] = prop.multiProcessorCount;
  kb200::g_inited[device] = true;
  return 0;
}
