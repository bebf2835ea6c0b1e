// Status strings, last-error text, device checks.
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace amoe {
static thread_local char g_last_error[512] = "";

void set_last_error(const char* what, cudaError_t err) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", what, cudaGetErrorName(err), cudaGetErrorString(err));
}

static thread_local unsigned long long g_launches = 0;
void note_launch() { ++g_launches; }
unsigned long long launches_so_far() { return g_launches; }

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}
}  // namespace amoe

extern "C" {

int amoe_version(void) { return 100; }

const char* amoe_status_string(int status) {
  switch (status) {
    case AMOE_OK: return "ok";
    case AMOE_ERR_BAD_SHAPE: return "bad shape: a size is non-positive or violates a documented limit";
    case AMOE_ERR_BAD_DTYPE: return "bad dtype";
    case AMOE_ERR_NULL_POINTER: return "a required pointer is NULL";
    case AMOE_ERR_WORKSPACE: return "workspace missing or too small";
    case AMOE_ERR_CUDA: return "CUDA call failed";
    case AMOE_ERR_UNSUPPORTED: return "unsupported combination of options";
    case AMOE_ERR_DEVICE: return "current device is not an sm_100 GPU";
    case AMOE_ERR_INDEX_RANGE: return "device-side check: index out of range";
    case AMOE_ERR_WAIT_LIMIT: return "device-side bounded wait gave up";
    default: return "unknown status";
  }
}

const char* amoe_last_error_string(void) { return amoe::g_last_error; }

unsigned long long amoe_launch_count(void) { return amoe::launches_so_far(); }

int amoe_check_device(void) {
  int dev = 0;
  AMOE_CUDA(cudaGetDevice(&dev));
  int major = 0;
  AMOE_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  return major == 10 ? AMOE_OK : AMOE_ERR_DEVICE;
}

int amoe_read_device_status(const int32_t* dev_status, int32_t host_copy[4], amoe_stream_t stream) {
  AMOE_REQUIRE(dev_status != nullptr && host_copy != nullptr, AMOE_ERR_NULL_POINTER);
  AMOE_CUDA(cudaMemcpyAsync(host_copy, dev_status, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost,
                            reinterpret_cast<cudaStream_t>(stream)));
  AMOE_CUDA(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  return host_copy[0];
}

}  // extern "C"
