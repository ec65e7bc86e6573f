// Host-side state shared by the tensor-core launchers, kept per device: the address of the device
// status word, the SM count, and which kernels already carry their dynamic shared-memory limit.
// A process may drive several GPUs from several threads; everything here is safe for that.
#include <mutex>
#include <utility>
#include <vector>
#include "common.cuh"
#include "launch.h"

namespace flare {

// Bit 0 is set by a tensor-core kernel that gave up on a bounded wait (tc::kErrWaitTimeout).
__device__ int g_tc_status = 0;

namespace {

constexpr int kMaxDevices = 64;

struct DeviceState {
  std::once_flag once;
  int* status = nullptr;
  int sms = 0;
};
DeviceState g_dev[kMaxDevices];

std::mutex g_attr_mutex;
std::vector<std::pair<const void*, int>> g_attr_done;   // (kernel, device) pairs already configured

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

DeviceState* device_state() {
  const int dev = current_device();
  if (dev < 0) return nullptr;
  DeviceState& d = g_dev[dev];
  std::call_once(d.once, [&] {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_tc_status) == cudaSuccess) d.status = static_cast<int*>(p);
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    d.sms = n;
  });
  return &d;
}

}  // namespace

int* tc_status_ptr() {
  DeviceState* d = device_state();
  return d ? d->status : nullptr;
}

int num_sms() {
  DeviceState* d = device_state();
  return d ? d->sms : 148;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a property of (kernel, device context): set once for each.
int tc_set_dyn_smem(const void* kernel, int bytes) {
  const int dev = current_device();
  if (dev < 0) return FLARE_ECUDA;
  std::lock_guard<std::mutex> lock(g_attr_mutex);
  for (const auto& e : g_attr_done)
    if (e.first == kernel && e.second == dev) return FLARE_OK;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return FLARE_ECUDA;
  g_attr_done.emplace_back(kernel, dev);
  return FLARE_OK;
}

int tc_read_status(int* out, bool clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return FLARE_ECUDA;
  if (clear && v) {
    int z = 0;
    if (cudaMemcpyToSymbol(g_tc_status, &z, sizeof(int)) != cudaSuccess) return FLARE_ECUDA;
  }
  *out = v;
  return FLARE_OK;
}

}  // namespace flare
