// Version, status text and per-device property cache of the C ABI.
#include <mutex>
#include <vector>

#include "host_common.h"
#include "ptx.cuh"

namespace tome {

static thread_local char g_last_error[512] = "";

int32_t fail(int32_t status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return status;
}

int32_t check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return TOME_OK;
  return fail(TOME_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

int32_t current_device_info(DeviceInfo* out) {
  constexpr int MAX_DEV = 64;
  static std::mutex mu;
  static DeviceInfo cache[MAX_DEV];
  static bool valid[MAX_DEV] = {false};
  int dev = 0;
  int32_t st = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (st != TOME_OK) return st;
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < MAX_DEV && valid[dev]) {
    *out = cache[dev];
    return TOME_OK;
  }
  DeviceInfo info;
  info.device = dev;
  st = check_cuda(cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev),
                  "cudaDeviceGetAttribute(sm count)");
  if (st != TOME_OK) return st;
  st = check_cuda(
      cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev),
      "cudaDeviceGetAttribute(smem optin)");
  if (st != TOME_OK) return st;
  st = check_cuda(cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, dev),
                  "cudaDeviceGetAttribute(cc major)");
  if (st != TOME_OK) return st;
  if (dev >= 0 && dev < MAX_DEV) {
    cache[dev] = info;
    valid[dev] = true;
  }
  *out = info;
  return TOME_OK;
}

int32_t ensure_dynamic_smem(const void* kernel, int bytes) {
  struct Entry {
    int device;
    const void* kernel;
    int bytes;
  };
  static std::mutex mu;
  static std::vector<Entry> cache;
  int dev = 0;
  int32_t st = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
  if (st != TOME_OK) return st;
  std::lock_guard<std::mutex> lock(mu);
  for (Entry& e : cache) {
    if (e.device != dev || e.kernel != kernel) continue;
    if (e.bytes >= bytes) return TOME_OK;
    st = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes),
                    "cudaFuncSetAttribute(dynamic shared memory)");
    if (st == TOME_OK) e.bytes = bytes;
    return st;
  }
  st = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes),
                  "cudaFuncSetAttribute(dynamic shared memory)");
  if (st == TOME_OK) cache.push_back({dev, kernel, bytes});
  return st;
}

int max_active_clusters(const void* kernel, int threads, int dyn_smem, int cluster) {
  struct Entry {
    int device;
    const void* kernel;
    int cluster;
    int value;
  };
  static std::mutex mu;
  static std::vector<Entry> cache;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const Entry& e : cache)
      if (e.device == dev && e.kernel == kernel && e.cluster == cluster) return e.value;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(cluster), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(dyn_smem);
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = static_cast<unsigned>(cluster);
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();  // the query's failure is not the caller's error
    n = 0;
  }
  std::lock_guard<std::mutex> lock(mu);
  cache.push_back({dev, kernel, cluster, n});
  return n;
}

}  // namespace tome

namespace tome {

// Waits on an mbarrier that nothing ever arrives on, with a short limit: exercises the path
// every bounded wait of the library takes when it runs out (status bit, normal kernel exit).
__global__ void selftest_bounded_wait_kernel(long long limit_cycles, int32_t* status,
                                             int32_t* waited_out) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t addr = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(addr, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool completed = mbar_wait(addr, 0, limit_cycles);
    if (!completed && status != nullptr) atomicOr(status, TOME_DEV_TIMEOUT);
    if (waited_out != nullptr) *waited_out = completed ? 0 : 1;
  }
}

}  // namespace tome

extern "C" int32_t tome_selftest_bounded_wait(int64_t limit_cycles, int32_t* dev_status,
                                              int32_t* out_gave_up, void* stream) {
  using namespace tome;
  if (limit_cycles <= 0 || limit_cycles > 2000000000LL)
    return fail(TOME_ERR_BAD_SHAPE, "limit_cycles=%lld must be in (0, 2e9]",
                (long long)limit_cycles);
  selftest_bounded_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      limit_cycles, dev_status, out_gave_up);
  return check_cuda(cudaGetLastError(), "selftest launch");
}

extern "C" {

int32_t tome_version(void) { return TOME_B200_VERSION; }

const char* tome_status_string(int32_t status) {
  switch (status) {
    case TOME_OK: return "TOME_OK";
    case TOME_ERR_NULL_POINTER: return "TOME_ERR_NULL_POINTER";
    case TOME_ERR_MISALIGNED: return "TOME_ERR_MISALIGNED";
    case TOME_ERR_BAD_DTYPE: return "TOME_ERR_BAD_DTYPE";
    case TOME_ERR_BAD_SHAPE: return "TOME_ERR_BAD_SHAPE";
    case TOME_ERR_BAD_STRIDE: return "TOME_ERR_BAD_STRIDE";
    case TOME_ERR_WORKSPACE_TOO_SMALL: return "TOME_ERR_WORKSPACE_TOO_SMALL";
    case TOME_ERR_BAD_TEMPERATURE: return "TOME_ERR_BAD_TEMPERATURE";
    case TOME_ERR_UNSUPPORTED: return "TOME_ERR_UNSUPPORTED";
    case TOME_ERR_TOO_LARGE: return "TOME_ERR_TOO_LARGE";
    case TOME_ERR_CUDA: return "TOME_ERR_CUDA";
    default: return "TOME_STATUS_UNKNOWN";
  }
}

const char* tome_last_error_string(void) { return tome::g_last_error; }

}  // extern "C"
