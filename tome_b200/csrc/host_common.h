// Host-side helpers shared by the C-ABI entry points: error text, argument checks,
// per-device properties.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/tome_b200.h"

namespace tome {

// Records the detail text returned by tome_last_error_string() and passes `status` through.
int32_t fail(int32_t status, const char* fmt, ...);

// Maps a cudaError_t to TOME_OK / TOME_ERR_CUDA and records its text.
int32_t check_cuda(cudaError_t e, const char* what);

struct DeviceInfo {
  int device;
  int sm_count;
  int max_smem_optin;
  int cc_major;
};

// Properties of the current device (cached per device id; thread-safe).
int32_t current_device_info(DeviceInfo* out);

// How many clusters of `cluster` CTAs (threads x dyn_smem each) of `kernel` the current device
// can hold at once; 0 if the query fails.  Cached per (device, kernel, cluster); thread-safe.
int max_active_clusters(const void* kernel, int threads, int dyn_smem, int cluster);

// Makes sure `kernel` may be launched with `bytes` of dynamic shared memory on the current
// device.  The attribute is set once per (device, kernel) and remembered (thread-safe), which
// keeps cudaFuncSetAttribute out of the per-call path.
int32_t ensure_dynamic_smem(const void* kernel, int bytes);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline bool temperature_ok(float t) { return t > 0.0f && t <= 3.0e38f; }

constexpr float LOG2E = 1.4426950408889634f;

}  // namespace tome
