// Host-side helpers shared by the entry points: launch geometry, error text, fault injection.
#pragma once
#include <atomic>

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../include/arcsample.h"

namespace arcs {

constexpr int kSmCount = 148;  // B200
constexpr int kMaxSeg = 64;

// How a [rows][V] problem is cut into CTAs: each row is split into nseg segments of seg_len
// elements (a multiple of 2048, at least 8192) so that about per_sm work items per SM exist even
// when there are few rows (four for the argmax grid; one for the persistent stream kernel of the
// sampler, whose finishing step pays for every segment it has to merge). The same function sizes
// the workspaces, so it depends on (rows, V) only.
inline void plan_segments(int rows, int V, int* nseg, int* seg_len, int per_sm = 4) {
  const int target = kSmCount * per_sm;
  int want = (target + rows - 1) / rows;
  if (want < 1) want = 1;
  if (want > kMaxSeg) want = kMaxSeg;
  int len = (V + want - 1) / want;
  len = ((len + 2047) / 2048) * 2048;
  if (len < 8192) len = 8192;
  *seg_len = len;
  *nseg = (V + len - 1) / len;
}

char* error_buffer();  // thread-local, 256 bytes
inline int set_error(int code, const char* what) {
  snprintf(error_buffer(), 256, "%s", what);
  return code;
}
inline int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return ARCS_OK;
  snprintf(error_buffer(), 256, "%s: %s", what, cudaGetErrorString(e));
  return ARCS_ERR_CUDA;
}
// Raises a kernel's dynamic shared-memory limit once per device and process (the attribute belongs
// to the device's context; setting it costs microseconds, which a small batch notices on every
// call). `done`: one bit per device, owned by the call site.
template <typename K>
inline cudaError_t ensure_dynamic_smem(K kernel, int bytes, std::atomic<unsigned long long>& done) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const unsigned long long bit = 1ull << (dev & 63);
  if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
  return e;
}

// Host-side fault injection (no device is ever faulted): with ARCS_FAIL_CALL=N in the
// environment the N-th entry-point call of the process returns ARCS_ERR_INJECTED before
// anything is launched. Returns 0 when the call should proceed.
int fault_injected();

}  // namespace arcs
