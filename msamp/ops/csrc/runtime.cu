// Host-side runtime pieces shared by all kernels: last-error text, the device status word and
// cached device properties.
#include <stdarg.h>
#include <stdio.h>

#include <mutex>

#include "common.cuh"

static thread_local char g_error[512] = "";

void msamp_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int msamp_check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    msamp_set_error("%s: %s", what, cudaGetErrorString(e));
    return MSAMP_ELAUNCH;
  }
  return MSAMP_OK;
}

static unsigned int* g_status = nullptr;
static std::mutex g_mutex;

unsigned int* msamp_device_status_ptr() {
  if (!g_status) {
    std::lock_guard<std::mutex> lk(g_mutex);
    if (!g_status) {
      unsigned int* p = nullptr;
      // Pinned, mapped and portable: every device of the process can write it, the host reads it
      // without a copy even while a kernel is still running.
      if (cudaHostAlloc((void**)&p, 64, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
        for (int i = 0; i < 16; ++i) p[i] = 0;
        g_status = p;
      }
    }
  }
  return g_status;
}

int msamp_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

MSAMP_API const char* msamp_last_error() { return g_error; }

// Returns the accumulated device status bits and clears them. Bit 0: a bounded wait in a GEMM
// pipeline gave up; bit 1: a peer-flag wait gave up; bit 2: an attention pipeline wait gave up; bit 3: the ranks'
// sequences of fused calls ran out of step (a peer's flag was ahead of this rank's epoch); bit 4: a wait on the bulk-copy
// ring of a streaming kernel (LayerNorm backward) gave up.
MSAMP_API unsigned int msamp_read_device_status() {
  unsigned int* p = msamp_device_status_ptr();
  if (!p) return 0;
  unsigned int v = *(volatile unsigned int*)p;
  *(volatile unsigned int*)p = 0;
  return v;
}

// Same word without clearing it: a plain host read of mapped memory, cheap enough to call before every launch.
MSAMP_API unsigned int msamp_peek_device_status() {
  unsigned int* p = msamp_device_status_ptr();
  return p ? *(volatile unsigned int*)p : 0u;
}

MSAMP_API int msamp_device_sm_count() { return msamp_sm_count(); }

MSAMP_API int msamp_version() { return 100; }
