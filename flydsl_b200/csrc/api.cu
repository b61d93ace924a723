// Host-side plumbing of libflyb200: thread-local error text, per-device cached properties and the
// device error word that kernels write when a bounded wait runs out.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace flyb200 {

// One word per device; kernels atomicCAS a DeviceError code (| blockIdx << 8) into it.
__device__ int g_error_word[4];

static thread_local char tl_error[512] = "";

int set_error(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
  return status;
}

constexpr int kMaxDevices = 64;

int* device_error_word() {
  static int* cache[kMaxDevices] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error(FLYB200_ERR_CUDA, "cudaGetDevice failed");
    return nullptr;
  }
  if (!cache[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_error_word);
    if (e != cudaSuccess) {
      set_error(FLYB200_ERR_CUDA, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cache[dev] = static_cast<int*>(ptr);
  }
  return cache[dev];
}

int sm_count() {
  static int cache[kMaxDevices] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error(FLYB200_ERR_CUDA, "cudaGetDevice failed");
    return -1;
  }
  if (!cache[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      set_error(FLYB200_ERR_CUDA, "cannot read the SM count");
      return -1;
    }
    cache[dev] = n;
  }
  return cache[dev];
}

}  // namespace flyb200

using namespace flyb200;

extern "C" const char* flyb200_last_error_string(void) { return tl_error; }

extern "C" int flyb200_version(void) { return 100; }

extern "C" int flyb200_query_device_error(void* stream, int32_t* code_out) {
  if (!code_out) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "code_out is NULL");
  int* word = device_error_word();
  if (!word) return FLYB200_ERR_CUDA;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int host = 0;
  FLYB200_CUDA_CHECK(cudaMemcpyAsync(&host, word, sizeof(int), cudaMemcpyDeviceToHost, st));
  FLYB200_CUDA_CHECK(cudaStreamSynchronize(st));
  if (host != 0) {
    FLYB200_CUDA_CHECK(cudaMemsetAsync(word, 0, sizeof(int), st));
    FLYB200_CUDA_CHECK(cudaStreamSynchronize(st));
  }
  *code_out = host;
  if (host != 0)
    return set_error(FLYB200_ERR_DEVICE_TIMEOUT,
                     "a kernel gave up on a bounded wait: code %d in CTA %d", host & 0xFF, host >> 8);
  return FLYB200_OK;
}
