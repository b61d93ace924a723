// Weight repack for the tcgen05 kernels. The reference preshuffles weights for AMD MFMA lanes
// (shuffle_weight, tests/utils.py:76-96: [N/16][K/64][4][16][16 B]); here the one-time repack writes
// the exact shared-memory image the B200 tensor core reads:
//
//   dst[batch][kb = K/128][atom = N/8][r = 8][128 B],  16-byte chunk c of row r stored at c ^ r
//
// i.e. K-major rows of 128 bytes with the 128-byte swizzle already applied, 8-row atoms contiguous
// along N. For one K block, any run of rows n0..n0+R (R % 8 == 0) is one contiguous R*128-byte
// range, so a CTA brings a whole weight tile with a single bulk copy and HBM sees long sequential
// bursts. Byte count is unchanged (N*K per batch item).
#include "common.cuh"

namespace flyb200 {

__global__ void __launch_bounds__(256)
repack_weight_fp8_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int64_t batch,
                         int64_t N, int64_t K) {
  const int64_t chunks_per_row = K / 16;
  const int64_t per_batch = N * chunks_per_row;
  const int64_t total = batch * per_batch;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t b = i / per_batch;
    const int64_t rem = i - b * per_batch;
    const int64_t n = rem / chunks_per_row;
    const int64_t kc16 = rem - n * chunks_per_row;  // 16-byte chunk index along K
    const int64_t kb = kc16 >> 3;
    const int c = static_cast<int>(kc16 & 7);
    const int r = static_cast<int>(n & 7);
    const int64_t atom = n >> 3;
    const int64_t d = b * per_batch + ((kb * (N >> 3) + atom) * 8 + r) * 8 + (c ^ r);
    dst[d] = src[i];
  }
}

}  // namespace flyb200

using namespace flyb200;

extern "C" int flyb200_repack_weight_fp8(void* dst, const void* src, int64_t batch, int64_t N,
                                         int64_t K, void* stream) {
  if (!dst || !src) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "dst/src is NULL");
  if (dst == src) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "repack cannot run in place");
  if ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "dst and src must be 16-byte aligned");
  if (batch < 1 || N < 8 || K < 128 || N % 8 || K % 128)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "repack needs batch >= 1, N %% 8 == 0, K %% 128 == 0 (batch=%lld N=%lld K=%lld)",
                     static_cast<long long>(batch), static_cast<long long>(N),
                     static_cast<long long>(K));
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const int64_t total = batch * N * (K / 16);
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sms) * 16;
  if (blocks > cap) blocks = cap;
  repack_weight_fp8_kernel<<<static_cast<int>(blocks), 256, 0,
                             reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<uint4*>(dst), reinterpret_cast<const uint4*>(src), batch, N, K);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}
