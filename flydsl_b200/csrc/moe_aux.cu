// Bandwidth-bound helpers around the MoE GEMMs:
//   * top-k reduce  Y[t,d] = sum_s X[t,s,d]           (compile_moe_reduction,
//                                                       kernels/moe_blockscale_2stage.py:2446-2638)
//   * 1x128 group quantiser to fp8 e4m3 with transposed scales (the re-quantisation between the
//     stages, tests/kernels/test_moe_blockscale.py:346-361 + pertoken_quant tests/utils.py:29-73)
#include <cuda_fp8.h>

#include <type_traits>

#include "common.cuh"

namespace flyb200 {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// One thread owns VEC consecutive d for one token and walks the k slots in order (fixed summation
// order => deterministic). 16-byte loads.
template <typename T>
__global__ void __launch_bounds__(256)
moe_reduce_kernel(const T* __restrict__ x, T* __restrict__ y, const uint8_t* __restrict__ mask,
                  int tokens, int k, int H) {
  constexpr int VEC = 16 / sizeof(T);
  const int vec_per_row = H / VEC;
  const int64_t total = static_cast<int64_t>(tokens) * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_row);
    const int v = static_cast<int>(i - static_cast<int64_t>(t) * vec_per_row);
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    for (int s = 0; s < k; ++s) {
      if (mask && mask[t * k + s] == 0) continue;
      const uint4 raw = *reinterpret_cast<const uint4*>(
          x + (static_cast<int64_t>(t) * k + s) * H + static_cast<int64_t>(v) * VEC);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] += to_f32<T>(e[j]);
    }
    uint4 outv;
    T* o = reinterpret_cast<T*>(&outv);
#pragma unroll
    for (int j = 0; j < VEC; ++j) o[j] = from_f32<T>(acc[j]);
    *reinterpret_cast<uint4*>(y + static_cast<int64_t>(t) * H + static_cast<int64_t>(v) * VEC) = outv;
  }
}

// 16-bit inputs: half a warp per 128-wide group (16 lanes x 16 bytes), so a warp moves 512 bytes per
// load instruction; the amax reduction stays inside the half-warp. `raw` holds the lane's 8 values
// (zeros for a lane without work). The kernel is bound by its instruction count, so the group's amax
// is taken on the packed 16-bit patterns: |v| as unsigned 16-bit integers order like the values, and
// anything at or above the pattern of +Inf is an Inf/NaN, so one and + one packed max per PAIR of
// elements finds both the amax and whether the rare clean-up path (NaN -> 0, +-Inf -> +-448, as
// pertoken_quant's nan_to_num does) is needed at all.
template <typename T>
__device__ __forceinline__ void quant_group16(const uint4& raw, uint8_t* __restrict__ q_dst,
                                              float* __restrict__ scale_dst, bool active, int sub) {
  constexpr uint32_t kInfBits = (sizeof(T) == 2 && std::is_same<T, __half>::value) ? 0x7c00u : 0x7f80u;
  const uint32_t m2 = __vmaxu2(__vmaxu2(raw.x & 0x7fff7fffu, raw.y & 0x7fff7fffu),
                               __vmaxu2(raw.z & 0x7fff7fffu, raw.w & 0x7fff7fffu));
  uint32_t amax_bits = max(m2 & 0xffffu, m2 >> 16);
#pragma unroll
  for (int o = 8; o > 0; o >>= 1)  // xor distances < 16 stay inside the half-warp
    amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, o));
  float v[8];
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = to_f32<T>(e[j]);
  float amax;
  if (__any_sync(0xffffffffu, amax_bits >= kInfBits)) {
    float vmax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (v[j] != v[j]) v[j] = 0.f;
      else if (isinf(v[j])) v[j] = v[j] > 0 ? 448.f : -448.f;
      vmax = fmaxf(vmax, fabsf(v[j]));
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    amax = vmax;
  } else if constexpr (std::is_same<T, __half>::value) {
    amax = __half2float(__ushort_as_half(static_cast<unsigned short>(amax_bits)));
  } else {
    amax = __uint_as_float(amax_bits << 16);
  }
  // Quotients from one reciprocal: q0 = y*rc, q = fma(fma(-d, q0, y), rc, q0) is the IEEE quotient
  // y/d when rc is the correctly rounded reciprocal of d, the mantissa of d is not all ones and
  // nothing is subnormal (Markstein); the rare other cases take the true division.
  float scale;
  {
    constexpr float kRc448 = 1.0f / 448.0f;   // correctly rounded by the compiler
    const float q0 = amax * kRc448;
    scale = __fmaf_rn(__fmaf_rn(-448.f, q0, amax), kRc448, q0);
  }
  const bool tiny = amax < 1e-30f;            // quotient or residual may be subnormal
  if (__any_sync(0xffffffffu, tiny)) scale = __fdiv_rn(amax, 448.f);
  if (scale == 0.f) scale = 1.f;
  if (active) {
    float qv[8];
    if (((__float_as_uint(scale) & 0x7fffffu) == 0x7fffffu) || tiny) {
#pragma unroll
      for (int j = 0; j < 8; ++j) qv[j] = __fdiv_rn(v[j], scale);
    } else {
      const float rc = __frcp_rn(scale);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float q0 = v[j] * rc;
        const float qc = __fmaf_rn(__fmaf_rn(-scale, q0, v[j]), rc, q0);
        // the sign of the input, for the one case the correction step loses it: -0 / scale = -0
        qv[j] = __uint_as_float(__float_as_uint(qc) | (__float_as_uint(v[j]) & 0x80000000u));
      }
    }
    const uint32_t lo = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[0], qv[1]), __NV_SATFINITE, __NV_E4M3)) |
                        (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[2], qv[3]), __NV_SATFINITE, __NV_E4M3)) << 16);
    const uint32_t hi = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[4], qv[5]), __NV_SATFINITE, __NV_E4M3)) |
                        (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[6], qv[7]), __NV_SATFINITE, __NV_E4M3)) << 16);
    *reinterpret_cast<uint2*>(q_dst) = make_uint2(lo, hi);
    if (sub == 0) *scale_dst = scale;
  }
}

// A warp takes whole rows (the input streams sequentially, no index arithmetic beyond additions),
// two groups per step (one per half-warp), four steps' loads in flight at once: a dependent load ->
// reduce -> divide -> store chain per group is latency-bound with one.
template <typename T>
__device__ __forceinline__ void quant_rows16(const T* __restrict__ x, uint8_t* __restrict__ q,
                                             float* __restrict__ scale_t, int64_t rows,
                                             int64_t scale_stride, int cols) {
  constexpr int kInFlight = 4;
  const int groups = cols / 128;
  const int lane = threadIdx.x & 31;
  const int sub = lane & 15;
  const int hw = lane >> 4;
  const int64_t warp0 = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t row = warp0; row < rows; row += nwarps) {
    const T* xrow = x + row * cols + sub * 8;
    uint8_t* qrow = q + row * cols + sub * 8;
    float* srow = scale_t + row;
    for (int g0 = 0; g0 < groups; g0 += 2 * kInFlight) {
      uint4 raw[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int g = g0 + 2 * u + hw;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (g < groups) raw[u] = *reinterpret_cast<const uint4*>(xrow + g * 128);
      }
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int g = g0 + 2 * u + hw;
        if (g0 + 2 * u < groups)   // warp-uniform: the shuffles inside need the whole warp
          quant_group16<T>(raw[u], qrow + g * 128, srow + static_cast<int64_t>(g) * scale_stride, g < groups, sub);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
quant_1x128_kernel16(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale_t,
                     int64_t rows, int cols) {
  quant_rows16<T>(x, q, scale_t, rows, rows, cols);
}

// One warp per (row, 128-wide group): lane owns 4 consecutive elements.
template <typename T>
__global__ void __launch_bounds__(256)
quant_1x128_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale_t,
                   int64_t rows, int cols) {
  const int groups = cols / 128;
  const int64_t total = rows * groups;
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t w = warp0; w < total; w += nwarps) {
    const int64_t row = w / groups;
    const int g = static_cast<int>(w - row * groups);
    const T* src = x + row * cols + g * 128 + lane * 4;
    float v[4];
    if constexpr (sizeof(T) == 4) {
      const float4 raw = *reinterpret_cast<const float4*>(src);
      v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
    } else {
      const uint2 raw = *reinterpret_cast<const uint2*>(src);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = to_f32<T>(e[j]);
    }
    // NaN -> 0, +-Inf -> +-448, as pertoken_quant's nan_to_num does.
    float vmax = -3.4e38f, vmin = 3.4e38f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (v[j] != v[j]) v[j] = 0.f;
      else if (isinf(v[j])) v[j] = v[j] > 0 ? 448.f : -448.f;
      vmax = fmaxf(vmax, v[j]);
      vmin = fminf(vmin, v[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
      vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
    }
    const float amax = fmaxf(vmax, -vmin);
    float scale = __fdiv_rn(amax, 448.f);
    if (scale == 0.f) scale = 1.f;
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_fp8_storage_t b =
          __nv_cvt_float_to_fp8(__fdiv_rn(v[j], scale), __NV_SATFINITE, __NV_E4M3);
      packed |= static_cast<uint32_t>(b) << (8 * j);
    }
    *reinterpret_cast<uint32_t*>(q + row * cols + g * 128 + lane * 4) = packed;
    if (lane == 0) scale_t[static_cast<int64_t>(g) * rows + row] = scale;
  }
}

}  // namespace flyb200

using namespace flyb200;

extern "C" int flyb200_moe_reduce(const void* x, void* y, const uint8_t* valid_mask, int32_t T,
                                  int32_t k, int32_t H, int32_t dtype, void* stream) {
  if (!x || !y) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_reduce: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_reduce: buffers must be 16-byte aligned");
  if (T < 0 || k < 1 || H < 8)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_reduce: bad sizes T=%d k=%d H=%d", T, k, H);
  const int vec = dtype == FLYB200_F32 ? 4 : 8;
  if (H % vec) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_reduce: H %% %d != 0", vec);
  if (T == 0) return FLYB200_OK;
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const int64_t total = static_cast<int64_t>(T) * (H / vec);
  int64_t blocks = (total + 255) / 256;
  if (blocks > static_cast<int64_t>(sms) * 16) blocks = static_cast<int64_t>(sms) * 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int g = static_cast<int>(blocks);
  switch (dtype) {
    case FLYB200_BF16:
      moe_reduce_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(
          static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), valid_mask, T, k, H);
      break;
    case FLYB200_F16:
      moe_reduce_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x),
                                                   static_cast<__half*>(y), valid_mask, T, k, H);
      break;
    case FLYB200_F32:
      moe_reduce_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(x),
                                                  static_cast<float*>(y), valid_mask, T, k, H);
      break;
    default:
      return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_reduce: bad dtype %d", dtype);
  }
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

extern "C" int flyb200_quant_1x128(const void* x, void* q, float* scale_t, int64_t rows,
                                   int32_t cols, int32_t in_dtype, void* stream) {
  if (!x || !q || !scale_t) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(x) % 16) || (reinterpret_cast<uintptr_t>(q) % 8))
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant: x must be 16-byte, q 8-byte aligned");
  if (rows < 0 || cols < 128 || cols % 128)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant: cols (%d) must be a multiple of 128", cols);
  if (rows == 0) return FLYB200_OK;
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const int64_t warps = rows * (cols / 128);
  int64_t blocks = (warps + 7) / 8;
  if (blocks > static_cast<int64_t>(sms) * 16) blocks = static_cast<int64_t>(sms) * 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int g = static_cast<int>(blocks);
  uint8_t* qo = static_cast<uint8_t*>(q);
  switch (in_dtype) {
    case FLYB200_BF16:
      quant_1x128_kernel16<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), qo,
                                                             scale_t, rows, cols);
      break;
    case FLYB200_F16:
      quant_1x128_kernel16<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x), qo, scale_t,
                                                      rows, cols);
      break;
    case FLYB200_F32:
      quant_1x128_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(x), qo, scale_t, rows,
                                                   cols);
      break;
    default:
      return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant: bad in_dtype %d", in_dtype);
  }
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

// ---------------------------------------------------------------------------------------------
// Activations into routing order: row i of the output is the activation row of sorted position i
// (zero for padding rows), with its 1x128 scales in the transposed layout [K/128, rows_out]. Lets
// the stage kernels fetch their A tiles with TMA instead of gathering rows (cfg.path bit 0).
namespace flyb200 {
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const uint4* __restrict__ x, const float* __restrict__ scale_t,
                       const int* __restrict__ sorted_ids, const int* __restrict__ num_valid,
                       uint4* __restrict__ x_out, float* __restrict__ scale_out_t, int rows_in,
                       int K, int topk, int rows_out, int by_slot, int nscale) {
  // nscale: scale rows per activation row (K/128 for 1x128 groups, 1 for per-token scales)
  const int chunks = K / 16;               // 16-byte chunks per row
  const int valid = min(num_valid[0], rows_out);
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = warp; i < valid; i += nwarps) {
    const int id = sorted_ids[i];
    const int t = id & 0xFFFFFF;
    const int slot = static_cast<unsigned>(id) >> 24;
    // source row: the token (stage 1) or the (token, slot) route (stage 2 style inputs)
    const long long src = by_slot ? static_cast<long long>(t) * topk + slot : t;
    const bool ok = by_slot ? (slot < topk && src < rows_in) : (t < rows_in);
    // four 16-byte loads per lane in flight (the copy is latency-bound otherwise)
    const uint4* srow = x + src * chunks;
    uint4* drow = x_out + static_cast<long long>(i) * chunks;
    for (int c0 = lane; c0 < chunks; c0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + 32 * u;
        v[u] = (ok && c < chunks) ? __ldg(srow + c) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + 32 * u;
        if (c < chunks) drow[c] = v[u];
      }
    }
  }
  // scales: one thread per (scale row s, sorted position i), i fastest, so that the stores to the
  // transposed output are coalesced (the reads are 4-byte gathers inside one row of scale_t)
  const long long total = static_cast<long long>(nscale) * valid;
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < total;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int s = static_cast<int>(j / valid);
    const int i = static_cast<int>(j - static_cast<long long>(s) * valid);
    const int id = sorted_ids[i];
    const int t = id & 0xFFFFFF;
    const int slot = static_cast<unsigned>(id) >> 24;
    const long long src = by_slot ? static_cast<long long>(t) * topk + slot : t;
    const bool ok = by_slot ? (slot < topk && src < rows_in) : (t < rows_in);
    scale_out_t[static_cast<long long>(s) * rows_out + i] =
        ok ? __ldg(scale_t + static_cast<long long>(s) * rows_in + src) : 0.f;
  }
}
}  // namespace flyb200

extern "C" int flyb200_moe_gather_rows(const void* x, const float* scale_t, const int32_t* sorted_ids,
                                       const int32_t* num_valid_ids, void* x_out, float* scale_out_t,
                                       int32_t rows_in, int32_t K, int32_t topk, int32_t rows_out,
                                       int32_t by_slot, void* stream) {
  if (!x || !scale_t || !sorted_ids || !num_valid_ids || !x_out || !scale_out_t)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_gather_rows: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(x_out)) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_gather_rows: x and x_out must be 16-byte aligned");
  if (rows_in < 1 || rows_out < 1 || K < 128 || K % 128 || topk < 1)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_gather_rows: bad sizes");
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  moe_gather_rows_kernel<<<sms * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), scale_t, sorted_ids, num_valid_ids, static_cast<uint4*>(x_out),
      scale_out_t, rows_in, K, topk, rows_out, by_slot ? 1 : 0, K / 128);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

// The same permutation for activations with ONE scale per row (the per-token-scale MoE): scale
// [rows_in] -> scale_out [rows_out].
extern "C" int flyb200_moe_gather_rows_pertoken(const void* x, const float* scale, const int32_t* sorted_ids,
                                                const int32_t* num_valid_ids, void* x_out, float* scale_out,
                                                int32_t rows_in, int32_t K, int32_t topk, int32_t rows_out,
                                                int32_t by_slot, void* stream) {
  if (!x || !scale || !sorted_ids || !num_valid_ids || !x_out || !scale_out)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_gather_rows_pertoken: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(x_out)) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_gather_rows_pertoken: x and x_out must be 16-byte aligned");
  if (rows_in < 1 || rows_out < 1 || K < 16 || K % 16 || topk < 1)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_gather_rows_pertoken: bad sizes");
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  moe_gather_rows_kernel<<<sms * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), scale, sorted_ids, num_valid_ids, static_cast<uint4*>(x_out), scale_out,
      rows_in, K, topk, rows_out, by_slot ? 1 : 0, 1);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

// ---------------------------------------------------------------------------------------------
// Whole-row quantiser (pertoken_quant of the reference, tests/utils.py:29-73, on 16-bit rows): one
// scale per row, scale = amax/448 (0 -> 1), q = x/scale; NaN -> 0, +-Inf -> +-448 first. One warp per
// row, two passes over the row (the second finds it in L1/L2). Used between the stages of the
// per-token-scale MoE, where the reference test calls the torch function on the host side.
namespace flyb200 {
template <typename T>
__global__ void __launch_bounds__(256)
quant_pertoken_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale,
                      const int* __restrict__ num_rows_dev, int64_t rows_alloc, int cols) {
  const int64_t rows = num_rows_dev ? min(static_cast<int64_t>(num_rows_dev[0]), rows_alloc) : rows_alloc;
  const int lane = threadIdx.x & 31;
  const int chunks = cols / 8;   // 16-byte chunks of 8 values
  const int64_t warp0 = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  auto clean = [](float v) -> float {
    if (v != v) return 0.f;
    if (isinf(v)) return v > 0 ? 448.f : -448.f;
    return v;
  };
  for (int64_t row = warp0; row < rows; row += nwarps) {
    const uint4* xrow = reinterpret_cast<const uint4*>(x + row * cols);
    float amax = 0.f;
    for (int c0 = lane; c0 < chunks; c0 += 128) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + 32 * u;
        raw[u] = c < chunks ? xrow[c] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(clean(to_f32<T>(e[j]))));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float sc = __fdiv_rn(amax, 448.f);
    if (sc == 0.f) sc = 1.f;
    // Quotients from one reciprocal: q0 = v*rc, q = fma(fma(-sc, q0, v), rc, q0) is the IEEE quotient
    // v/sc when rc is the correctly rounded reciprocal, the mantissa of sc is not all ones and
    // nothing is subnormal (Markstein); the other rows take the true division. The sign of v is put
    // back for the one case the correction step loses it (-0 / sc = -0).
    const bool true_div = ((__float_as_uint(sc) & 0x7fffffu) == 0x7fffffu) || amax < 1e-20f;
    const float rc = __frcp_rn(sc);
    uint2* qrow = reinterpret_cast<uint2*>(q + row * cols);
    for (int c = lane; c < chunks; c += 32) {
      const uint4 raw = xrow[c];
      const T* e = reinterpret_cast<const T*>(&raw);
      float qv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float v = clean(to_f32<T>(e[j]));
        if (true_div) {
          qv[j] = __fdiv_rn(v, sc);
        } else {
          const float q0 = v * rc;
          const float qc = __fmaf_rn(__fmaf_rn(-sc, q0, v), rc, q0);
          qv[j] = __uint_as_float(__float_as_uint(qc) | (__float_as_uint(v) & 0x80000000u));
        }
      }
      const uint32_t lo = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[0], qv[1]), __NV_SATFINITE, __NV_E4M3)) |
                          (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[2], qv[3]), __NV_SATFINITE, __NV_E4M3)) << 16);
      const uint32_t hi = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[4], qv[5]), __NV_SATFINITE, __NV_E4M3)) |
                          (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[6], qv[7]), __NV_SATFINITE, __NV_E4M3)) << 16);
      qrow[c] = make_uint2(lo, hi);
    }
    if (lane == 0) scale[row] = sc;
  }
}
}  // namespace flyb200

extern "C" int flyb200_quant_pertoken(const void* x, void* q, float* scale, const int32_t* num_rows_dev,
                                      int64_t rows, int32_t cols, int32_t in_dtype, void* stream) {
  if (!x || !q || !scale) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant_pertoken: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(x) % 16) || (reinterpret_cast<uintptr_t>(q) % 8))
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant_pertoken: x must be 16-byte, q 8-byte aligned");
  if (rows < 0 || cols < 8 || cols % 8)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant_pertoken: cols (%d) must be a multiple of 8", cols);
  if (in_dtype != FLYB200_BF16 && in_dtype != FLYB200_F16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant_pertoken: input must be BF16 or F16");
  if (rows == 0) return FLYB200_OK;
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  int64_t blocks = (rows + 7) / 8;
  if (blocks > static_cast<int64_t>(sms) * 16) blocks = static_cast<int64_t>(sms) * 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* qo = static_cast<uint8_t*>(q);
  if (in_dtype == FLYB200_BF16)
    quant_pertoken_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), qo, scale, num_rows_dev, rows, cols);
  else
    quant_pertoken_kernel<__half><<<static_cast<int>(blocks), 256, 0, st>>>(static_cast<const __half*>(x), qo,
                                                                            scale, num_rows_dev, rows, cols);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

// 1x128 quantiser over the first num_rows_dev[0] rows only (row count known on the device, e.g. the
// padded route count of the sorter); scales go to [cols/128, rows_alloc].
namespace flyb200 {
template <typename T>
__global__ void __launch_bounds__(256)
quant_1x128_devrows_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale_t,
                           const int* __restrict__ num_rows_dev, int64_t rows_alloc, int cols) {
  const int64_t rows = min(static_cast<int64_t>(num_rows_dev[0]), rows_alloc);
  quant_rows16<T>(x, q, scale_t, rows, rows_alloc, cols);
}
}  // namespace flyb200

extern "C" int flyb200_quant_1x128_devrows(const void* x, void* q, float* scale_t,
                                           const int32_t* num_rows_dev, int64_t rows_alloc,
                                           int32_t cols, int32_t in_dtype, void* stream) {
  if (!x || !q || !scale_t || !num_rows_dev)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant_devrows: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(x) % 16) || (reinterpret_cast<uintptr_t>(q) % 8))
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant_devrows: x must be 16-byte, q 8-byte aligned");
  if (rows_alloc < 1 || cols < 128 || cols % 128)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant_devrows: bad sizes");
  if (in_dtype != FLYB200_BF16 && in_dtype != FLYB200_F16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "quant_devrows: input must be BF16 or F16");
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* qo = static_cast<uint8_t*>(q);
  if (in_dtype == FLYB200_BF16)
    quant_1x128_devrows_kernel<__nv_bfloat16><<<sms * 16, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), qo, scale_t, num_rows_dev, rows_alloc, cols);
  else
    quant_1x128_devrows_kernel<__half><<<sms * 16, 256, 0, st>>>(static_cast<const __half*>(x), qo,
                                                                 scale_t, num_rows_dev, rows_alloc, cols);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}
