// Bandwidth-bound helpers around the MoE GEMMs:
//   * top-k reduce  Y[t,d] = sum_s X[t,s,d]           (compile_moe_reduction,
//                                                       kernels/moe_blockscale_2stage.py:2446-2638)
//   * 1x128 group quantiser to fp8 e4m3 with transposed scales (the re-quantisation between the
//     stages, tests/kernels/test_moe_blockscale.py:346-361 + pertoken_quant tests/utils.py:29-73)
#include <cuda_fp8.h>

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
// load instruction; the amax reduction stays inside the half-warp. `raw` holds the lane's 8 values.
template <typename T>
__device__ __forceinline__ void quant_group16(const uint4& raw, uint8_t* __restrict__ q,
                                              float* __restrict__ scale_t, int64_t row, int g,
                                              int cols, int64_t scale_stride, bool active, int sub) {
  float v[8];
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = active ? to_f32<T>(e[j]) : 0.f;
  float vmax = -3.4e38f, vmin = 3.4e38f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (v[j] != v[j]) v[j] = 0.f;
    else if (isinf(v[j])) v[j] = v[j] > 0 ? 448.f : -448.f;
    vmax = fmaxf(vmax, v[j]);
    vmin = fminf(vmin, v[j]);
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) {  // xor distances < 16 stay inside the half-warp
    vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
  }
  float scale = __fdiv_rn(fmaxf(vmax, -vmin), 448.f);
  if (scale == 0.f) scale = 1.f;
  if (active) {
    // v / scale, correctly rounded, from one reciprocal: q0 = v*rc, q = fma(fma(-scale, q0, v), rc, q0)
    // is the IEEE quotient when rc is the correctly rounded reciprocal and the mantissa of scale is
    // not all ones (Markstein); that rare scale takes the true division. Eight IEEE divisions per
    // lane made this kernel compute-bound at a quarter of the copy bandwidth.
    const float rc = __frcp_rn(scale);
    const bool exact_div = (__float_as_uint(scale) & 0x7fffffu) == 0x7fffffu;
    float qv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float q0 = v[j] * rc;
      qv[j] = exact_div ? __fdiv_rn(v[j], scale) : __fmaf_rn(__fmaf_rn(-scale, q0, v[j]), rc, q0);
    }
    const uint32_t lo = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[0], qv[1]), __NV_SATFINITE, __NV_E4M3)) |
                        (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[2], qv[3]), __NV_SATFINITE, __NV_E4M3)) << 16);
    const uint32_t hi = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[4], qv[5]), __NV_SATFINITE, __NV_E4M3)) |
                        (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(qv[6], qv[7]), __NV_SATFINITE, __NV_E4M3)) << 16);
    *reinterpret_cast<uint2*>(q + row * cols + g * 128 + sub * 8) = make_uint2(lo, hi);
    if (sub == 0) scale_t[static_cast<int64_t>(g) * scale_stride + row] = scale;
  }
}

// rows x (cols/128) groups, two groups per warp per step (one per half-warp), four steps' loads in
// flight at once: the kernel is a dependent load -> reduce -> divide -> store chain per group and was
// latency-bound at a quarter of the copy bandwidth with one group per thread in flight.
template <typename T>
__device__ __forceinline__ void quant_rows16(const T* __restrict__ x, uint8_t* __restrict__ q,
                                             float* __restrict__ scale_t, int64_t rows,
                                             int64_t scale_stride, int cols) {
  constexpr int kInFlight = 4;
  const int groups = cols / 128;
  const int64_t total = rows * groups;
  const int lane = threadIdx.x & 31;
  const int sub = lane & 15;
  const int64_t hw0 = ((blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5) * 2 + (lane >> 4);
  const int64_t nhw = ((static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5) * 2;
  for (int64_t w = hw0 - (lane >> 4); w < total; w += nhw * kInFlight) {  // warp-uniform trip count
    uint4 raw[kInFlight];
    int64_t row[kInFlight];
    int g[kInFlight];
    bool active[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int64_t idx = w + u * nhw + (lane >> 4);
      active[u] = idx < total;
      // rows fastest: neighbouring half-warps write neighbouring entries of the transposed scales.
      // 32-bit division when the group count allows it (a 64-bit one costs more than the rest of
      // the group's arithmetic).
      if (total <= 0x7fffffffLL) {
        const unsigned gi = active[u] ? static_cast<unsigned>(idx) / static_cast<unsigned>(rows) : 0u;
        g[u] = static_cast<int>(gi);
        row[u] = active[u] ? static_cast<int64_t>(static_cast<unsigned>(idx) - gi * static_cast<unsigned>(rows)) : 0;
      } else {
        g[u] = active[u] ? static_cast<int>(idx / rows) : 0;
        row[u] = active[u] ? idx - static_cast<int64_t>(g[u]) * rows : 0;
      }
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (active[u]) raw[u] = *reinterpret_cast<const uint4*>(x + row[u] * cols + g[u] * 128 + sub * 8);
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u)
      if (w + u * nhw < total)   // warp-uniform: the shuffles inside need the whole warp
        quant_group16<T>(raw[u], q, scale_t, row[u], g[u], cols, scale_stride, active[u], sub);
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
                       int K, int topk, int rows_out, int by_slot) {
  const int chunks = K / 16;               // 16-byte chunks per row
  const int nscale = K / 128;
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
      scale_out_t, rows_in, K, topk, rows_out, by_slot ? 1 : 0);
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
