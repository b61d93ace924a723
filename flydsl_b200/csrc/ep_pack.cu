// Expert-parallel dispatch preparation: which ranks each local token must visit, where its row goes
// in the fixed-size send blocks, and the packed send buffer -- two launches instead of a few dozen
// framework ops (at 8 ranks the local expert work is only a few hundred microseconds, so the
// preparation has to be of the order of ten). The reference has no counterpart (it is single-GPU).
//
// Send layout: W blocks of T row slots; row = [H fp8 | H/128 f32 scales | k i32 expert ids | k f32
// route weights]. Unused slots carry expert id -1 in every position, which the receiver's sorter drops.
#include "common.cuh"
#include "ep_plan.cuh"

namespace flyb200 {

// One warp per send row.
__global__ void __launch_bounds__(256)
ep_pack_kernel(const uint8_t* __restrict__ x, const float* __restrict__ x_scale,
               const int* __restrict__ topk_ids, const float* __restrict__ topk_w,
               const int* __restrict__ src, uint8_t* __restrict__ send, int rows, int H, int k) {
  const int nscale = H / 128;
  const int row_bytes = H + 4 * nscale + 8 * k;
  const int lane = threadIdx.x & 31;
  const int warp0 = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int i = warp0; i < rows; i += nwarps) {
    const int t = src[i];
    uint8_t* dst = send + static_cast<size_t>(i) * row_bytes;
    int* dst_ids = reinterpret_cast<int*>(dst + H + 4 * nscale);
    if (t < 0) {
      for (int j = lane; j < k; j += 32) dst_ids[j] = -1;
      continue;
    }
    const uint4* s4 = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int c = lane; c < H / 16; c += 32) d4[c] = s4[c];
    float* dsc = reinterpret_cast<float*>(dst + H);
    for (int c = lane; c < nscale; c += 32) dsc[c] = x_scale[static_cast<size_t>(t) * nscale + c];
    float* dw = reinterpret_cast<float*>(dst + H + 4 * nscale + 4 * k);
    for (int j = lane; j < k; j += 32) {
      dst_ids[j] = topk_ids[t * k + j];
      dw[j] = topk_w[t * k + j];
    }
  }
}

}  // namespace flyb200

using namespace flyb200;

extern "C" int flyb200_ep_plan_pack(const void* x, const float* x_scale, const int32_t* topk_ids,
                                    const float* topk_weights, int32_t T, int32_t H, int32_t k,
                                    int32_t W, int32_t experts_per_rank, uint8_t* need_out,
                                    int32_t* slot_out, int32_t* src_out, void* send_out, void* stream) {
  if (!x || !x_scale || !topk_ids || !topk_weights || !need_out || !slot_out || !src_out || !send_out)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_plan_pack: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(send_out)) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_plan_pack: x and send_out must be 16-byte aligned");
  if (T < 1 || H < 128 || H % 128 || k < 1 || W < 1 || experts_per_rank < 1 || (8 * k) % 16 ||
      (H + 4 * (H / 128) + 8 * k) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "ep_plan_pack: bad sizes (H %% 128 == 0, k even so that rows stay 16-byte aligned)");
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  ep_plan_kernel<<<W, kPlanThreads, 0, st>>>(topk_ids, T, k, W, experts_per_rank, need_out, slot_out, src_out);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  const int rows = W * T;
  int blocks = (rows + 7) / 8;
  if (blocks > sms * 8) blocks = sms * 8;
  ep_pack_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint8_t*>(x), x_scale, topk_ids, topk_weights,
                                         src_out, static_cast<uint8_t*>(send_out), rows, H, k);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

// ---------------------------------------------------------------------------------------------
// Receiving side: activations straight from the packed receive buffer into routing order (what
// flyb200_moe_gather_rows does for plain tensors), so the packed rows are never copied apart.
namespace flyb200 {
__global__ void __launch_bounds__(256)
ep_gather_packed_kernel(const uint8_t* __restrict__ packed, const int* __restrict__ sorted_ids,
                        const int* __restrict__ num_valid, uint4* __restrict__ x_out,
                        float* __restrict__ scale_out_t, int rows_in, int H, int row_bytes,
                        int rows_out) {
  const int chunks = H / 16, nscale = H / 128;
  const int valid = min(num_valid[0], rows_out);
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = warp; i < valid; i += nwarps) {
    const int t = sorted_ids[i] & 0xFFFFFF;
    const bool ok = t < rows_in;
    const uint8_t* row = packed + static_cast<size_t>(ok ? t : 0) * row_bytes;
    const uint4* s4 = reinterpret_cast<const uint4*>(row);
    for (int c = lane; c < chunks; c += 32)
      x_out[static_cast<size_t>(i) * chunks + c] = ok ? s4[c] : make_uint4(0u, 0u, 0u, 0u);
    const float* sc = reinterpret_cast<const float*>(row + H);
    for (int s = lane; s < nscale; s += 32)
      scale_out_t[static_cast<size_t>(s) * rows_out + i] = ok ? sc[s] : 0.f;
  }
}

// Expert ids, route weights and the "expert lives on this rank" mask of every packed row, as the
// dense tensors the sorter and the masked reduce take: one launch instead of five framework ops.
__global__ void __launch_bounds__(256)
ep_unpack_meta_kernel(const uint8_t* __restrict__ packed, int rows, int H, int k, int row_bytes,
                      int experts_per_rank, int rank, int local_ids, int* __restrict__ ids_out,
                      float* __restrict__ w_out, uint8_t* __restrict__ valid_out) {
  const int total = rows * k;
  const int meta = H + 4 * (H / 128);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int r = i / k, j = i - r * k;
    const uint8_t* row = packed + static_cast<size_t>(r) * row_bytes + meta;
    const int id = reinterpret_cast<const int*>(row)[j];
    const bool mine = id >= 0 && id / experts_per_rank == rank;
    // local_ids: ids relative to this rank's first expert, -1 for every foreign or unused route, so
    // that the routing sort runs over experts_per_rank experts only
    ids_out[i] = local_ids ? (mine ? id - rank * experts_per_rank : -1) : id;
    w_out[i] = reinterpret_cast<const float*>(row + 4 * k)[j];
    valid_out[i] = mine ? 1 : 0;
  }
}

// Sending side, after the combine all-to-all: out[t] = sum over ranks r (ascending) of the partial row
// back[r*T + slot[t][r]] where need[t][r]; fp32 accumulate, one 16-byte vector per thread.
template <typename T>
__global__ void __launch_bounds__(256)
ep_combine_kernel(const T* __restrict__ back, const uint8_t* __restrict__ need,
                  const int* __restrict__ slot, T* __restrict__ out, int tokens, int W, int H) {
  constexpr int VEC = 16 / sizeof(T);
  const int vec_per_row = H / VEC;
  const long long total = static_cast<long long>(tokens) * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_row);
    const int v = static_cast<int>(i - static_cast<long long>(t) * vec_per_row);
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    for (int r = 0; r < W; ++r) {
      if (!need[t * W + r]) continue;
      const long long row = static_cast<long long>(r) * tokens + slot[t * W + r];
      const uint4 raw = *reinterpret_cast<const uint4*>(back + row * H + static_cast<long long>(v) * VEC);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] += static_cast<float>(e[j]);
    }
    uint4 o;
    T* po = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < VEC; ++j) po[j] = static_cast<T>(acc[j]);
    *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H + static_cast<long long>(v) * VEC) = o;
  }
}
}  // namespace flyb200

extern "C" int flyb200_ep_gather_packed(const void* packed, const int32_t* sorted_ids,
                                        const int32_t* num_valid_ids, void* x_out, float* scale_out_t,
                                        int32_t rows_in, int32_t H, int32_t k, int32_t rows_out,
                                        void* stream) {
  if (!packed || !sorted_ids || !num_valid_ids || !x_out || !scale_out_t)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_gather_packed: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(x_out)) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_gather_packed: buffers must be 16-byte aligned");
  if (rows_in < 1 || rows_out < 1 || H < 128 || H % 128 || k < 1 || (8 * k) % 16 ||
      (H + 4 * (H / 128) + 8 * k) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_gather_packed: bad sizes");
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const int row_bytes = H + 4 * (H / 128) + 8 * k;
  ep_gather_packed_kernel<<<sms * 4, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(packed), sorted_ids, num_valid_ids, static_cast<uint4*>(x_out),
      scale_out_t, rows_in, H, row_bytes, rows_out);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

extern "C" int flyb200_ep_unpack_meta(const void* packed, int32_t rows, int32_t H, int32_t k,
                                      int32_t experts_per_rank, int32_t rank, int32_t local_ids,
                                      int32_t* ids_out, float* weights_out, uint8_t* valid_out,
                                      void* stream) {
  if (!packed || !ids_out || !weights_out || !valid_out)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_unpack_meta: NULL buffer");
  if (rows < 1 || H < 128 || H % 128 || k < 1 || experts_per_rank < 1 || rank < 0 ||
      reinterpret_cast<uintptr_t>(packed) % 4)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_unpack_meta: bad sizes");
  const int row_bytes = H + 4 * (H / 128) + 8 * k;
  const long long total = static_cast<long long>(rows) * k;
  if (total > 0x7fffffffLL) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_unpack_meta: too many routes");
  const int blocks = static_cast<int>((total + 255) / 256);
  ep_unpack_meta_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(packed), rows, H, k, row_bytes, experts_per_rank, rank, local_ids, ids_out,
      weights_out, valid_out);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

extern "C" int flyb200_ep_combine(const void* back, const uint8_t* need, const int32_t* slot, void* out,
                                  int32_t T, int32_t W, int32_t H, int32_t dtype, void* stream) {
  if (!back || !need || !slot || !out)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_combine: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(back) | reinterpret_cast<uintptr_t>(out)) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_combine: buffers must be 16-byte aligned");
  if (T < 1 || W < 1 || H < 8 || H % 8 || (dtype != FLYB200_BF16 && dtype != FLYB200_F16))
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_combine: bad sizes or dtype");
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const long long total = static_cast<long long>(T) * (H / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > static_cast<long long>(sms) * 16) blocks = static_cast<long long>(sms) * 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == FLYB200_BF16)
    ep_combine_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(back), need, slot, static_cast<__nv_bfloat16*>(out), T, W, H);
  else
    ep_combine_kernel<__half><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const __half*>(back), need, slot, static_cast<__half*>(out), T, W, H);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}
