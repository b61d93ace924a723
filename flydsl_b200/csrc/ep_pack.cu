// Expert-parallel dispatch preparation: which ranks each local token must visit, where its row goes
// in the fixed-size send blocks, and the packed send buffer -- two launches instead of a few dozen
// framework ops (at 8 ranks the local expert work is only a few hundred microseconds, so the
// preparation has to be of the order of ten). The reference has no counterpart (it is single-GPU).
//
// Send layout: W blocks of T row slots; row = [H fp8 | H/128 f32 scales | k i32 expert ids | k f32
// route weights]. Unused slots carry expert id -1 in every position, which the receiver's sorter drops.
#include "common.cuh"

namespace flyb200 {

constexpr int kPlanThreads = 1024;

// One CTA per destination rank r: need[t][r], slot[t][r] (exclusive running count of needed tokens)
// and src[r*T + slot] = t; the tail of the block is filled with -1.
__global__ void __launch_bounds__(kPlanThreads)
ep_plan_kernel(const int* __restrict__ topk_ids, int T, int k, int W, int experts_per_rank,
               uint8_t* __restrict__ need, int* __restrict__ slot, int* __restrict__ src) {
  __shared__ int warp_tot[kPlanThreads / 32];
  __shared__ int base_s;
  const int r = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base_s = 0;
  __syncthreads();
  for (int t0 = 0; t0 < T; t0 += kPlanThreads) {
    const int t = t0 + threadIdx.x;
    bool nd = false;
    if (t < T) {
      for (int j = 0; j < k; ++j) {
        const int id = topk_ids[t * k + j];
        nd |= (id >= 0) && (id / experts_per_rank == r);
      }
    }
    const unsigned bal = __ballot_sync(0xffffffffu, nd);
    if (lane == 0) warp_tot[warp] = __popc(bal);
    __syncthreads();
    int before = base_s;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    const int s = before + __popc(bal & ((1u << lane) - 1u));
    if (t < T) {
      need[t * W + r] = nd ? 1 : 0;
      slot[t * W + r] = nd ? s : 0;
      if (nd) src[r * T + s] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < kPlanThreads / 32; ++w) tot += warp_tot[w];
      base_s += tot;
    }
    __syncthreads();
  }
  for (int s = base_s + threadIdx.x; s < T; s += kPlanThreads) src[r * T + s] = -1;
}

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
  if (T < 1 || H < 128 || H % 128 || k < 1 || W < 1 || experts_per_rank < 1 || (8 * k) % 16)
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
