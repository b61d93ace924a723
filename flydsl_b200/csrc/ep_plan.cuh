// Dispatch plan of the expert-parallel exchange, shared by the packed (NCCL) and the peer-memory path.
#pragma once
#include "common.cuh"

namespace flyb200 {

constexpr int kPlanThreads = 1024;

// One CTA per destination rank r: need[t][r], slot[t][r] (exclusive running count of needed tokens)
// and src[r*T + slot] = t; the tail of the block is filled with -1.
static __global__ void __launch_bounds__(kPlanThreads)
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

}  // namespace flyb200
