// MoE routing sort: one launch, one CTA per expert, no inter-CTA communication and no
// order-dependent atomics, so the result is deterministic and bit-identical to the reference's
// per-expert Python loop (moe_sorting_torch_native, tests/kernels/test_moe_gemm.py:97-161):
//   for each unmasked expert in ascending order, its (token, slot) routes in row-major order as
//   (slot << 24) | token, padded to a multiple of block_m with (k << 24) | T.
//
// Every CTA rebuilds the full per-expert histogram (the id array is at most a few hundred KB and
// comes from L2), scans the padded counts to find its own base offset, then compacts its expert's
// routes in order: each warp owns a contiguous segment, counts its matches, and after one
// block-level prefix writes them at base + earlier-warps + running rank.
#include "common.cuh"

namespace flyb200 {

constexpr int kSortThreads = 1024;

struct SortParams {
  const int* topk_ids;
  const float* topk_weights;
  const int* expert_mask;
  int* sorted_ids;
  float* sorted_weights;
  int* sorted_expert_ids;
  int* num_valid_ids;
  int T;        // tokens in the id tensor (sentinel token id)
  int T_eff;    // tokens that take part (num_local_tokens)
  int k;
  int E;
  int block_m;
  int max_len;     // T*k + E*block_m - k
  int max_blocks;  // ceil(max_len / block_m)
};

__global__ void __launch_bounds__(kSortThreads)
moe_sort_kernel(const SortParams p) {
  extern __shared__ int sm[];
  int* hist = sm;               // [E]   route count per expert
  int* base = sm + p.E;         // [E]   first sorted row of each expert (exclusive scan of padded)
  __shared__ int warp_cnt[kSortThreads / 32];
  __shared__ int scan_tmp[kSortThreads / 32];
  __shared__ int total_rows;
  __shared__ int my_compact_id;

  const int e = blockIdx.x;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n = p.T_eff * p.k;
  const int sentinel = (p.k << 24) | p.T;

  for (int i = tid; i < p.E; i += kSortThreads) hist[i] = 0;
  __syncthreads();
  for (int i = tid; i < n; i += kSortThreads) {
    const int id = p.topk_ids[i];
    if (id >= 0 && id < p.E) atomicAdd(&hist[id], 1);
  }
  __syncthreads();

  // Exclusive scan of padded counts over experts (E is small: loop in chunks of the block size).
  int carry = 0, carry_masked = 0;
  for (int e0 = 0; e0 < p.E; e0 += kSortThreads) {
    const int idx = e0 + tid;
    int padded = 0, masked = 0;
    if (idx < p.E) {
      const bool on = !p.expert_mask || p.expert_mask[idx] != 0;
      masked = on ? 0 : 1;
      padded = on ? ((hist[idx] + p.block_m - 1) / p.block_m) * p.block_m : 0;
    }
    // warp inclusive scans of (padded, masked)
    int v = padded, m = masked;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int tv = __shfl_up_sync(0xffffffffu, v, o);
      const int tm = __shfl_up_sync(0xffffffffu, m, o);
      if (lane >= o) { v += tv; m += tm; }
    }
    if (lane == 31) { warp_cnt[warp] = v; scan_tmp[warp] = m; }
    __syncthreads();
    int wv = 0, wm = 0;
    for (int w = 0; w < warp; ++w) { wv += warp_cnt[w]; wm += scan_tmp[w]; }
    if (idx < p.E) {
      base[idx] = carry + wv + v - padded;
      if (idx == e) my_compact_id = masked ? -1 : idx - (carry_masked + wm + m - masked);
    }
    int tot_v = 0, tot_m = 0;
    for (int w = 0; w < kSortThreads / 32; ++w) { tot_v += warp_cnt[w]; tot_m += scan_tmp[w]; }
    carry += tot_v;
    carry_masked += tot_m;
    __syncthreads();
  }
  if (tid == 0) total_rows = carry;
  __syncthreads();
  const int total = total_rows;

  // Tail of the buffers beyond the used rows/blocks, and the counters: CTA 0.
  if (e == 0) {
    for (int i = total + tid; i < p.max_len; i += kSortThreads) {
      p.sorted_ids[i] = sentinel;
      p.sorted_weights[i] = 0.f;
    }
    for (int b = total / p.block_m + tid; b < p.max_blocks; b += kSortThreads)
      p.sorted_expert_ids[b] = -1;
    if (tid == 0) {
      p.num_valid_ids[0] = total;
      p.num_valid_ids[1] = p.T_eff;
    }
  }

  const int cid = my_compact_id;
  if (cid < 0) return;  // masked expert: owns no rows
  const int my_base = base[e];
  const int my_cnt = hist[e];
  const int my_padded = ((my_cnt + p.block_m - 1) / p.block_m) * p.block_m;

  // Ordered compaction. Warp w owns routes [w*seg, (w+1)*seg).
  const int seg = (((n + kSortThreads / 32 - 1) / (kSortThreads / 32)) + 31) & ~31;
  const int lo = warp * seg;
  const int hi = min(n, lo + seg);
  int cnt = 0;
  for (int i0 = lo; i0 < hi; i0 += 32) {
    const int i = i0 + lane;
    const bool hit = (i < hi) && (p.topk_ids[i] == e);
    cnt += __popc(__ballot_sync(0xffffffffu, hit));
  }
  if (lane == 0) warp_cnt[warp] = cnt;
  __syncthreads();
  int rank = my_base;
  for (int w = 0; w < warp; ++w) rank += warp_cnt[w];
  for (int i0 = lo; i0 < hi; i0 += 32) {
    const int i = i0 + lane;
    const bool hit = (i < hi) && (p.topk_ids[i] == e);
    const unsigned bal = __ballot_sync(0xffffffffu, hit);
    if (hit) {
      const int pos = rank + __popc(bal & ((1u << lane) - 1u));
      const int t = i / p.k;
      const int slot = i - t * p.k;
      p.sorted_ids[pos] = (slot << 24) | t;
      p.sorted_weights[pos] = p.topk_weights[i];
    }
    rank += __popc(bal);
  }
  for (int i = my_cnt + tid; i < my_padded; i += kSortThreads) {
    p.sorted_ids[my_base + i] = sentinel;
    p.sorted_weights[my_base + i] = 0.f;
  }
  for (int b = tid; b < my_padded / p.block_m; b += kSortThreads)
    p.sorted_expert_ids[my_base / p.block_m + b] = cid;
}

}  // namespace flyb200

using namespace flyb200;

extern "C" int flyb200_moe_sort(const int32_t* topk_ids, const float* topk_weights, int32_t T,
                                int32_t k, int32_t E, int32_t block_m, const int32_t* expert_mask,
                                int32_t num_local_tokens, int32_t* sorted_ids,
                                float* sorted_weights, int32_t* sorted_expert_ids,
                                int32_t* num_valid_ids, void* stream) {
  if (!topk_ids || !topk_weights || !sorted_ids || !sorted_weights || !sorted_expert_ids ||
      !num_valid_ids)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_sort: NULL buffer");
  if (T < 0 || T >= (1 << 24) || k < 1 || k > 255 || E < 1 || E > 8192 || block_m < 1)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "moe_sort: bad sizes T=%d k=%d E=%d block_m=%d (T < 2^24, k <= 255, E <= 8192)",
                     T, k, E, block_m);
  const long long max_len = static_cast<long long>(T) * k + static_cast<long long>(E) * block_m - k;
  if (max_len <= 0 || max_len > 0x7fffffffLL)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_sort: sorted length out of range");
  SortParams p;
  p.topk_ids = topk_ids; p.topk_weights = topk_weights; p.expert_mask = expert_mask;
  p.sorted_ids = sorted_ids; p.sorted_weights = sorted_weights;
  p.sorted_expert_ids = sorted_expert_ids; p.num_valid_ids = num_valid_ids;
  p.T = T;
  p.T_eff = (num_local_tokens < 0 || num_local_tokens > T) ? T : num_local_tokens;
  p.k = k; p.E = E; p.block_m = block_m;
  p.max_len = static_cast<int>(max_len);
  p.max_blocks = static_cast<int>((max_len + block_m - 1) / block_m);
  moe_sort_kernel<<<E, kSortThreads, 2 * E * sizeof(int),
                    reinterpret_cast<cudaStream_t>(stream)>>>(p);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}
