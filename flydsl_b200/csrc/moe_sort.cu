// MoE routing sort: one launch, one CTA per expert, no inter-CTA communication and no
// order-dependent atomics, so the result is deterministic and bit-identical to the reference's
// per-expert Python loop (moe_sorting_torch_native, tests/kernels/test_moe_gemm.py:97-161):
//   for each unmasked expert in ascending order, its (token, slot) routes in row-major order as
//   (slot << 24) | token, padded to a multiple of block_m with (k << 24) | T.
//
// Every CTA rebuilds the full per-expert histogram (the id array is at most a few hundred KB and
// comes from L2), scans the padded counts to find its own base offset, then compacts its expert's
// routes in order. Both passes over the ids work in rounds of 32 768 ids: a warp takes 1 024
// consecutive ids as eight fully coalesced 16-byte loads per lane, all in flight at once (the passes
// are latency-bound otherwise); a lane holds ids (j*32 + lane)*4 .. +3 of the warp's span for
// j = 0..7. Positions follow the global id order (warp, j, lane, element): per-j warp prefix sums
// (packed four to a register), one block-level prefix over the warps, then each lane writes its
// matches.
//
// Fused permute (flyb200_moe_sort_permute): the CTA that has just placed an expert's routes also
// copies the activation rows of those routes into routing order -- fp8 rows and their 1x128 scales,
// the layout the TMA-fed stage kernels read -- so sort and permute are one launch and one pass of
// latency instead of two. The reference gathers inside its stage kernels
// (kernels/moe_blockscale_2stage.py:394-439); here the gather happens once for both stages.
#include "common.cuh"

namespace flyb200 {

constexpr int kSortThreads = 1024;
constexpr int kChunk = 32;                       // ids per thread per round (eight 16-byte loads)
constexpr int kWarpSpan = 32 * kChunk;           // consecutive ids a warp covers per round

// Element q of group j of this lane = ids[warp_base + (j*32 + lane)*4 + q]; -1 (matches no expert)
// beyond n.
__device__ __forceinline__ void load_chunk(const int* __restrict__ ids, int warp_base, int lane, int n,
                                           bool vec_ok, int (&v)[kChunk]) {
  if (vec_ok && warp_base + kWarpSpan <= n) {
    const int4* p4 = reinterpret_cast<const int4*>(ids + warp_base);
#pragma unroll
    for (int j = 0; j < kChunk / 4; ++j) {
      const int4 q = __ldg(p4 + j * 32 + lane);
      v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < kChunk / 4; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int i = warp_base + (j * 32 + lane) * 4 + q;
        v[4 * j + q] = (i < n) ? __ldg(ids + i) : -1;
      }
  }
}

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
  // optional fused permute (x == nullptr: sort only)
  const uint4* x;       // activations [rows_in, K] fp8, 16-byte chunks
  const float* xs_t;    // their scales [K/128, rows_in]
  uint4* x_out;         // [max_len, K]
  float* xs_out;        // [K/128, max_len]
  int K;
  int rows_in;
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
  // Fused permute with few experts: gridDim.y CTAs per expert. Each repeats the (cheap, L2-fed)
  // placement of the expert's routes -- all of them write the same sorted ids -- and copies every
  // gridDim.y-th row, so that the copy is spread over the whole GPU instead of E SMs.
  const int part = blockIdx.y, parts = gridDim.y;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int n = p.T_eff * p.k;
  const int sentinel = (p.k << 24) | p.T;

  // A masked expert owns no rows and nobody depends on its CTA (CTA 0 also writes the buffer tails).
  if ((e != 0 || part != 0) && p.expert_mask && p.expert_mask[e] == 0) return;
  for (int i = tid; i < p.E; i += kSortThreads) hist[i] = 0;
  __syncthreads();
  const bool vec_ok = (reinterpret_cast<uintptr_t>(p.topk_ids) & 15) == 0;
  for (int r0 = 0; r0 < n; r0 += kSortThreads * kChunk) {
    int v[kChunk];
    load_chunk(p.topk_ids, r0 + warp * kWarpSpan, lane, n, vec_ok, v);
#pragma unroll
    for (int j = 0; j < kChunk; ++j)
      if (v[j] >= 0 && v[j] < p.E) atomicAdd(&hist[v[j]], 1);
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
  if (e == 0 && part == 0) {
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

  // Ordered compaction.
  int running = my_base;
  for (int r0 = 0; r0 < n; r0 += kSortThreads * kChunk) {
    int v[kChunk];
    const int warp_base = r0 + warp * kWarpSpan;
    load_chunk(p.topk_ids, warp_base, lane, n, vec_ok, v);
    // matches per group j (0..4), four groups to a register, 8 bits each (a warp-wide inclusive sum
    // is at most 128)
    unsigned cnt[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < kChunk / 4; ++j) {
      int c = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) c += (v[4 * j + q] == e) ? 1 : 0;
      cnt[j >> 2] |= static_cast<unsigned>(c) << (8 * (j & 3));
    }
    unsigned incl[2] = {cnt[0], cnt[1]};
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned u0 = __shfl_up_sync(0xffffffffu, incl[0], o);
      const unsigned u1 = __shfl_up_sync(0xffffffffu, incl[1], o);
      if (lane >= o) { incl[0] += u0; incl[1] += u1; }
    }
    const unsigned tot0 = __shfl_sync(0xffffffffu, incl[0], 31);   // per-group totals of the warp
    const unsigned tot1 = __shfl_sync(0xffffffffu, incl[1], 31);
    int warp_total = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) warp_total += ((tot0 >> (8 * j)) & 0xFF) + ((tot1 >> (8 * j)) & 0xFF);
    if (lane == 0) warp_cnt[warp] = warp_total;
    __syncthreads();
    int before = 0, all = 0;
    for (int w = 0; w < kSortThreads / 32; ++w) {
      const int c = warp_cnt[w];
      before += (w < warp) ? c : 0;
      all += c;
    }
    if (warp_total) {
      int group_base = running + before;     // first position of group j of this warp
#pragma unroll
      for (int j = 0; j < kChunk / 4; ++j) {
        const unsigned tj = ((j < 4 ? tot0 : tot1) >> (8 * (j & 3))) & 0xFF;
        const unsigned ij = ((j < 4 ? incl[0] : incl[1]) >> (8 * (j & 3))) & 0xFF;
        const unsigned cj = ((j < 4 ? cnt[0] : cnt[1]) >> (8 * (j & 3))) & 0xFF;
        if (cj) {
          int pos = group_base + static_cast<int>(ij - cj);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (v[4 * j + q] == e) {
              const int i = warp_base + (j * 32 + lane) * 4 + q;
              const int t = i / p.k;
              const int slot = i - t * p.k;
              p.sorted_ids[pos] = (slot << 24) | t;
              p.sorted_weights[pos] = p.topk_weights[i];
              ++pos;
            }
          }
        }
        group_base += static_cast<int>(tj);
      }
    }
    running += all;
    __syncthreads();
  }
  for (int i = my_cnt + tid; i < my_padded; i += kSortThreads) {
    p.sorted_ids[my_base + i] = sentinel;
    p.sorted_weights[my_base + i] = 0.f;
  }
  for (int b = tid; b < my_padded / p.block_m; b += kSortThreads)
    p.sorted_expert_ids[my_base / p.block_m + b] = cid;

  if (p.x == nullptr) return;
  // ---- fused permute: rows my_base .. my_base + my_padded of the routing-order buffers ----
  __syncthreads();   // this CTA's sorted ids are visible to all of its threads
  const int chunks = p.K / 16;
  const int nscale = p.K / 128;
  for (int i = warp + part * (kSortThreads / 32); i < my_padded; i += parts * (kSortThreads / 32)) {
    const int r = my_base + i;
    const int t = p.sorted_ids[r] & 0xFFFFFF;
    const bool ok = i < my_cnt && t < p.rows_in;
    const uint4* srow = p.x + static_cast<long long>(ok ? t : 0) * chunks;
    uint4* drow = p.x_out + static_cast<long long>(r) * chunks;
    for (int c0 = lane; c0 < chunks; c0 += 128) {   // four 16-byte loads per lane in flight
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
  // scales: sorted position fastest, so that the stores to the transposed output are coalesced
  for (int j = tid + part * kSortThreads; j < nscale * my_padded; j += parts * kSortThreads) {
    const int sidx = j / my_padded;
    const int i = j - sidx * my_padded;
    const int t = p.sorted_ids[my_base + i] & 0xFFFFFF;
    const bool ok = i < my_cnt && t < p.rows_in;
    p.xs_out[static_cast<long long>(sidx) * p.max_len + my_base + i] =
        ok ? __ldg(p.xs_t + static_cast<long long>(sidx) * p.rows_in + t) : 0.f;
  }
}

// Router: top-k of a token's expert scores in descending order (= slot order) and a softmax over the
// k selected values, as the reference's test router does with torch.topk + torch.softmax
// (tests/kernels/test_moe_blockscale.py:228-230). One warp per token; a lane keeps every 32nd score
// in registers; k rounds of warp arg-max (ties go to the lower expert id).
constexpr int kRouteMaxPerLane = 32;  // experts <= 1024

__global__ void __launch_bounds__(256)
moe_route_topk_kernel(const float* __restrict__ logits, int T, int E, int k, int* __restrict__ ids_out,
                      float* __restrict__ w_out) {
  const int lane = threadIdx.x & 31;
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  float v[kRouteMaxPerLane];
#pragma unroll
  for (int j = 0; j < kRouteMaxPerLane; ++j) {
    const int e = j * 32 + lane;
    v[j] = (e < E) ? logits[static_cast<size_t>(t) * E + e] : -INFINITY;
    if (v[j] != v[j]) v[j] = -INFINITY;   // NaN scores are never selected
  }
  float top = 0.f, sum = 0.f, mine = 0.f;
  int mine_id = 0;
  for (int s = 0; s < k; ++s) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
      const int e = j * 32 + lane;
      if (e < E && (v[j] > best || (v[j] == best && e < best_e))) { best = v[j]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (s == 0) top = best;
    const float p = expf(best - top);
    sum += p;
    if (lane == s % 32) { mine = p; mine_id = best_e; }
    if (s % 32 == 31 || s == k - 1) {   // flush up to 32 selections (k <= 32 in practice: one flush)
      const int s0 = s - (s % 32);
      if (s0 + lane <= s) {
        ids_out[static_cast<size_t>(t) * k + s0 + lane] = mine_id;
        w_out[static_cast<size_t>(t) * k + s0 + lane] = mine;   // normalised below
      }
    }
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j)
      if (j * 32 + lane == best_e) v[j] = -INFINITY;
  }
  __syncwarp();
  for (int s = lane; s < k; s += 32)
    w_out[static_cast<size_t>(t) * k + s] = __fdiv_rn(w_out[static_cast<size_t>(t) * k + s], sum);
}

}  // namespace flyb200

using namespace flyb200;

extern "C" int flyb200_moe_route_topk(const float* logits, int32_t T, int32_t E, int32_t k,
                                      int32_t* topk_ids, float* topk_weights, void* stream) {
  if (!logits || !topk_ids || !topk_weights)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "route_topk: NULL buffer");
  if (T < 1 || E < 1 || E > 32 * kRouteMaxPerLane || k < 1 || k > E)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "route_topk: bad sizes T=%d E=%d k=%d (E <= %d, k <= E)", T,
                     E, k, 32 * kRouteMaxPerLane);
  const int blocks = (T + 7) / 8;
  moe_route_topk_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(logits, T, E, k, topk_ids,
                                                                                 topk_weights);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

static int moe_sort_impl(const int32_t* topk_ids, const float* topk_weights, int32_t T, int32_t k, int32_t E,
                         int32_t block_m, const int32_t* expert_mask, int32_t num_local_tokens,
                         int32_t* sorted_ids, float* sorted_weights, int32_t* sorted_expert_ids,
                         int32_t* num_valid_ids, const void* x, const float* xs_t, void* x_out,
                         float* xs_out, int32_t K, void* stream) {
  if (!topk_ids || !topk_weights || !sorted_ids || !sorted_weights || !sorted_expert_ids ||
      !num_valid_ids)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_sort: NULL buffer");
  // k <= E: the buffers are sized T*k + E*block_m - k (the reference's formula), which bounds the
  // padded total T*k + E*(block_m - 1) only then.
  if (T < 0 || T >= (1 << 24) || k < 1 || k > 255 || E < 1 || E > 8192 || block_m < 1 || k > E)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "moe_sort: bad sizes T=%d k=%d E=%d block_m=%d (T < 2^24, k <= 255, k <= E <= 8192)",
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
  p.x = static_cast<const uint4*>(x); p.xs_t = xs_t;
  p.x_out = static_cast<uint4*>(x_out); p.xs_out = xs_out;
  p.K = K; p.rows_in = T;
  int parts = 1;
  if (x) {
    const int sms = sm_count();
    if (sms <= 0) return FLYB200_ERR_CUDA;
    parts = (2 * sms) / E;
    parts = parts < 1 ? 1 : (parts > 8 ? 8 : parts);
  }
  moe_sort_kernel<<<dim3(E, parts), kSortThreads, 2 * E * sizeof(int),
                    reinterpret_cast<cudaStream_t>(stream)>>>(p);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

extern "C" int flyb200_moe_sort(const int32_t* topk_ids, const float* topk_weights, int32_t T,
                                int32_t k, int32_t E, int32_t block_m, const int32_t* expert_mask,
                                int32_t num_local_tokens, int32_t* sorted_ids,
                                float* sorted_weights, int32_t* sorted_expert_ids,
                                int32_t* num_valid_ids, void* stream) {
  return moe_sort_impl(topk_ids, topk_weights, T, k, E, block_m, expert_mask, num_local_tokens, sorted_ids,
                       sorted_weights, sorted_expert_ids, num_valid_ids, nullptr, nullptr, nullptr, nullptr, 0,
                       stream);
}

extern "C" int flyb200_moe_sort_permute(const int32_t* topk_ids, const float* topk_weights, int32_t T,
                                        int32_t k, int32_t E, int32_t block_m, const int32_t* expert_mask,
                                        int32_t num_local_tokens, int32_t* sorted_ids,
                                        float* sorted_weights, int32_t* sorted_expert_ids,
                                        int32_t* num_valid_ids, const void* x, const float* x_scale_t,
                                        void* x_sorted, float* x_scale_sorted_t, int32_t K, void* stream) {
  if (!x || !x_scale_t || !x_sorted || !x_scale_sorted_t)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_sort_permute: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(x_sorted)) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_sort_permute: x and x_sorted must be 16-byte aligned");
  if (K < 128 || K % 128)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_sort_permute: K (%d) must be a multiple of 128", K);
  return moe_sort_impl(topk_ids, topk_weights, T, k, E, block_m, expert_mask, num_local_tokens, sorted_ids,
                       sorted_weights, sorted_expert_ids, num_valid_ids, x, x_scale_t, x_sorted,
                       x_scale_sorted_t, K, stream);
}
