// FP8 (e4m3) block-scale GEMM core for sm_100a: one persistent, warp-specialised kernel template
// that serves the dense GEMM and both MoE stages.
//
//   C[m,n] = sum_kb ( sum_{k in kb} A[m,k] * B[n,k] ) * sa[kb,m] * sb[n/128,kb]
//
// Roles inside a 384-thread CTA (one CTA per SM):
//   warp 0      producer: TMA tensor load of the A tile (dense) and bulk copies of the repacked,
//               pre-swizzled weight tile into a multistage shared-memory ring
//   warp 1      MMA issuer: tcgen05.mma kind::f8f6f4, 128 x BN x 32, four per 128-wide K block,
//               each K block into a fresh TMEM accumulator buffer (512/BN buffers in rotation)
//   warps 2-3   one of: (dense) lane 0 of warp 2 turns every staged tile into TMA stores;
//               (MoE, activations in routing order) both warps copy every staged tile to its output
//               rows -- coalesced row stores or vector reductions to the scattered (token, slot) rows;
//               (MoE, reference-shaped inputs) gather activation rows by sorted id with cp.async
//               into the same swizzled image TMA would have produced
//   warps 4-11  epilogue: tcgen05.ld the K-block partial (loads pipelined against the FMAs),
//               acc = fma(partial, sa*sb, acc) in fp32 registers (the per-128-K scale promotion),
//               release the TMEM buffer; after the last K block convert, stage the tile in shared
//               memory and hand it to warps 2-3 (in the gather mode they store it themselves)
//
// The computation follows kernel_gemm / compute_tile_blockscale of the reference
// (kernels/blockscale_preshuffle_gemm.py:161-839, :509-587) and the stage kernels of
// kernels/moe_blockscale_2stage.py (:206-1161, :1386-2387); none of its AMD data movement is kept.
#include <cuda_fp8.h>

#include "common.cuh"

namespace flyb200 {

constexpr int BM = 128;            // MMA M = accumulator lanes
constexpr int BK = 128;            // K bytes per pipeline stage = one scale block
constexpr int kThreads = 384;
constexpr int kEpiWarp0 = 4;       // first epilogue warp
constexpr int kEpiWarps = 8;
constexpr int kATileBytes = BM * BK;
constexpr int kRegionBytes = BM * 128;  // one 64-column (16-bit) slab of the staged output tile

// kDensePT: dense GEMM with one scale per token (row) and one per output channel (column) instead
// of block scales: C[m,n] = (sum_k A[m,k] B[n,k]) * sa[m] * sb[n]. The whole K range accumulates in
// one TMEM buffer (no per-128-K promotion), so the epilogue touches a tile once and the tensor pipe
// runs from one tile into the next. Reference: kernels/preshuffle_gemm.py:206-1266 (in_dtype fp8).
// kMoe1PT / kMoe2PT: the two MoE stages with per-token activation scales ([rows]) and per-channel
// weight scales ([experts * output channels]) -- the routing, gather and output code of kMoe1 / kMoe2
// with the whole-K accumulation of kDensePT. Reference: kernels/moe_gemm_2stage.py:93-1264 (stage 1)
// and :1267-2481 (stage 2), in_dtype fp8.
enum Mode : int { kDense = 0, kMoe1 = 1, kMoe2 = 2, kDensePT = 3, kMoe1PT = 4, kMoe2PT = 5 };
__host__ __device__ constexpr bool is_dense(int mode) { return mode == kDense || mode == kDensePT; }
__host__ __device__ constexpr bool is_moe1(int mode) { return mode == kMoe1 || mode == kMoe1PT; }
__host__ __device__ constexpr bool is_moe2(int mode) { return mode == kMoe2 || mode == kMoe2PT; }
__host__ __device__ constexpr bool is_pt(int mode) { return mode >= kDensePT; }

struct GemmParams {
  const uint8_t* a;        // MoE: activation rows to gather from (dense uses the tensor map)
  const uint8_t* b;        // repacked weights
  const float* scale_a;    // [K/128, rows]
  const float* scale_b;    // [blocks_n, K/128]
  void* out;
  int* err;                // device error word
  int M;                   // dense: rows of A; MoE: tokens T
  int N;                   // dense: N; stage 1: inter_dim I; stage 2: model_dim H
  int K;
  int a_box_rows;          // dense: rows the A tensor-map box brings per stage
  // Dense: 0, or the number of row blocks per group of the tile order (see TileWalker): set by the
  // host when the activations alone are larger than half the L2.
  int group_m;
  // MoE only
  const int* sorted_ids;
  const int* expert_ids;
  const float* sorted_weights;
  const int* num_valid;
  int topk;
  int tile_m;
  int num_blocks;
  int experts;
  int doweight;
  int accumulate;
  // MoE, optional "sorted" layouts (cfg.path bits): activations already permuted into routing order
  // ([a_rows, K] with scales [K/128, a_rows]; row i belongs to sorted position i), fetched by TMA
  // like the dense A tile instead of being gathered; stage-1 output written in the same order.
  int a_sorted;
  int out_sorted;
  int a_rows;
  // Stage 1 with the 1x128 re-quantisation fused into the epilogue (256-wide tiles, routing-order
  // output): fp8 rows [a_rows, N] and their scales [N/128, a_rows] instead of the 16-bit `out`.
  uint8_t* out_q;
  float* out_scale_t;
};

template <int BN, int MODE, typename OutT>
struct Cfg {
  static constexpr int kOutCols = (is_moe1(MODE)) ? BN / 2 : BN;   // output columns per tile
  // 16-bit outputs of tiles at least 64 wide go through a shared-memory staging tile.
  static constexpr bool kStaged = (sizeof(OutT) == 2) && (kOutCols >= 32) && (BN >= 64);
  static constexpr int kRegions = (kOutCols + 63) / 64;
  // The per-token mode is bound by its operand feed, and its epilogue has a whole tile's K loop to
  // get the previous tile out: it stages and stores a tile in two halves of 128 columns, which leaves
  // shared memory for a fourth pipeline stage.
  static constexpr bool kHalfStaging = (MODE == kDensePT) && (BN == 256);
  static constexpr int kStageRegions = kHalfStaging ? kRegions / 2 : kRegions;
  static constexpr int kCBytes = kStaged ? kStageRegions * kRegionBytes : 0;
  static constexpr int kBTileBytes = BN * BK;
  static constexpr int kStageBytes = kATileBytes + kBTileBytes;
  static constexpr int kMiscBytes = 2048;  // row offsets (1 KB) + barriers + flags
  static constexpr int kAvail = 232448 - 1024 - kMiscBytes;  // 227 KB less alignment slack and misc
  static constexpr int kStagesFit = (kAvail - kCBytes) / kStageBytes;
  static constexpr int kStages = kStagesFit > 10 ? 10 : kStagesFit;
  // Accumulator buffers in TMEM (512 columns per SM): as many as fit, at most 8. The MMA issuer may
  // run that many K blocks ahead of the epilogue, which hides the MMA-completion -> promotion ->
  // release round trip (about a thousand cycles) for the narrow tiles.
  static constexpr int kAccBufs = (512 / BN) > 8 ? 8 : (512 / BN);
  static constexpr int kTmemCols = BN * kAccBufs;
  static constexpr int kCH = BN / 4;  // columns per epilogue thread per column group
  static constexpr int kSmemBytes = kStages * kStageBytes + kCBytes + kMiscBytes + 1024;
  static_assert(kStages >= 3, "pipeline too shallow");
};

template <typename OutT>
__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 q;
  q.x = pack2(v[0], v[1], OutT());
  q.y = pack2(v[2], v[3], OutT());
  q.z = pack2(v[4], v[5], OutT());
  q.w = pack2(v[6], v[7], OutT());
  return q;
}
template <typename OutT>
__device__ __forceinline__ void store8(OutT* dst, const float* v) {
  *reinterpret_cast<uint4*>(dst) = pack8<OutT>(v);
}
template <>
__device__ __forceinline__ void store8<float>(float* dst, const float* v) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// Atomic accumulate of 8 consecutive outputs (stage 2, accumulate mode).
__device__ __forceinline__ void red8_packed(__nv_bfloat16* dst, const uint4& q) {
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(q.x),
               "r"(q.y), "r"(q.z), "r"(q.w)
               : "memory");
}
__device__ __forceinline__ void red8_packed(__half* dst, const uint4& q) {
  asm volatile("red.global.add.noftz.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(q.x),
               "r"(q.y), "r"(q.z), "r"(q.w)
               : "memory");
}
__device__ __forceinline__ void red8_packed(float*, const uint4&) {}  // f32 never takes the staged path
template <typename OutT>
__device__ __forceinline__ void red8(OutT* dst, const float* v) {
  red8_packed(dst, pack8<OutT>(v));
}
template <>
__device__ __forceinline__ void red8<float>(float* dst, const float* v) {
#pragma unroll
  for (int i = 0; i < 2; ++i)
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * i),
                 "f"(v[4 * i]), "f"(v[4 * i + 1]), "f"(v[4 * i + 2]), "f"(v[4 * i + 3])
                 : "memory");
}

__device__ __forceinline__ float round_through(float v, __half) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ float round_through(float v, __nv_bfloat16) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float round_through(float v, float) { return v; }

__device__ __forceinline__ float silu_mul(float g, float u) {
  // silu(g) * u with the fast exp, as the reference does (moe_blockscale_2stage.py:239-251).
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

// Tile bookkeeping shared by every role so that all of them walk the same sequence: tile
// blockIdx.x, then one grid further, and so on. A position carries (m block, n tile) and is advanced
// with additions only (the integer division happens once, in start()).
struct TilePos {
  int tile, m_blk, n_tile;
};
template <int BN, int MODE>
struct TileWalker {
  int num_m, num_n, total;
  int step_major, step_minor;  // gridDim.x split by the minor dimension's extent
  // Dense with many row blocks: they are taken in groups of group_m; inside a group the order is the
  // usual one (row blocks fastest, then column tiles), so a group's slice of A (group_m x 128 x K
  // bytes) stays in L2 while all column tiles pass over it, instead of the whole of A streaming
  // through L2 once per column tile. Positions are decoded with divisions then (once per tile).
  int group_m;
  // tile -> (m block, n tile). Dense: consecutive CTAs share the weight tile and differ in rows
  // (minor = m). MoE: every row block has its own expert's weights, so that order shares nothing and
  // re-reads the whole routing-ordered activation tensor once per column tile (350 MB at 4096 tokens
  // x top-8, more than L2); instead consecutive CTAs take the column tiles of ONE row block (minor =
  // n): its activation tile is fetched once and shared through L2, and the second row block of an
  // expert follows its first closely enough to find the expert's weights (29 MB) still in L2.
  static constexpr bool kRowBlockMajor = (!is_dense(MODE));
  __device__ __forceinline__ TileWalker(const GemmParams& p) {
    group_m = 0;
    if constexpr (is_dense(MODE)) {
      num_m = (p.M + BM - 1) / BM;
      num_n = (p.N + BN - 1) / BN;
      if (p.group_m > 0 && p.group_m < num_m) group_m = p.group_m;
    } else {
      int valid_rows = p.num_valid[0];
      int nb = (valid_rows + p.tile_m - 1) / p.tile_m;
      num_m = nb < p.num_blocks ? nb : p.num_blocks;
      if (num_m < 0) num_m = 0;
      constexpr int kColsPerTile = (is_moe1(MODE)) ? BN / 2 : BN;
      num_n = (p.N + kColsPerTile - 1) / kColsPerTile;
    }
    total = num_m * num_n;
    const int minor = kRowBlockMajor ? num_n : num_m;
    const int g = static_cast<int>(gridDim.x);
    step_major = minor > 0 ? g / minor : 0;
    step_minor = minor > 0 ? g - step_major * minor : 0;
  }
  __device__ __forceinline__ void decode_grouped(TilePos& t) const {
    const int per_group = group_m * num_n;
    const int g = t.tile / per_group;
    const int r = t.tile - g * per_group;
    const int rows_here = min(group_m, num_m - g * group_m);   // the last group may be shorter
    // tiles of the earlier groups are all full, so r indexes this group's own (rows_here x num_n) grid
    t.n_tile = r / rows_here;
    t.m_blk = g * group_m + (r - t.n_tile * rows_here);
  }
  __device__ __forceinline__ TilePos start() const {
    TilePos t;
    t.tile = static_cast<int>(blockIdx.x);
    if (is_dense(MODE) && group_m > 0) {
      if (t.tile < total) decode_grouped(t);
      else t.m_blk = t.n_tile = 0;
      return t;
    }
    const int minor = kRowBlockMajor ? num_n : num_m;
    const int hi = minor > 0 ? t.tile / minor : 0;
    const int lo = t.tile - hi * minor;
    t.m_blk = kRowBlockMajor ? hi : lo;
    t.n_tile = kRowBlockMajor ? lo : hi;
    return t;
  }
  __device__ __forceinline__ bool valid(const TilePos& t) const { return t.tile < total; }
  __device__ __forceinline__ void advance(TilePos& t) const {
    t.tile += static_cast<int>(gridDim.x);
    if (is_dense(MODE) && group_m > 0) {
      if (t.tile < total) decode_grouped(t);
      return;
    }
    int& lo = kRowBlockMajor ? t.n_tile : t.m_blk;
    int& hi = kRowBlockMajor ? t.m_blk : t.n_tile;
    const int minor = kRowBlockMajor ? num_n : num_m;
    lo += step_minor;
    hi += step_major;
    if (lo >= minor) {
      lo -= minor;
      ++hi;
    }
  }
};

template <int BN, int MODE, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
bs_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_c,
               const GemmParams p) {
  using C = Cfg<BN, MODE, OutT>;
  constexpr int kStages = C::kStages;
  constexpr int CH = C::kCH;
  extern __shared__ uint8_t smem_raw[];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t cstage_base = smem_base + kStages * C::kStageBytes;       // 1024-aligned
  const uint32_t misc_base = cstage_base + C::kCBytes;
  uint8_t* misc = smem_al + kStages * C::kStageBytes + C::kCBytes;
  long long* row_off = reinterpret_cast<long long*>(misc);                 // [128], MoE staged output
  const uint32_t bar_base = misc_base + 1024;
  // Barriers. full[s]: operands of stage s have landed. done[i]: the MMAs of K-block iteration i
  // (mod kDone) have finished -- ONE tcgen05.commit per K block serves both consumers: the loaders
  // (stage it % kStages may be refilled once iteration it - kStages is done) and the epilogue
  // (partials of iteration it are in TMEM). kDone > kStages and >= kAccBufs, so a barrier is never
  // re-armed before every waiter of its previous phase has passed. tempty[b]: the epilogue has read
  // accumulator buffer b (one barrier per buffer: every wait costs the single issuing thread about a
  // hundred cycles). Dense tiles: cfull = the 8 epilogue warps have staged a tile; cfree = the store
  // warp's TMA store has read the staging tile, which may be overwritten.
  constexpr int kAccBufs = C::kAccBufs;
  constexpr int kDone = kStages + kAccBufs;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto done_bar = [&](uint32_t i) { return bar_base + 8u * (kStages + i); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (kStages + kDone + b); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (kStages + kDone + kAccBufs + b); };   // kDensePT
  constexpr int kNumBars = kStages + kDone + 2 * kAccBufs + 3;
  static_assert(8 * kNumBars + 8 <= 1024, "barrier area overflows the misc block");
  const uint32_t epi_bar = bar_base + 8u * (kNumBars - 3);
  const uint32_t cfull_bar = bar_base + 8u * (kNumBars - 2);
  const uint32_t cfree_bar = bar_base + 8u * (kNumBars - 1);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(misc + 1024 + 8 * kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 1024 + 8 * kNumBars + 4);
  // wait until the stage that iteration `it` is about to overwrite has been consumed
  auto wait_stage_free = [&](uint32_t it, int code) -> bool {
    if (it < static_cast<uint32_t>(kStages)) return true;
    const uint32_t j = it - kStages;
    return mbar_wait(done_bar(j % kDone), (j / kDone) & 1, abort_flag, p.err, code);
  };

  // arrivals per stage: the producer's expect_tx (+ the two gather warps when rows are gathered)
  const bool gather_a = (!is_dense(MODE)) && !p.a_sorted;
  // MoE tiles that leave through the staging tile are written out by warps 2-3 while the epilogue
  // warps go on with the next tile -- when those warps are not gathering rows and the epilogue does
  // stays with the arithmetic.
  const bool moe_async_store = (!is_dense(MODE)) && C::kStaged && !gather_a;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(full_bar(s), gather_a ? 3 : 1);
    for (int i = 0; i < kDone; ++i) mbar_init(done_bar(i), 1);
    for (int b = 0; b < kAccBufs; ++b) mbar_init(tempty_bar(b), kEpiWarps);  // one arrival per warp
    for (int b = 0; b < kAccBufs; ++b) mbar_init(tfull_bar(b), 1);
    mbar_init(epi_bar, kEpiWarps);
    mbar_init(cfull_bar, kEpiWarps);
    mbar_init(cfree_bar, is_dense(MODE) ? 1 : 2);
    *abort_flag = 0;
    fence_proxy_async_smem();
    fence_barrier_init();
    if (is_dense(MODE) || p.a_sorted) prefetch_tensormap(&tmap_a);
    if constexpr (is_dense(MODE) && C::kStaged) prefetch_tensormap(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Everything above touched no global memory, so it may overlap the tail of the previous kernel in
  // the stream (programmatic dependent launch); nothing below starts before that kernel's results
  // are visible. The next kernel may begin its own set-up as soon as SMs become free.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const TileWalker<BN, MODE> walk(p);
  const int KB = p.K / BK;

  // Register re-balancing. setmaxnreg.inc blocks until the CTA's own pool (registers per thread at
  // launch x 384 threads = 168 x 384) can satisfy it, so the totals after the exchange must fit in
  // that pool: 40 x 128 + 232 x 256 = 64512 <= 64512.
  if (warp < kEpiWarp0) {
    reg_dealloc<40>();
    if (warp == 0 && lane == 0) {
      // ---------------- producer: weights (and dense A) via TMA ----------------
      uint32_t it = 0;
      bool alive = true;
      const uint64_t pol_evict_first = l2_policy_evict_first();
      auto load_w = [&](uint32_t dst, const uint8_t* src, uint32_t bytes, uint32_t bar, bool last_use) {
        if (last_use) bulk_load_hint(dst, src, bytes, bar, pol_evict_first);
        else bulk_load(dst, src, bytes, bar);
      };
      for (TilePos pos = walk.start(); walk.valid(pos) && alive; walk.advance(pos)) {
        const int m_blk = pos.m_blk, n_tile = pos.n_tile;
        const uint8_t* wbase = p.b;
        int rows_b;  // weight rows this tile brings per column group
        size_t row_stride_kb;  // bytes between consecutive K blocks of the repacked weight
        int n0;
        bool w_last_use = false;
        if constexpr (is_dense(MODE)) {
          n0 = n_tile * BN;
          rows_b = min(BN, p.N - n0);
          row_stride_kb = static_cast<size_t>(p.N) * BK;
        } else {
          const int e = p.expert_ids[m_blk];
          if (e < 0 || e >= p.experts) continue;
          // An expert's weights are read by its row blocks only: the last of them marks the lines
          // "evict first", which keeps L2 for the activations and for weights that a following row
          // block still needs.
          w_last_use = (m_blk + 1 >= walk.num_m) || (p.expert_ids[m_blk + 1] != e);
          if constexpr (is_moe1(MODE)) {
            n0 = n_tile * (BN / 2);
            rows_b = min(BN / 2, p.N - n0);
            wbase += static_cast<size_t>(e) * 2 * p.N * p.K;
            row_stride_kb = static_cast<size_t>(2 * p.N) * BK;
          } else {
            n0 = n_tile * BN;
            rows_b = min(BN, p.N - n0);
            wbase += static_cast<size_t>(e) * p.N * p.K;
            row_stride_kb = static_cast<size_t>(p.N) * BK;
          }
        }
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kStages;
          if (!wait_stage_free(it, kErrWaitSmemEmpty)) {
            alive = false;
            break;
          }
          const uint32_t sa = smem_base + s * C::kStageBytes;
          const uint32_t sb = sa + kATileBytes;
          const uint8_t* src = wbase + kb * row_stride_kb + static_cast<size_t>(n0) * BK;
          if constexpr (is_dense(MODE)) {
            mbar_arrive_expect_tx(full_bar(s), p.a_box_rows * BK + rows_b * BK);
            tma_load_2d(sa, &tmap_a, kb * BK, m_blk * BM, full_bar(s));
            bulk_load(sb, src, rows_b * BK, full_bar(s));
          } else if constexpr (is_moe1(MODE)) {
            mbar_arrive_expect_tx(full_bar(s), 2 * rows_b * BK + (p.a_sorted ? p.a_box_rows * BK : 0));
            if (p.a_sorted) tma_load_2d(sa, &tmap_a, kb * BK, m_blk * p.tile_m, full_bar(s));
            load_w(sb, src, rows_b * BK, full_bar(s), w_last_use);
            load_w(sb + (BN / 2) * BK, src + static_cast<size_t>(p.N) * BK, rows_b * BK, full_bar(s),
                   w_last_use);
          } else {
            mbar_arrive_expect_tx(full_bar(s), rows_b * BK + (p.a_sorted ? p.a_box_rows * BK : 0));
            if (p.a_sorted) tma_load_2d(sa, &tmap_a, kb * BK, m_blk * p.tile_m, full_bar(s));
            load_w(sb, src, rows_b * BK, full_bar(s), w_last_use);
          }
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------- MMA issuer ----------------
      // One thread issues every MMA of the CTA. (Per K block it spends ~60-100 cycles in each barrier
      // wait, ~64 per tcgen05.mma and ~50-100 in the commit, less than the 512 cycles the tensor core
      // needs; a second issuing thread taking alternate K blocks was measured to change nothing,
      // the epilogue being the slower side.)
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(BM, BN);
      uint32_t it = 0;
      uint32_t tiles_issued = 0;   // kDensePT
      bool alive = true;
      for (TilePos pos = walk.start(); walk.valid(pos) && alive; walk.advance(pos)) {
        if constexpr (!is_dense(MODE)) {
          const int e = p.expert_ids[pos.m_blk];
          if (e < 0 || e >= p.experts) continue;
        }
        if constexpr (is_pt(MODE)) {
          // one accumulator buffer per TILE: wait for it once, accumulate every K block into it,
          // then tell the epilogue; the per-K-block commits only hand the stages back
          const int buf = static_cast<int>(tiles_issued % kAccBufs);
          if (!mbar_wait(tempty_bar(buf), ((tiles_issued / kAccBufs) & 1) ^ 1, abort_flag, p.err,
                         kErrWaitTmemEmpty)) {
            alive = false;
            break;
          }
          const uint32_t d = tmem_base + buf * BN;
          for (int kb = 0; kb < KB; ++kb, ++it) {
            const int s = it % kStages;
            const uint32_t sa = smem_base + s * C::kStageBytes;
            const uint64_t adesc = umma_desc_sw128(sa);
            const uint64_t bdesc = umma_desc_sw128(sa + kATileBytes);
            if (!mbar_wait(full_bar(s), (it / kStages) & 1, abort_flag, p.err, kErrWaitSmemFull)) {
              alive = false;
              break;
            }
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < BK / 32; ++k)
              tc_mma_f8(d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) ? 1u : 0u);
            tc_commit(done_bar(it % kDone));
          }
          if (!alive) break;
          tc_commit(tfull_bar(buf));
          ++tiles_issued;
          continue;
        }
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          const int buf = it % kAccBufs;
          const uint32_t tph = (it / kAccBufs) & 1;
          const uint32_t sa = smem_base + s * C::kStageBytes;
          const uint64_t adesc = umma_desc_sw128(sa);
          const uint64_t bdesc = umma_desc_sw128(sa + kATileBytes);
          const uint32_t d = tmem_base + buf * BN;
          // The operands normally landed long ago; the accumulator buffer is what the issuer really
          // waits for, so that wait comes last and nothing but the fence separates it from the MMAs.
          if (!mbar_wait(full_bar(s), ph, abort_flag, p.err, kErrWaitSmemFull) ||
              !mbar_wait(tempty_bar(buf), tph ^ 1, abort_flag, p.err, kErrWaitTmemEmpty)) {
            alive = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            tc_mma_f8(d, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
          // the MMAs of the K block are done: partial sums in TMEM, operands consumed
          tc_commit(done_bar(it % kDone));
        }
      }
    } else if (is_dense(MODE) && C::kStaged && warp == 2 && lane == 0) {
      // ---------------- dense: output store ----------------
      // One thread turns every staged tile into TMA stores, so the epilogue warps neither wait for
      // one another nor for the store engine at a tile boundary: they signal cfull and go on to the
      // next tile's first K block; cfree tells them when the staging tile may be overwritten.
      uint32_t n = 0;
      bool ok = true;
      for (TilePos pos = walk.start(); walk.valid(pos) && ok; walk.advance(pos)) {
        const int m_blk = pos.m_blk;
        constexpr int kPasses = C::kRegions / C::kStageRegions;   // 2 with half-tile staging
#pragma unroll
        for (int h = 0; h < kPasses; ++h, ++n) {
          if (!mbar_wait(cfull_bar, n & 1, abort_flag, p.err, kErrWaitEpilogue)) {
            ok = false;
            break;
          }
          const int n0 = pos.n_tile * BN + h * C::kStageRegions * 64;
#pragma unroll
          for (int reg = 0; reg < C::kStageRegions; ++reg)
            if (n0 + reg * 64 < p.N)
              tma_store_2d(&tmap_c, cstage_base + reg * kRegionBytes, n0 + reg * 64, m_blk * BM);
          bulk_commit_group();
          bulk_wait_group_read0();
          mbar_arrive(cfree_bar);
        }
      }
      bulk_wait_group0();  // every store has been written before the CTA exits
    } else if (!is_dense(MODE) && C::kStaged && warp >= 2 && moe_async_store) {
      // ---------------- MoE: output store (routing-order activations) ----------------
      // Warps 2-3 copy every staged tile to its output rows (row_off: element offset of each row,
      // -1 for rows without a token) while the epilogue warps run the next tile's K loop: cfull
      // says the tile and its row offsets are staged, cfree gives both back.
      if constexpr (C::kStaged) {
        OutT* const out = reinterpret_cast<OutT*>(p.out);
        constexpr int CPR = C::kOutCols / 8;   // 16-byte chunks per output row
        constexpr int RPI = 32 / CPR;          // rows per warp instruction
        const int sw = warp - 2;
        const int rows = min(BM, p.tile_m);
        const int ch = lane % CPR;
        const int col = ch * 8;
        uint32_t n = 0;
        for (TilePos pos = walk.start(); walk.valid(pos); walk.advance(pos)) {
          const int e = p.expert_ids[pos.m_blk];
          if (e < 0 || e >= p.experts) continue;
          const bool ok = mbar_wait(cfull_bar, n & 1, abort_flag, p.err, kErrWaitEpilogue);
          if (!__all_sync(0xffffffffu, ok)) break;
          ++n;
          const int n0 = pos.n_tile * C::kOutCols;
          if (MODE == kMoe1 && BN == 256 && p.out_q) {
            // re-quantised tile: 128 rows x 128 fp8 bytes in region 0, the rows' scales in region 1
            const float* scale_s = reinterpret_cast<const float*>(smem_al + kStages * C::kStageBytes +
                                                                  kRegionBytes) + 2 * BM;
            const int c8 = lane & 7;   // 8 chunks of 16 bytes per row
            if (n0 + 128 <= p.N) {
              for (int r0 = sw * 4; r0 < rows; r0 += 8) {
                const int rr = r0 + (lane >> 3);
                if (rr < rows) {
                  const long long srow = row_off[rr];
                  if (srow >= 0) {
                    const uint32_t addr = cstage_base + rr * 128 + ((c8 ^ (rr & 7)) << 4);
                    uint4 q;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                                 : "r"(addr)
                                 : "memory");
                    *reinterpret_cast<uint4*>(p.out_q + srow * p.N + n0 + c8 * 16) = q;
                    if (c8 == 0)
                      p.out_scale_t[static_cast<long long>(n0 / 128) * p.a_rows + srow] = scale_s[rr];
                  }
                }
              }
            }
          } else if (n0 + col + 8 <= p.N) {
            for (int r0 = sw * RPI; r0 < rows; r0 += 2 * RPI) {
              const int rr = r0 + lane / CPR;
              if (rr < rows) {
                const long long off = row_off[rr];
                if (off >= 0) {
                  const uint32_t addr = cstage_base + (col >> 6) * kRegionBytes + rr * 128 +
                                        ((((col & 63) >> 3) ^ (rr & 7)) << 4);
                  uint4 q;
                  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                               : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                               : "r"(addr)
                               : "memory");
                  OutT* dst = out + off + n0 + col;
                  if (is_moe2(MODE) && p.accumulate)
                    red8_packed(dst, q);
                  else
                    *reinterpret_cast<uint4*>(dst) = q;
                }
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(cfree_bar);
        }
      }
    } else if (!is_dense(MODE) && warp >= 2 && gather_a) {
      // ---------------- MoE: gather activation rows with cp.async ----------------
      // Thread g owns rows g and g+64 of the tile; row r, 16-byte chunk c lands at
      // r*128 + ((c ^ (r & 7)) << 4): the 128-byte-swizzled K-major image.
      constexpr int kDepth = (kStages > 4) ? 3 : 2;  // groups in flight before a stage is published
      static_assert(kDepth < kStages, "gather look-ahead must stay below the ring depth");
      const int g = threadIdx.x - 64;
      uint32_t it = 0, published = 0;
      bool alive = true;
      const size_t row_bytes = static_cast<size_t>(p.K);
      for (TilePos pos = walk.start(); walk.valid(pos) && alive; walk.advance(pos)) {
        const int m_blk = pos.m_blk;
        const int e = p.expert_ids[m_blk];
        if (e < 0 || e >= p.experts) continue;
        const uint8_t* src_row[2];
        uint32_t src_ok[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = g + 64 * h;
          src_row[h] = p.a;
          src_ok[h] = 0;
          if (r < p.tile_m) {
            const int id = p.sorted_ids[m_blk * p.tile_m + r];
            const int t = id & 0xFFFFFF;
            const int slot = static_cast<unsigned>(id) >> 24;
            if (t < p.M && slot < p.topk) {
              const size_t row = (is_moe1(MODE)) ? static_cast<size_t>(t)
                                                 : static_cast<size_t>(t) * p.topk + slot;
              src_row[h] = p.a + row * row_bytes;
              src_ok[h] = 16;
            }
          }
        }
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kStages;
          if (!wait_stage_free(it, kErrWaitGather)) {
            alive = false;
            break;
          }
          const uint32_t sa = smem_base + s * C::kStageBytes;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int r = g + 64 * h;
            if (r < p.tile_m) {
              const uint8_t* src = src_row[h] + (src_ok[h] ? kb * BK : 0);
#pragma unroll
              for (int c = 0; c < 8; ++c)
                cp_async_16(sa + r * 128 + ((c ^ (r & 7)) << 4), src + c * 16, src_ok[h]);
            }
          }
          cp_async_commit();
          if (it - published >= static_cast<uint32_t>(kDepth)) {
            cp_async_wait<kDepth>();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(full_bar(published % kStages));
            ++published;
          }
        }
      }
      // drain: publish whatever was issued
      cp_async_wait<0>();
      fence_proxy_async_smem();
      __syncwarp();
      if (alive && lane == 0)
        for (; published < it; ++published) mbar_arrive(full_bar(published % kStages));
    }
  } else {
    // ---------------- epilogue warps: scale promotion + output ----------------
    reg_alloc<232>();
    const int ew = warp - kEpiWarp0;
    const int quad = warp & 3;   // TMEM lane quadrant this warp may read
    const int half = ew >> 2;    // which CH-wide slice of each column group
    const int r = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    OutT* const out = reinterpret_cast<OutT*>(p.out);

    uint32_t it = 0;
    uint32_t epi_phase = 0;
    bool alive = true;
    // Barrier among the 256 epilogue threads (bounded like every other wait).
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(epi_bar);
      const bool ok = mbar_wait(epi_bar, epi_phase, abort_flag, p.err, kErrWaitEpilogue);
      epi_phase ^= 1;
      return __all_sync(0xffffffffu, ok);
    };

    // What the promotion loop needs per tile: where this thread's scales of K block 0 live. The loop
    // only bumps these pointers: a warp that runs a chain of dependent scalar instructions issues one
    // every 4-6 cycles, so index arithmetic per K block shows up directly in the K-block period.
    // Rows without a valid token read the scales of row 0 (their results are never stored).
    struct ScaleCtx {
      const float* sa;     // scale_a of this thread's row; K block kb at sa + kb * sa_step
      const float* sb0;    // scale_b of column group 0; K block kb at sb0 + kb
      const float* sb1;    // ... group 1
      long long sa_step;
      int c0, c1;          // per-token MoE modes: first output channel of group 0 / 1 (range check)
      bool active;         // MoE: some row of this warp's 32 holds a token (warp-uniform)
    };
    // What the store phase needs; recomputed after the loop instead of being kept live through it.
    struct OutCtx {
      size_t out_row;
      int n0;                // first output column of the tile
      int col0, col1;        // tile-relative first output column of group 0 / group 1
      int m_blk;
      float route_w;
      bool row_ok;
    };
    // decode (token, slot) of this thread's row for MoE tiles
    auto moe_row = [&](int m_blk, int& t, int& slot) -> bool {
      t = 0; slot = 0;
      if (r >= p.tile_m) return false;
      const int id = p.sorted_ids[m_blk * p.tile_m + r];
      const int tt = id & 0xFFFFFF;
      const int ss = static_cast<unsigned>(id) >> 24;
      if (tt >= p.M || ss >= p.topk) return false;
      t = tt; slot = ss;
      return true;
    };
    // Fills the scale context of `tile`; false if the tile has nothing to do (MoE block without expert).
    auto setup_scales = [&](const TilePos& pos, ScaleCtx& c) -> bool {
      const int m_blk = pos.m_blk, n_tile = pos.n_tile;
      long long sa_idx, sb_idx0, sb_idx1;
      if constexpr (is_dense(MODE)) {
        const int row = m_blk * BM + r;
        sa_idx = row < p.M ? row : 0;
        c.sa_step = p.M;
        const int n0 = n_tile * BN;
        const int nblk_max = (p.N + 127) / 128 - 1;
        sb_idx0 = static_cast<long long>(min((n0 + half * CH) / 128, nblk_max)) * KB;
        sb_idx1 = static_cast<long long>(min((n0 + BN / 2 + half * CH) / 128, nblk_max)) * KB;
      } else {
        const int e = p.expert_ids[m_blk];
        if (e < 0 || e >= p.experts) return false;
        int t, slot;
        // (0, 0) for rows without a valid token. A warp whose 32 rows are all padding (most of an
        // expert's second row block) skips the TMEM reads and the promotion of the whole tile: its
        // results are never stored, and the kernel runs against the power cap.
        c.active = __any_sync(0xffffffffu, moe_row(m_blk, t, slot));
        if (p.a_sorted) {   // scales follow the permuted activations: one per sorted row
          sa_idx = static_cast<long long>(m_blk) * p.tile_m + (r < p.tile_m ? r : 0);
          c.sa_step = p.a_rows;
        }
        if constexpr (is_moe1(MODE)) {
          if (!p.a_sorted) {
            sa_idx = t;
            c.sa_step = p.M;
          }
          if constexpr (is_pt(MODE)) {
            // one weight scale per output channel: gate channel c of expert e at e*2N + c, up at +N
            c.c0 = c.c1 = n_tile * (BN / 2) + half * CH;
            sb_idx0 = static_cast<long long>(e) * 2 * p.N + c.c0;
            sb_idx1 = sb_idx0 + p.N;
          } else {
            const long long nb_exp = (2 * p.N) / 128;  // scale rows per expert
            const int cg = min(n_tile * (BN / 2) + half * CH, p.N - 1);
            sb_idx0 = (e * nb_exp + cg / 128) * KB;
            sb_idx1 = (e * nb_exp + (p.N + cg) / 128) * KB;
          }
        } else {
          if (!p.a_sorted) {
            sa_idx = static_cast<long long>(t) * p.topk + slot;
            c.sa_step = static_cast<long long>(p.M) * p.topk;
          }
          const int n0 = n_tile * BN;
          if constexpr (is_pt(MODE)) {
            c.c0 = n0 + half * CH;
            c.c1 = c.c0 + BN / 2;
            sb_idx0 = static_cast<long long>(e) * p.N + c.c0;
            sb_idx1 = sb_idx0 + BN / 2;
          } else {
            const long long nb_exp = p.N / 128;
            sb_idx0 = (e * nb_exp + min(n0 + half * CH, p.N - 1) / 128) * KB;
            sb_idx1 = (e * nb_exp + min(n0 + BN / 2 + half * CH, p.N - 1) / 128) * KB;
          }
        }
      }
      c.sa = p.scale_a + sa_idx;
      c.sb0 = p.scale_b + sb_idx0;
      c.sb1 = p.scale_b + sb_idx1;
      return true;
    };
    auto setup_output = [&](const TilePos& pos, OutCtx& c) {
      const int m_blk = pos.m_blk, n_tile = pos.n_tile;
      c.m_blk = m_blk;
      c.route_w = 1.0f;
      if constexpr (is_dense(MODE)) {
        const int row = m_blk * BM + r;
        c.row_ok = row < p.M;
        c.n0 = n_tile * BN;
        c.col0 = half * CH;
        c.col1 = BN / 2 + half * CH;
        c.out_row = static_cast<size_t>(row) * p.N;
      } else {
        int t, slot;
        c.row_ok = moe_row(m_blk, t, slot);
        if (c.row_ok && p.doweight) c.route_w = p.sorted_weights[m_blk * p.tile_m + r];
        if constexpr (is_moe1(MODE)) {
          c.n0 = n_tile * (BN / 2);
          c.col0 = c.col1 = half * CH;
          c.out_row = p.out_sorted ? static_cast<size_t>(m_blk * p.tile_m + r) * p.N
                                   : (static_cast<size_t>(t) * p.topk + slot) * p.N;
        } else {
          c.n0 = n_tile * BN;
          c.col0 = half * CH;
          c.col1 = BN / 2 + half * CH;
          c.out_row = p.accumulate ? static_cast<size_t>(t) * p.N
                                   : (static_cast<size_t>(t) * p.topk + slot) * p.N;
        }
      }
    };
    // first position at or after `pos` (stepping by the grid) that has work
    auto find_tile = [&](TilePos& pos, ScaleCtx& c) {
      while (walk.valid(pos) && !setup_scales(pos, c)) walk.advance(pos);
    };

    // Scales are prefetched kRing K blocks ahead into a register ring; the ring of the NEXT tile is
    // loaded before the current tile's store phase so that its latency hides behind the stores.
    constexpr int kRing = 2;
    ScaleCtx cur;
    float ring_a[kRing], ring_b0[kRing], ring_b1[kRing];
    TilePos pos = walk.start();
    find_tile(pos, cur);
    if (!is_pt(MODE) && walk.valid(pos)) {
#pragma unroll
      for (int j = 0; j < kRing; ++j) {
        const int kb = j < KB ? j : 0;
        ring_a[j] = __ldg(cur.sa + kb * cur.sa_step);
        ring_b0[j] = __ldg(cur.sb0 + kb);
        ring_b1[j] = __ldg(cur.sb1 + kb);
      }
    }

    // Columns per tcgen05.ld. Measured on B200 (MMA issuer + epilogue alone, no loads): 16-, 32- and
    // 64-column loads give the same K-block period (608-630 cycles against 512 of MMA) -- the TMEM
    // read path moves one 32-lane column per cycle and sub-partition, 256 cycles per 128 x 256 block,
    // whatever the instruction width -- so the narrowest pipelined load, which needs the fewest
    // registers, stays.
    constexpr int LDW = (CH > 32) ? 16 : CH;
    constexpr int NSUB = CH / LDW;            // loads per column group
    constexpr int NQ = 2 * NSUB;              // loads per K block (two column groups)
    uint32_t tiles_done = 0;                  // dense: tiles (per-token mode: half tiles) staged so far
    uint32_t pt_tiles = 0;                    // per-token mode: tiles drained so far
    uint32_t dn_i = 0, dn_ph = 0;             // it % kDone and (it / kDone) & 1, kept as counters

    while (walk.valid(pos) && alive) {
      // acc[0 .. CH/2) = column group 0, acc[CH/2 .. CH) = column group 1, two columns per float2.
      float2 acc[CH];
#pragma unroll
      for (int j = 0; j < CH; ++j) acc[j] = make_float2(0.f, 0.f);
      // addresses of the scales that the next prefetch takes (K block kRing of this tile)
      const float* pf_a = cur.sa + kRing * cur.sa_step;
      const float* pf_b0 = cur.sb0 + kRing;
      const float* pf_b1 = cur.sb1 + kRing;
      const long long pf_step = cur.sa_step;

      ScaleCtx nxt;
      float nring_a[kRing], nring_b0[kRing], nring_b1[kRing];
      TilePos npos = pos;
      for (int kb0 = 0; !is_pt(MODE) && kb0 < KB && alive; kb0 += kRing) {
        if (kb0 + kRing >= KB) {
          // last trip: the next tile's scale context and first scales are fetched now, so that their
          // latency is over when the store phase ends
          walk.advance(npos);
          find_tile(npos, nxt);
          if (walk.valid(npos)) {
#pragma unroll
            for (int j = 0; j < kRing; ++j) {
              const int kbn = j < KB ? j : 0;
              nring_a[j] = __ldg(nxt.sa + kbn * nxt.sa_step);
              nring_b0[j] = __ldg(nxt.sb0 + kbn);
              nring_b1[j] = __ldg(nxt.sb1 + kbn);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < kRing; ++j) {
          const int kb = kb0 + j;
          if (kb < KB && alive) {
            const int buf = it % kAccBufs;
            const float s0 = ring_a[j] * ring_b0[j];
            const float s1 = ring_a[j] * ring_b1[j];
            if (kb + kRing < KB) {
              ring_a[j] = __ldg(pf_a);
              ring_b0[j] = __ldg(pf_b0);
              ring_b1[j] = __ldg(pf_b1);
            }
            pf_a += pf_step;
            ++pf_b0;
            ++pf_b1;
            const uint32_t t0 = tmem_base + lane_base + buf * BN + half * CH;
            auto taddr = [&](int q) {  // load q: q < NSUB -> group 0, else group 1
              return t0 + (q >= NSUB ? BN / 2 : 0) + (q % NSUB) * LDW;
            };
            // warp-uniform outcome: the tcgen05.ld below needs the whole warp
            const bool got = mbar_wait(done_bar(dn_i), dn_ph, abort_flag, p.err, kErrWaitTmemFull);
            if (!__all_sync(0xffffffffu, got)) {
              alive = false;
              break;
            }
            tc_fence_after();
            auto release = [&]() {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(tempty_bar(buf));
            };
            // Loads of LDW columns are software-pipelined against the FMAs of the previous load (two
            // register buffers); the buffer goes back to the issuer as soon as the last load landed.
            uint32_t va[LDW], vb[LDW];
            if (!is_dense(MODE) && !cur.active) {
              release();
            } else {
            tmem_ld<LDW>(taddr(0), va);
            tmem_wait_dep<LDW>(va);
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
              uint32_t* cv = (q & 1) ? vb : va;
              uint32_t* nv = (q & 1) ? va : vb;
              if (q + 1 < NQ) tmem_ld<LDW>(taddr(q + 1), nv);   // in flight during the FMAs
              const float s = (q >= NSUB) ? s1 : s0;
              const float2 s2 = make_float2(s, s);
              float2* a = acc + (q >= NSUB ? CH / 2 : 0) + (q % NSUB) * (LDW / 2);
#pragma unroll
              for (int c = 0; c < LDW / 2; ++c)
                a[c] = __ffma2_rn(make_float2(__uint_as_float(cv[2 * c]),
                                              __uint_as_float(cv[2 * c + 1])), s2, a[c]);
              if (q + 1 < NQ) {
                tmem_wait_dep<LDW>(nv);
                if (q + 2 == NQ) release();
              }
            }
            }
            ++it;
            if (++dn_i == kDone) {
              dn_i = 0;
              dn_ph ^= 1;
            }
          }
        }
      }
      if constexpr (is_pt(MODE)) {
        // Per-token / per-channel scales: the tile's whole K range has been accumulated in TMEM
        // buffer pt_tiles % kAccBufs; read it once, scale by sa[row] * sb[column], hand it back.
        walk.advance(npos);
        if constexpr (!is_dense(MODE)) find_tile(npos, nxt);
        const int buf = static_cast<int>(pt_tiles % kAccBufs);
        const bool got = mbar_wait(tfull_bar(buf), (pt_tiles / kAccBufs) & 1, abort_flag, p.err,
                                   kErrWaitTmemFull);
        ++pt_tiles;
        if (!__all_sync(0xffffffffu, got)) {
          alive = false;
          break;
        }
        tc_fence_after();
        // this thread's row scale, and for each column group the address of its first channel's
        // scale and that channel's index (channels at or beyond N are not read)
        float sa;
        const float *sbp0, *sbp1;
        int cb0, cb1;
        if constexpr (is_dense(MODE)) {
          const int row = pos.m_blk * BM + r;
          sa = row < p.M ? __ldg(p.scale_a + row) : 0.f;
          cb0 = pos.n_tile * BN + half * CH;
          cb1 = cb0 + BN / 2;
          sbp0 = p.scale_b + cb0;
          sbp1 = p.scale_b + cb1;
        } else {
          sa = __ldg(cur.sa);
          cb0 = cur.c0;
          cb1 = cur.c1;
          sbp0 = cur.sb0;
          sbp1 = cur.sb1;
        }
        if (!is_dense(MODE) && !cur.active) {
          // a warp whose rows are all padding hands the buffer back unread
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(buf));
        } else {
        const uint32_t t0 = tmem_base + lane_base + buf * BN + half * CH;
        auto taddr = [&](int q) { return t0 + (q >= NSUB ? BN / 2 : 0) + (q % NSUB) * LDW; };
        uint32_t va[LDW], vb[LDW];
        tmem_ld<LDW>(taddr(0), va);
        tmem_wait_dep<LDW>(va);
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          uint32_t* cv = (q & 1) ? vb : va;
          uint32_t* nv = (q & 1) ? va : vb;
          if (q + 1 < NQ) tmem_ld<LDW>(taddr(q + 1), nv);
          const int off = (q % NSUB) * LDW;   // first channel of this load inside its group
          const float* sbp = (q >= NSUB ? sbp1 : sbp0) + off;
          float2* a = acc + (q >= NSUB ? CH / 2 : 0) + (q % NSUB) * (LDW / 2);
          // N % 16 == 0: a load's channels are all in or all out
          const bool in_n = (q >= NSUB ? cb1 : cb0) + off < p.N;
#pragma unroll
          for (int c = 0; c < LDW / 2; ++c) {
            const float s0 = in_n ? sa * __ldg(sbp + 2 * c) : 0.f;
            const float s1 = in_n ? sa * __ldg(sbp + 2 * c + 1) : 0.f;
            a[c] = make_float2(__uint_as_float(cv[2 * c]) * s0, __uint_as_float(cv[2 * c + 1]) * s1);
          }
          if (q + 1 < NQ) {
            tmem_wait_dep<LDW>(nv);
            if (q + 2 == NQ) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(tempty_bar(buf));
            }
          }
        }
        }
      }
      if (!alive) break;

      OutCtx oc;
      setup_output(pos, oc);
      const bool row_ok = oc.row_ok;
      const int m_blk = oc.m_blk;
      const int n0 = oc.n0, col0 = oc.col0, col1 = oc.col1;
      const size_t out_row = oc.out_row;
      const float route_w = oc.route_w;
      const float* accf = reinterpret_cast<const float*>(acc);  // [0,CH) group 0, [CH,2CH) group 1
      // ---- output ----
      if constexpr (C::kStaged) {
        // (1) the staging tile must be free. Dense: the store warp's TMA store of the previous tile
        //     has read it (cfree; 16 K blocks have passed, so this wait is normally over at once).
        //     MoE: the previous tile's cooperative row stores are done (every thread passes this
        //     barrier after its own).
        if constexpr (is_dense(MODE)) {
          if (tiles_done > 0) {
            const bool ok = mbar_wait(cfree_bar, (tiles_done - 1) & 1, abort_flag, p.err, kErrWaitEpilogue);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
          }
        } else if (moe_async_store) {
          if (tiles_done > 0) {
            const bool ok = mbar_wait(cfree_bar, (tiles_done - 1) & 1, abort_flag, p.err, kErrWaitEpilogue);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
          }
        } else {
          if (!epi_sync()) { alive = false; break; }
        }
        // (2) thread r writes its columns of row r into the swizzled staging tile
        auto stage8 = [&](int col, const float* v) {   // col: tile-relative output column, % 8 == 0
          const uint32_t addr = cstage_base + (col >> 6) * kRegionBytes + r * 128 +
                                ((((col & 63) >> 3) ^ (r & 7)) << 4);
          const uint4 q = pack8<OutT>(v);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(q.x), "r"(q.y),
                       "r"(q.z), "r"(q.w)
                       : "memory");
        };
        bool tile_stored = false;
        if constexpr (MODE == kMoe1 && BN == 256) {
          if (p.out_q) {
            // Fused 1x128 re-quantisation (what flyb200_quant_1x128 does to the 16-bit stage-1
            // output, bit for bit): the tile's 128 output columns are exactly one scale group of
            // each row. Values are rounded through the 16-bit type first, as the unfused path
            // stores them; the row's two threads (64 columns each) exchange their amax through
            // shared memory. fp8 tile: 128 rows x 128 bytes in staging region 0 (16-byte chunks
            // swizzled by row); amax/scale scratch in region 1.
            float* amax_s = reinterpret_cast<float*>(smem_al + kStages * C::kStageBytes + kRegionBytes);
            float* scale_s = amax_s + 2 * BM;
            float* yq = const_cast<float*>(accf);   // y overwrites the gate half of the accumulators
            float vmax = -3.4e38f, vmin = 3.4e38f;
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              float v = round_through(silu_mul(accf[j], accf[CH + j]) * route_w, OutT());
              if (v != v) v = 0.f;
              else if (isinf(v)) v = v > 0.f ? 448.f : -448.f;
              yq[j] = v;
              vmax = fmaxf(vmax, v);
              vmin = fminf(vmin, v);
            }
            amax_s[half * BM + r] = fmaxf(vmax, -vmin);
            if (!epi_sync()) { alive = false; break; }
            float scale = __fdiv_rn(fmaxf(amax_s[r], amax_s[BM + r]), 448.f);
            if (scale == 0.f) scale = 1.f;
            // y / scale, correctly rounded, from one reciprocal: q0 = y*rc, q = fma(fma(-scale, q0,
            // y), rc, q0) is the IEEE quotient when rc is the correctly rounded reciprocal and the
            // mantissa of scale is not all ones (Markstein); that rare scale takes the true
            // division. |y / scale| <= 448, so nothing overflows; 64 IEEE divisions per thread per
            // tile were measured to cost more than the separate quantiser kernel saves.
            const float rc = __frcp_rn(scale);
            const bool exact_div = (__float_as_uint(scale) & 0x7fffffu) == 0x7fffffu;
            auto quot = [&](float y) -> float {
              if (exact_div) return __fdiv_rn(y, scale);
              const float q0 = y * rc;
              const float qc = __fmaf_rn(__fmaf_rn(-scale, q0, y), rc, q0);
              // the sign of y, for the one case the correction step loses it: -0 / scale = -0
              return __uint_as_float(__float_as_uint(qc) | (__float_as_uint(y) & 0x80000000u));
            };
#pragma unroll
            for (int j = 0; j < CH; j += 16) {
              uint32_t w4[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float* y4 = yq + j + 4 * q;
                const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(quot(y4[0]), quot(y4[1])),
                                                             __NV_SATFINITE, __NV_E4M3);
                const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(quot(y4[2]), quot(y4[3])),
                                                             __NV_SATFINITE, __NV_E4M3);
                w4[q] = lo | (hi << 16);
              }
              const int chunk = (half * CH + j) >> 4;
              const uint32_t addr = cstage_base + r * 128 + ((chunk ^ (r & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w4[0]), "r"(w4[1]),
                           "r"(w4[2]), "r"(w4[3])
                           : "memory");
            }
            if (half == 0) {
              row_off[r] = row_ok ? static_cast<long long>(m_blk * p.tile_m + r) : -1LL;  // sorted row
              scale_s[r] = scale;
            }
            if (moe_async_store) {   // the store warps write the rows and scales out
              __syncwarp();
              if (lane == 0) mbar_arrive(cfull_bar);
              ++tiles_done;
            } else {
            if (!epi_sync()) { alive = false; break; }
            const int rows = min(BM, p.tile_m);
            const int ch = lane & 7;                       // 8 chunks of 16 bytes per row
            if (n0 + 128 <= p.N) {
              for (int r0 = ew * 4; r0 < rows; r0 += kEpiWarps * 4) {
                const int rr = r0 + (lane >> 3);
                if (rr < rows) {
                  const long long srow = row_off[rr];
                  if (srow >= 0) {
                    const uint32_t addr = cstage_base + rr * 128 + ((ch ^ (rr & 7)) << 4);
                    uint4 q;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                                 : "r"(addr)
                                 : "memory");
                    *reinterpret_cast<uint4*>(p.out_q + srow * p.N + n0 + ch * 16) = q;
                    if (ch == 0)
                      p.out_scale_t[static_cast<long long>(n0 / 128) * p.a_rows + srow] = scale_s[rr];
                  }
                }
              }
            }
            }
            tile_stored = true;
          }
        }
        if (tile_stored) {
          // nothing left to do for this tile
        } else if constexpr (is_moe1(MODE)) {
#pragma unroll
          for (int j = 0; j < CH; j += 8) {
            float y[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) y[q] = silu_mul(accf[j + q], accf[CH + j + q]) * route_w;
            stage8(col0 + j, y);
          }
        } else if constexpr (C::kHalfStaging) {
          // column group 0 (tile columns [0, 128)) and group 1 ([128, 256)) go through the same two
          // staging regions one after the other; each is handed to the store thread on its own
#pragma unroll
          for (int grp = 0; grp < 2; ++grp) {
            if (grp == 1) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) mbar_arrive(cfull_bar);
              ++tiles_done;
              const bool ok = mbar_wait(cfree_bar, (tiles_done - 1) & 1, abort_flag, p.err, kErrWaitEpilogue);
              if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            }
#pragma unroll
            for (int j = 0; j < CH; j += 8) {
              float y[8];
#pragma unroll
              for (int q = 0; q < 8; ++q) y[q] = accf[grp * CH + j + q];
              stage8(col0 + j, y);   // col0 = this thread's columns inside a 128-column half
            }
          }
          if (!alive) break;
        } else {
#pragma unroll
          for (int grp = 0; grp < 2; ++grp) {
#pragma unroll
            for (int j = 0; j < CH; j += 8) {
              float y[8];
#pragma unroll
              for (int q = 0; q < 8; ++q) y[q] = accf[grp * CH + j + q] * route_w;
              stage8((grp ? col1 : col0) + j, y);
            }
          }
        }
        if constexpr (is_dense(MODE)) {
          // (3) hand the staged tile to the store warp and go on with the next tile
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the TMA store
          __syncwarp();
          if (lane == 0) mbar_arrive(cfull_bar);
          ++tiles_done;
        } else if (moe_async_store && tile_stored) {
          // the re-quantised tile has been handed over above
        } else if (moe_async_store) {
          // (3) hand the staged tile and its row offsets to the store warps
          if (half == 0) row_off[r] = row_ok ? static_cast<long long>(out_row) : -1LL;
          __syncwarp();
          if (lane == 0) mbar_arrive(cfull_bar);
          ++tiles_done;
        } else if (!tile_stored) {
          if (half == 0) row_off[r] = row_ok ? static_cast<long long>(out_row) : -1LL;
          if (!epi_sync()) { alive = false; break; }
          // (3) write the tile out
          {
            constexpr int CPR = C::kOutCols / 8;   // 16-byte chunks per output row
            constexpr int RPI = 32 / CPR;          // rows per warp instruction
            const int rows = min(BM, p.tile_m);
            const int ch = lane % CPR;
            const int col = ch * 8;
            if (n0 + col + 8 <= p.N) {
              for (int r0 = ew * RPI; r0 < rows; r0 += kEpiWarps * RPI) {
                const int rr = r0 + lane / CPR;
                if (rr < rows) {
                  const long long off = row_off[rr];
                  if (off >= 0) {
                    const uint32_t addr = cstage_base + (col >> 6) * kRegionBytes + rr * 128 +
                                          ((((col & 63) >> 3) ^ (rr & 7)) << 4);
                    uint4 q;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                                 : "r"(addr)
                                 : "memory");
                    OutT* dst = out + off + n0 + col;
                    if (is_moe2(MODE) && p.accumulate)
                      red8_packed(dst, q);
                    else
                      *reinterpret_cast<uint4*>(dst) = q;
                  }
                }
              }
            }
          }
        }
      } else {
        // direct path (narrow tiles, f32 output): each thread stores its own row segments
        if (row_ok) {
          if constexpr (is_moe1(MODE)) {
#pragma unroll
            for (int j = 0; j < CH; j += 8) {
              if (n0 + col0 + j + 8 <= p.N) {
                float y[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) y[q] = silu_mul(accf[j + q], accf[CH + j + q]) * route_w;
                store8<OutT>(out + out_row + n0 + col0 + j, y);
              }
            }
          } else {
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) {
              const int cb = n0 + (grp ? col1 : col0);
#pragma unroll
              for (int j = 0; j < CH; j += 8) {
                if (cb + j + 8 <= p.N) {
                  float y[8];
#pragma unroll
                  for (int q = 0; q < 8; ++q) y[q] = accf[grp * CH + j + q] * route_w;
                  if (is_moe2(MODE) && p.accumulate)
                    red8<OutT>(out + out_row + cb + j, y);
                  else
                    store8<OutT>(out + out_row + cb + j, y);
                }
              }
            }
          }
        }
      }

      // rotate to the prefetched tile
      if constexpr (is_pt(MODE)) {
        if constexpr (!is_dense(MODE)) cur = nxt;
      } else {
        cur = nxt;
#pragma unroll
        for (int j = 0; j < kRing; ++j) {
          ring_a[j] = nring_a[j];
          ring_b0[j] = nring_b0[j];
          ring_b1[j] = nring_b1[j];
        }
      }
      pos = npos;
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A role gave up: let copies that are still in flight land before the CTA's shared memory and
    // TMEM are handed back.
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ================================= host side =====================================================

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// Row-major 2-D tensor [rows, cols] of elem_bytes-wide elements; box = 128 bytes x box_rows rows;
// 128-byte swizzle; out-of-range parts read as 0 / are not written.
int make_tensor_map_2d(CUtensorMap* map, const void* base, int rows, int cols, int elem_bytes,
                       int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return set_error(FLYB200_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16,
                  2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(FLYB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d",
                     static_cast<int>(r));
  return FLYB200_OK;
}

template <int BN, int MODE, typename OutT>
static int launch(const CUtensorMap& tmap_a, const CUtensorMap& tmap_c, const GemmParams& p,
                  int grid, cudaStream_t stream) {
  using C = Cfg<BN, MODE, OutT>;
  auto kern = bs_gemm_kernel<BN, MODE, OutT>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  FLYB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    FLYB200_CUDA_CHECK(
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  FLYB200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmap_a, tmap_c, p));
  return FLYB200_OK;
}

template <int MODE, typename OutT>
static int launch_bn(int bn, const CUtensorMap& tmap_a, const CUtensorMap& tmap_c,
                     const GemmParams& p, int grid, cudaStream_t stream) {
  switch (bn) {
    case 32:
      if constexpr (is_moe1(MODE)) break;  // 16 gate + 16 up columns: not built
      else return launch<32, MODE, OutT>(tmap_a, tmap_c, p, grid, stream);
    case 64: return launch<64, MODE, OutT>(tmap_a, tmap_c, p, grid, stream);
    case 128: return launch<128, MODE, OutT>(tmap_a, tmap_c, p, grid, stream);
    case 256: return launch<256, MODE, OutT>(tmap_a, tmap_c, p, grid, stream);
    default: break;
  }
  return set_error(FLYB200_ERR_INVALID_ARGUMENT, "block_n must be 32, 64, 128 or 256 (got %d)", bn);
}

static inline int cdiv(int a, int b) { return (a + b - 1) / b; }

// Tile-width heuristic (role of select_tile_config in the reference's test). Cost model per K block
// of one tile, fitted to measurements on B200: the tensor-core side costs a fixed ~360 ns (MMA
// issue, TMEM round trip of the promotion) plus ~0.9 ns per output column; the memory side costs
// the tile's weight bytes at one SM's share of HBM bandwidth when few row blocks share them. The
// persistent loop runs ceil(tiles / SMs) rounds; pick the width with the smallest total.
static int pick_block_n(int m_blocks, int n_cols, int sms, bool moe1) {
  const int cands[4] = {256, 128, 64, 32};
  int best = 128;
  double best_cost = 1e30;
  for (int i = 0; i < 4; ++i) {
    const int bn = cands[i];
    if (moe1 && bn < 64) continue;
    const int cols = moe1 ? bn / 2 : bn;
    const long tiles = static_cast<long>(m_blocks) * cdiv(n_cols, cols);
    const long rounds = (tiles + sms - 1) / sms;
    const double compute_ns = 360.0 + 0.9 * bn;
    // weight tile bytes per K block over ~44 GB/s per SM; row blocks that run concurrently on the
    // same weight tile share one HBM read through L2
    const int sharing = m_blocks < 8 ? (m_blocks < 1 ? 1 : m_blocks) : 8;
    const double memory_ns = (bn * 128.0 / 44.0) / sharing;
    const double per_kb = compute_ns > memory_ns ? compute_ns : memory_ns;
    const double cost = rounds * per_kb;
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

static int check_ptr(const void* p, size_t align, const char* name) {
  if (!p) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "%s is NULL", name);
  if (reinterpret_cast<uintptr_t>(p) % align)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "%s must be %zu-byte aligned", name, align);
  return FLYB200_OK;
}

// decode_gemm.cu
int launch_decode_gemm(void* c, const void* a, const void* b_repacked, const float* scale_a_t,
                       const float* scale_b, int M, int N, int K, int out_dtype, int force_splits,
                       cudaStream_t stream, bool pertoken);
bool decode_path_pays_off(int M, int N, int K);
// pt_pair_gemm.cu
int launch_pertoken_pair_gemm(void* c, const void* a, const void* b_repacked, const float* scale_a,
                              const float* scale_b, int M, int N, int K, int out_dtype, int max_ctas, int group_m,
                              cudaStream_t stream);

}  // namespace flyb200

using namespace flyb200;

// Row blocks per group of the dense tile order (TileWalker::group_m): groups whose slice of A is
// about 24 MB (8..64 row blocks), used when there are at least two such groups. Measured on B200 at
// M = 16384: (N, K) = (4096, 7168) 544 -> 439-449 us with groups of 8-32 (504 with 64), (7168, 2048)
// 255 -> 240 us and (24576, 1536) 680 -> 625 us with 64; at M = 4096 (32 row blocks) smaller groups
// are neutral or slower, and the rule leaves those shapes alone.
static int dense_group_m(int M, int K) {
  int gm = static_cast<int>((static_cast<size_t>(24) << 20) / (static_cast<size_t>(BM) * K));
  gm = gm < 8 ? 8 : (gm > 64 ? 64 : gm);
  return cdiv(M, BM) >= 2 * gm ? gm : 0;
}

extern "C" int flyb200_blockscale_gemm(void* c, const void* a, const void* b_repacked,
                                       const float* scale_a_t, const float* scale_b, int32_t M,
                                       int32_t N, int32_t K, int32_t out_dtype,
                                       const flyb200_gemm_cfg* cfg, void* stream) {
  int rc;
  if ((rc = check_ptr(c, 16, "c")) || (rc = check_ptr(a, 16, "a")) ||
      (rc = check_ptr(b_repacked, 16, "b_repacked")) || (rc = check_ptr(scale_a_t, 4, "scale_a_t")) ||
      (rc = check_ptr(scale_b, 4, "scale_b")))
    return rc;
  if (M < 1 || N < 16 || K < 128)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "bad shape M=%d N=%d K=%d", M, N, K);
  if (N % 16) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "N (%d) must be a multiple of 16", N);
  if (K % 128) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "K (%d) must be a multiple of 128", K);
  if (out_dtype != FLYB200_BF16 && out_dtype != FLYB200_F16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "out_dtype must be BF16 or F16");

  // Decode-size M: the swap-AB split-K kernel (decode_gemm.cu), unless a tile width or the tiled
  // path was asked for explicitly.
  const int path = cfg ? cfg->path : 0;
  if (path < 0 || path > 2)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "cfg.path must be 0 (auto), 1 (tiled) or 2 (decode)");
  if (path == 2 && M > 64)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "the decode path takes M <= 64 (got %d)", M);
  if (path == 2 || (path == 0 && M <= 64 && !(cfg && cfg->block_n) && decode_path_pays_off(M, N, K)))
    return launch_decode_gemm(c, a, b_repacked, scale_a_t, scale_b, M, N, K, out_dtype,
                              cfg ? cfg->split_k : 0, reinterpret_cast<cudaStream_t>(stream), false);

  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const int m_blocks = cdiv(M, BM);
  int bn = (cfg && cfg->block_n) ? cfg->block_n : pick_block_n(m_blocks, N, sms, false);
  int grid = sms;
  if (cfg && cfg->max_ctas > 0 && cfg->max_ctas < grid) grid = cfg->max_ctas;
  const long tiles = static_cast<long>(m_blocks) * cdiv(N, bn);
  if (tiles < grid) grid = static_cast<int>(tiles);

  GemmParams p{};
  p.a = reinterpret_cast<const uint8_t*>(a);
  p.b = reinterpret_cast<const uint8_t*>(b_repacked);
  p.scale_a = scale_a_t;
  p.scale_b = scale_b;
  p.out = c;
  p.err = device_error_word();
  if (!p.err) return FLYB200_ERR_CUDA;
  p.M = M; p.N = N; p.K = K;
  p.group_m = dense_group_m(M, K);
  // Small M: bring only as many rows as exist (rounded up to the 8-row swizzle atom).
  p.a_box_rows = M >= BM ? BM : ((M + 7) / 8) * 8;

  CUtensorMap tmap_a, tmap_c;
  if ((rc = make_tensor_map_2d(&tmap_a, a, M, K, 1, p.a_box_rows))) return rc;
  if ((rc = make_tensor_map_2d(&tmap_c, c, M, N, 2, p.a_box_rows))) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (out_dtype == FLYB200_BF16)
    return launch_bn<kDense, __nv_bfloat16>(bn, tmap_a, tmap_c, p, grid, st);
  return launch_bn<kDense, __half>(bn, tmap_a, tmap_c, p, grid, st);
}

extern "C" int flyb200_pertoken_gemm(void* c, const void* a, const void* b_repacked, const float* scale_a,
                                     const float* scale_b, int32_t M, int32_t N, int32_t K,
                                     int32_t out_dtype, const flyb200_gemm_cfg* cfg, void* stream) {
  int rc;
  if ((rc = check_ptr(c, 16, "c")) || (rc = check_ptr(a, 16, "a")) ||
      (rc = check_ptr(b_repacked, 16, "b_repacked")) || (rc = check_ptr(scale_a, 4, "scale_a")) ||
      (rc = check_ptr(scale_b, 4, "scale_b")))
    return rc;
  if (M < 1 || N < 16 || K < 128)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "bad shape M=%d N=%d K=%d", M, N, K);
  if (N % 16) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "N (%d) must be a multiple of 16", N);
  if (K % 128) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "K (%d) must be a multiple of 128", K);
  if (out_dtype != FLYB200_BF16 && out_dtype != FLYB200_F16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "out_dtype must be BF16 or F16");
  if (cfg && cfg->block_n && cfg->block_n != 256)
    return set_error(FLYB200_ERR_UNSUPPORTED, "the per-token-scale GEMM is built with 256-wide tiles only");
  // Decode-size M: the swap-AB split-K kernel with the token's scale on every K block and the
  // channel's scale applied once (cfg.path as for flyb200_blockscale_gemm).
  const int path = cfg ? cfg->path : 0;
  if (path < 0 || path > 3)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "cfg.path must be 0 (auto), 1 (tiled), 2 (decode) or 3 (CTA pairs)");
  if (path == 2 && M > 64)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "the decode path takes M <= 64 (got %d)", M);
  if (path == 2 || (path == 0 && M <= 64 && !(cfg && cfg->block_n) && decode_path_pays_off(M, N, K)))
    return launch_decode_gemm(c, a, b_repacked, scale_a, scale_b, M, N, K, out_dtype,
                              cfg ? cfg->split_k : 0, reinterpret_cast<cudaStream_t>(stream), true);
  // Large problems: the CTA-pair kernel (256 x 256 tiles over two SMs, 32 KB stages), measured faster
  // than the single-CTA tiles on every benchmarked shape from M = 1024 up (equal at 256-512).
  if (path == 3 && (M < 256 || N % 256))
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "the CTA-pair path takes M >= 256 and N %% 256 == 0");
  if (path == 3 || (path == 0 && M >= 1024 && N % 256 == 0 && !(cfg && cfg->block_n))) {
    return launch_pertoken_pair_gemm(c, a, b_repacked, scale_a, scale_b, M, N, K, out_dtype,
                                     cfg ? cfg->max_ctas : 0, dense_group_m(M, K),
                                     reinterpret_cast<cudaStream_t>(stream));
  }
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const int m_blocks = cdiv(M, BM);
  int grid = sms;
  if (cfg && cfg->max_ctas > 0 && cfg->max_ctas < grid) grid = cfg->max_ctas;
  const long tiles = static_cast<long>(m_blocks) * cdiv(N, 256);
  if (tiles < grid) grid = static_cast<int>(tiles);

  GemmParams p{};
  p.a = reinterpret_cast<const uint8_t*>(a);
  p.b = reinterpret_cast<const uint8_t*>(b_repacked);
  p.scale_a = scale_a;   // [M]
  p.scale_b = scale_b;   // [N]
  p.out = c;
  p.err = device_error_word();
  if (!p.err) return FLYB200_ERR_CUDA;
  p.M = M; p.N = N; p.K = K;
  p.group_m = dense_group_m(M, K);
  p.a_box_rows = M >= BM ? BM : ((M + 7) / 8) * 8;
  CUtensorMap tmap_a, tmap_c;
  if ((rc = make_tensor_map_2d(&tmap_a, a, M, K, 1, p.a_box_rows))) return rc;
  if ((rc = make_tensor_map_2d(&tmap_c, c, M, N, 2, p.a_box_rows))) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (out_dtype == FLYB200_BF16) return launch<256, kDensePT, __nv_bfloat16>(tmap_a, tmap_c, p, grid, st);
  return launch<256, kDensePT, __half>(tmap_a, tmap_c, p, grid, st);
}

static int moe_common_checks(const void* out, const void* x, const void* w, const float* scale_x,
                             const float* scale_w, const int32_t* sorted_ids,
                             const int32_t* expert_ids, const float* sorted_weights,
                             const int32_t* num_valid_ids, int T, int n, int kdim, int num_blocks,
                             int E, int k, int tile_m, int doweight) {
  int rc;
  if ((rc = check_ptr(out, 16, "out")) || (rc = check_ptr(x, 16, "x")) ||
      (rc = check_ptr(w, 16, "w")) || (rc = check_ptr(scale_x, 4, "scale_x")) ||
      (rc = check_ptr(scale_w, 4, "scale_w")) || (rc = check_ptr(sorted_ids, 4, "sorted_ids")) ||
      (rc = check_ptr(expert_ids, 4, "expert_ids")) ||
      (rc = check_ptr(num_valid_ids, 4, "num_valid_ids")))
    return rc;
  if (doweight && (rc = check_ptr(sorted_weights, 4, "sorted_weights"))) return rc;
  if (T < 1 || T >= (1 << 24) || E < 1 || k < 1 || k > 255 || k > E || num_blocks < 0)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "bad MoE sizes T=%d E=%d k=%d blocks=%d (k <= E)", T, E, k,
                     num_blocks);
  if (tile_m < 1 || tile_m > BM)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "tile_m (%d) must be in [1,128]", tile_m);
  if (n % 128 || kdim % 128 || n < 128 || kdim < 128)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "MoE dims must be multiples of 128 (n=%d, k=%d)", n, kdim);
  return FLYB200_OK;
}

// cfg.path of the MoE entry points is a bit set: bit 0 = the activation argument is already in
// routing order ([T*k + E*tile_m - k, K] rows, scales [K/128, same rows]) and is fetched by TMA;
// bit 1 (stage 1 only) = write the output in routing order too.
static int moe_sorted_layout(const flyb200_gemm_cfg* cfg, int T, int E, int k, int tile_m, int kdim,
                             const void* act, GemmParams* p, CUtensorMap* tmap) {
  const int bits = cfg ? cfg->path : 0;
  if (bits < 0 || bits > 3)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "MoE cfg.path must be a combination of bits 0 and 1");
  p->a_sorted = bits & 1;
  p->out_sorted = (bits >> 1) & 1;
  const long long rows = static_cast<long long>(T) * k + static_cast<long long>(E) * tile_m - k;
  if (rows <= 0 || rows > 0x7fffffffLL)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "T*k + E*tile_m - k = %lld rows is out of range", rows);
  p->a_rows = static_cast<int>(rows);
  if (!p->a_sorted) return FLYB200_OK;
  if (tile_m % 8)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "sorted activations need tile_m to be a multiple of 8 (got %d)", tile_m);
  p->a_box_rows = tile_m;
  return make_tensor_map_2d(tmap, act, p->a_rows, kdim, 1, tile_m);
}

static int moe_gemm1_impl(void* out, void* out_q, float* out_scale_t, const void* x, const void* w_repacked,
                          const float* scale_x, const float* scale_w, const int32_t* sorted_ids,
                          const int32_t* expert_ids, const float* sorted_weights,
                          const int32_t* num_valid_ids, int32_t T, int32_t I, int32_t H,
                          int32_t num_blocks, int32_t E, int32_t k, int32_t tile_m, int32_t doweight,
                          int32_t out_dtype, const flyb200_gemm_cfg* cfg, void* stream,
                          bool pertoken = false) {
  int rc = moe_common_checks(out_q ? out_q : out, x, w_repacked, scale_x, scale_w, sorted_ids, expert_ids,
                             sorted_weights, num_valid_ids, T, I, H, num_blocks, E, k, tile_m,
                             doweight);
  if (rc) return rc;
  if (out_dtype != FLYB200_BF16 && out_dtype != FLYB200_F16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "stage-1 out_dtype must be BF16 or F16");
  if (pertoken && cfg && cfg->block_n && cfg->block_n != 256)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "the per-token MoE kernels are built for block_n 256");
  if (num_blocks == 0) return FLYB200_OK;
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  int bn = (cfg && cfg->block_n) ? cfg->block_n : pick_block_n(num_blocks, I, sms, true);
  if (bn < 64) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "stage-1 block_n must be >= 64");
  if (pertoken) bn = 256;
  if (out_q) {
    if (cfg && cfg->block_n && cfg->block_n != 256)
      return set_error(FLYB200_ERR_INVALID_ARGUMENT, "fused re-quantisation needs block_n 256");
    bn = 256;   // 128 output columns per tile = one 1x128 scale group per row
    if (!cfg || (cfg->path & 3) != 3)
      return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                       "fused re-quantisation needs routing-order input and output (cfg.path bits 0 and 1)");
    if (I % 128) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "fused re-quantisation needs I %% 128 == 0");
    if (reinterpret_cast<uintptr_t>(out_q) % 16 || !out_scale_t)
      return set_error(FLYB200_ERR_INVALID_ARGUMENT, "out_q must be 16-byte aligned, out_scale_t non-NULL");
  }
  int grid = sms;
  if (cfg && cfg->max_ctas > 0 && cfg->max_ctas < grid) grid = cfg->max_ctas;
  const long tiles = static_cast<long>(num_blocks) * cdiv(I, bn / 2);
  if (tiles < grid) grid = static_cast<int>(tiles);

  GemmParams p{};
  p.a = reinterpret_cast<const uint8_t*>(x);
  p.b = reinterpret_cast<const uint8_t*>(w_repacked);
  p.scale_a = scale_x; p.scale_b = scale_w; p.out = out;
  p.out_q = static_cast<uint8_t*>(out_q); p.out_scale_t = out_scale_t;
  p.err = device_error_word();
  if (!p.err) return FLYB200_ERR_CUDA;
  p.M = T; p.N = I; p.K = H; p.a_box_rows = 0;
  p.sorted_ids = sorted_ids; p.expert_ids = expert_ids; p.sorted_weights = sorted_weights;
  p.num_valid = num_valid_ids; p.topk = k; p.tile_m = tile_m; p.num_blocks = num_blocks;
  p.experts = E; p.doweight = doweight; p.accumulate = 0;
  CUtensorMap tmap{};
  if ((rc = moe_sorted_layout(cfg, T, E, k, tile_m, H, x, &p, &tmap))) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (pertoken) {
    if (out_dtype == FLYB200_BF16) return launch<256, kMoe1PT, __nv_bfloat16>(tmap, tmap, p, grid, st);
    return launch<256, kMoe1PT, __half>(tmap, tmap, p, grid, st);
  }
  if (out_dtype == FLYB200_BF16)
    return launch_bn<kMoe1, __nv_bfloat16>(bn, tmap, tmap, p, grid, st);
  return launch_bn<kMoe1, __half>(bn, tmap, tmap, p, grid, st);
}

extern "C" int flyb200_moe_gemm1(void* out, const void* x, const void* w_repacked,
                                 const float* scale_x, const float* scale_w,
                                 const int32_t* sorted_ids, const int32_t* expert_ids,
                                 const float* sorted_weights, const int32_t* num_valid_ids,
                                 int32_t T, int32_t I, int32_t H, int32_t num_blocks, int32_t E,
                                 int32_t k, int32_t tile_m, int32_t doweight, int32_t out_dtype,
                                 const flyb200_gemm_cfg* cfg, void* stream) {
  return moe_gemm1_impl(out, nullptr, nullptr, x, w_repacked, scale_x, scale_w, sorted_ids, expert_ids,
                        sorted_weights, num_valid_ids, T, I, H, num_blocks, E, k, tile_m, doweight,
                        out_dtype, cfg, stream);
}

extern "C" int flyb200_moe_gemm1_q8(void* out_q, float* out_scale_t, const void* x, const void* w_repacked,
                                    const float* scale_x, const float* scale_w,
                                    const int32_t* sorted_ids, const int32_t* expert_ids,
                                    const float* sorted_weights, const int32_t* num_valid_ids,
                                    int32_t T, int32_t I, int32_t H, int32_t num_blocks, int32_t E,
                                    int32_t k, int32_t tile_m, int32_t doweight, int32_t mid_dtype,
                                    const flyb200_gemm_cfg* cfg, void* stream) {
  if (!out_q || !out_scale_t) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "gemm1_q8: NULL output");
  return moe_gemm1_impl(nullptr, out_q, out_scale_t, x, w_repacked, scale_x, scale_w, sorted_ids, expert_ids,
                        sorted_weights, num_valid_ids, T, I, H, num_blocks, E, k, tile_m, doweight,
                        mid_dtype, cfg, stream);
}

static int moe_gemm2_impl(void* out, const void* a2, const void* w_repacked,
                          const float* scale_x, const float* scale_w,
                          const int32_t* sorted_ids, const int32_t* expert_ids,
                          const float* sorted_weights, const int32_t* num_valid_ids,
                          int32_t T, int32_t H, int32_t I, int32_t num_blocks, int32_t E,
                          int32_t k, int32_t tile_m, int32_t doweight, int32_t accumulate,
                          int32_t out_dtype, const flyb200_gemm_cfg* cfg, void* stream, bool pertoken) {
  int rc = moe_common_checks(out, a2, w_repacked, scale_x, scale_w, sorted_ids, expert_ids,
                             sorted_weights, num_valid_ids, T, H, I, num_blocks, E, k, tile_m,
                             doweight);
  if (rc) return rc;
  if (out_dtype != FLYB200_BF16 && out_dtype != FLYB200_F16 && out_dtype != FLYB200_F32)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "stage-2 out_dtype must be BF16, F16 or F32");
  if (pertoken && cfg && cfg->block_n && cfg->block_n != 256)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "the per-token MoE kernels are built for block_n 256");
  if (num_blocks == 0) return FLYB200_OK;
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  int bn = (cfg && cfg->block_n) ? cfg->block_n : pick_block_n(num_blocks, H, sms, false);
  if (pertoken) bn = 256;
  int grid = sms;
  if (cfg && cfg->max_ctas > 0 && cfg->max_ctas < grid) grid = cfg->max_ctas;
  const long tiles = static_cast<long>(num_blocks) * cdiv(H, bn);
  if (tiles < grid) grid = static_cast<int>(tiles);

  GemmParams p{};
  p.a = reinterpret_cast<const uint8_t*>(a2);
  p.b = reinterpret_cast<const uint8_t*>(w_repacked);
  p.scale_a = scale_x; p.scale_b = scale_w; p.out = out;
  p.err = device_error_word();
  if (!p.err) return FLYB200_ERR_CUDA;
  p.M = T; p.N = H; p.K = I; p.a_box_rows = 0;
  p.sorted_ids = sorted_ids; p.expert_ids = expert_ids; p.sorted_weights = sorted_weights;
  p.num_valid = num_valid_ids; p.topk = k; p.tile_m = tile_m; p.num_blocks = num_blocks;
  p.experts = E; p.doweight = doweight; p.accumulate = accumulate ? 1 : 0;
  CUtensorMap tmap{};
  if ((rc = moe_sorted_layout(cfg, T, E, k, tile_m, I, a2, &p, &tmap))) return rc;
  if (p.out_sorted)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "stage 2 has no sorted output layout (cfg.path bit 1)");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (pertoken) {
    if (out_dtype == FLYB200_BF16) return launch<256, kMoe2PT, __nv_bfloat16>(tmap, tmap, p, grid, st);
    if (out_dtype == FLYB200_F16) return launch<256, kMoe2PT, __half>(tmap, tmap, p, grid, st);
    return launch<256, kMoe2PT, float>(tmap, tmap, p, grid, st);
  }
  if (out_dtype == FLYB200_BF16)
    return launch_bn<kMoe2, __nv_bfloat16>(bn, tmap, tmap, p, grid, st);
  if (out_dtype == FLYB200_F16) return launch_bn<kMoe2, __half>(bn, tmap, tmap, p, grid, st);
  return launch_bn<kMoe2, float>(bn, tmap, tmap, p, grid, st);
}

extern "C" int flyb200_moe_gemm2(void* out, const void* a2, const void* w_repacked,
                                 const float* scale_x, const float* scale_w,
                                 const int32_t* sorted_ids, const int32_t* expert_ids,
                                 const float* sorted_weights, const int32_t* num_valid_ids,
                                 int32_t T, int32_t H, int32_t I, int32_t num_blocks, int32_t E,
                                 int32_t k, int32_t tile_m, int32_t doweight, int32_t accumulate,
                                 int32_t out_dtype, const flyb200_gemm_cfg* cfg, void* stream) {
  return moe_gemm2_impl(out, a2, w_repacked, scale_x, scale_w, sorted_ids, expert_ids, sorted_weights,
                        num_valid_ids, T, H, I, num_blocks, E, k, tile_m, doweight, accumulate, out_dtype,
                        cfg, stream, false);
}

// The per-token-scale siblings: scale_x [rows] (one per activation row: token for stage 1,
// token*topk+slot -- or the sorted row with cfg.path bit 0 -- for stage 2), scale_w one per output
// channel of every expert ([E*2I] / [E*H]). Everything else as in the block-scale entry points.
extern "C" int flyb200_moe_gemm1_pertoken(void* out, const void* x, const void* w_repacked,
                                          const float* scale_x, const float* scale_w,
                                          const int32_t* sorted_ids, const int32_t* expert_ids,
                                          const float* sorted_weights, const int32_t* num_valid_ids,
                                          int32_t T, int32_t I, int32_t H, int32_t num_blocks, int32_t E,
                                          int32_t k, int32_t tile_m, int32_t doweight, int32_t out_dtype,
                                          const flyb200_gemm_cfg* cfg, void* stream) {
  return moe_gemm1_impl(out, nullptr, nullptr, x, w_repacked, scale_x, scale_w, sorted_ids, expert_ids,
                        sorted_weights, num_valid_ids, T, I, H, num_blocks, E, k, tile_m, doweight,
                        out_dtype, cfg, stream, true);
}

extern "C" int flyb200_moe_gemm2_pertoken(void* out, const void* a2, const void* w_repacked,
                                          const float* scale_x, const float* scale_w,
                                          const int32_t* sorted_ids, const int32_t* expert_ids,
                                          const float* sorted_weights, const int32_t* num_valid_ids,
                                          int32_t T, int32_t H, int32_t I, int32_t num_blocks, int32_t E,
                                          int32_t k, int32_t tile_m, int32_t doweight, int32_t accumulate,
                                          int32_t out_dtype, const flyb200_gemm_cfg* cfg, void* stream) {
  return moe_gemm2_impl(out, a2, w_repacked, scale_x, scale_w, sorted_ids, expert_ids, sorted_weights,
                        num_valid_ids, T, H, I, num_blocks, E, k, tile_m, doweight, accumulate, out_dtype,
                        cfg, stream, true);
}
