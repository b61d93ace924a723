// Dense FP8 block-scale GEMM for decode-size M (<= 64 tokens): HBM-bound, so the kernel is built
// around streaming the weights once at full bandwidth.
//
//   * swap-AB: the 128-row weight tile is the MMA "A" operand (128 accumulator lanes = output
//     columns n), the tokens are the MMA "B" operand (NT = 16/32/64 accumulator columns). One
//     tcgen05.mma 128 x NT x 32 consumes 4 KB of weights, half as many instructions per weight byte
//     as a 64-wide weight tile would need.
//   * split-K over a thread-block cluster: CTA (n_tile, split) streams K blocks [split*kbps, ...)
//     of its weight tile; fp32 partial sums travel through distributed shared memory (one bulk
//     copy per destination, counted on the destination's mbarrier) to the CTA that owns a slice of
//     the token columns, which adds them in rank order and stores. No global workspace, no atomics,
//     deterministic.
//   * each CTA issues its whole K range of bulk copies at once when it fits the ring (<= 8 stages),
//     so the HBM queue is full from the first microsecond.
//   * launched with programmatic stream serialisation: setup (barriers, TMEM) and the first ring fill
//     of WEIGHT tiles overlap the tail of the previous kernel in the stream; griddepcontrol.wait
//     precedes every access to activations, scales and the output.
//
// Same arithmetic contract as the main kernel (blockscale_gemm.cu): per 128-K block the exact fp8
// products are summed in fp32 by the tensor core, then acc += partial * (sa[kb,m] * sb[n/128,kb]).
// Reference: kernels/blockscale_preshuffle_gemm.py:161-839 (small-M tiles of its select_tile_config).
#include "common.cuh"
#include "cluster.cuh"

namespace flyb200 {

constexpr int kDecThreads = 192;    // warp 0 producer, warp 1 MMA, warps 2-5 epilogue
constexpr int kDecMaxStages = 8;
constexpr int kWTileBytes = 128 * 128;

struct DecodeParams {
  const uint8_t* b;        // repacked weights [K/128][N/8][8][128]
  const float* scale_a;    // [K/128, M]
  const float* scale_b;    // [ceil(N/128), K/128]
  void* out;               // [M, N]
  int* err;
  int M, N, K;
  int splits;              // cluster size along x
  int kbps;                // K blocks per split
  int stages;              // ring depth used (<= kDecMaxStages)
  int pertoken;            // scales are per token [M] and per output channel [N] (no K dimension)
};

template <int NT>
struct DecCfg {
  static constexpr int kXTileBytes = NT * 128;
  static constexpr int kStageBytes = kWTileBytes + kXTileBytes;
  // Four accumulator buffers (64-256 TMEM columns): with the small shared-memory footprint below,
  // three or four CTAs fit an SM, so the CTAs of the NEXT launch (programmatic dependent launch) are
  // resident and streaming their weights while this launch exchanges, reduces and stores.
  static constexpr int kAccBufs = (256 / NT) > 4 ? 4 : (256 / NT);
  static constexpr int kTmemCols = NT * kAccBufs < 32 ? 32 : NT * kAccBufs;
  // fp32 partial sums received from the cluster: [sender][local column][128]; sender count x
  // columns per owner can exceed NT by up to splits-1 because of rounding
  static constexpr int kPartialBytes = (NT + 8) * 128 * 4;
  // The pipeline ring doubles as send buffer ([0, NT) token rows) and receive area (behind it) of
  // the split-K exchange: every MMA of the whole cluster has completed before the first copy.
  static constexpr int kExchangeBytes = NT * 512 + kPartialBytes;
  __host__ __device__ static int ring_bytes(int stages) {
    const int r = stages * kStageBytes;
    return r > kExchangeBytes ? r : kExchangeBytes;
  }
  static constexpr int kScaleBytes = kDecMaxStages * 2 * (NT + 1) * 4 + 64;  // generous
  static constexpr int kMiscBytes = 1024;
  static int smem_bytes(int stages, int kbps) {
    return ring_bytes(stages) + (kbps * (NT + 1) * 4 + 64) + kMiscBytes + 1024;
  }
};

template <int NT, typename OutT>
__global__ void __launch_bounds__(kDecThreads)
bs_gemm_decode_kernel(const __grid_constant__ CUtensorMap tmap_x, const DecodeParams p) {
  using C = DecCfg<NT>;
  constexpr int kAccBufs = C::kAccBufs;
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int kDone = stages + kAccBufs;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const int ring_bytes = C::ring_bytes(stages);
  const uint32_t recv_base = smem_base + NT * 512;                  // fp32 [sender][column][128], in the ring
  float* recv = reinterpret_cast<float*>(smem_al + NT * 512);
  float* sa_s = reinterpret_cast<float*>(smem_al + ring_bytes);     // [kbps][NT]
  float* sb_s = sa_s + p.kbps * NT;                                            // [kbps]
  const uint32_t misc_off = static_cast<uint32_t>(ring_bytes) + ((p.kbps * (NT + 1) * 4 + 63) & ~63);
  const uint32_t bar_base = smem_base + misc_off;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto done_bar = [&](uint32_t i) { return bar_base + 8u * (kDecMaxStages + i); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kDecMaxStages + 8 + b); };
  const uint32_t recv_bar = bar_base + 8u * (2 * kDecMaxStages + 16);
  volatile uint32_t* tmem_slot =
      reinterpret_cast<volatile uint32_t*>(smem_al + misc_off + 8 * (2 * kDecMaxStages + 17));
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem_al + misc_off + 8 * (2 * kDecMaxStages + 17) + 4);

  const int split = static_cast<int>(cluster_ctarank());
  const int n_tile = blockIdx.x / p.splits;
  const int n0 = n_tile * 128;
  const int KBt = p.K / 128;
  const int kb_begin = split * p.kbps;
  const int kb_end = min(KBt, kb_begin + p.kbps);
  const int count = max(0, kb_end - kb_begin);
  const int rows_w = min(128, p.N - n0);

  if (warp == 0) {  // one barrier per lane: the inits run in parallel
    if (lane < stages) mbar_init(full_bar(lane), 1);
    if (lane < kDone) mbar_init(done_bar(lane), 1);
    if (lane < kAccBufs) mbar_init(tempty_bar(lane), 4);  // one arrival per epilogue warp
    if (lane == 0) {
      mbar_init(recv_bar, 1);
      *abort_flag = 0;
      prefetch_tensormap(&tmap_x);
    }
    fence_proxy_async_smem();
    fence_barrier_init();
    if (lane == 0) {
      // bytes this CTA will receive for its column slice: one slice from each CTA of the cluster
      const int cpc = (p.M + p.splits - 1) / p.splits;
      const int own = min(p.M, (split + 1) * cpc) - split * cpc;
      if (own > 0) mbar_arrive_expect_tx(recv_bar, static_cast<uint32_t>(own * p.splits) * 512u);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The receive barriers of the whole cluster exist before anybody may signal them.
  cluster_sync_all();

  // Everything above touched no global memory: it may overlap the previous kernel of the stream.
  // The WEIGHT tiles of the first ring fill are requested before the dependency wait as well:
  // weights are parameters, not results of the kernel that runs just before (a kernel that lets its
  // dependents start early -- the GEMM and MoE kernels of this library -- never writes weights, and
  // any other kernel has exited before this one starts), so back-to-back launches stream weights
  // without a gap. Activations, scales and the output are touched only after the wait.
  const int first_fill = count < stages ? count : stages;
  if (warp == 0 && lane == 0) {
    for (int i = 0; i < first_fill; ++i) {
      const uint32_t sw = smem_base + i * C::kStageBytes;
      mbar_arrive_expect_tx(full_bar(i), rows_w * 128 + C::kXTileBytes);
      bulk_load(sw, p.b + (static_cast<size_t>(kb_begin + i) * p.N + n0) * 128, rows_w * 128, full_bar(i));
    }
    // the weight tiles beyond the ring go to L2 now, so that their loads (issued when a stage frees
    // up, after the wait) do not pay an HBM latency each: 2.3 -> 0.9 us for the fourth K block of a
    // three-stage ring in a trace of back-to-back launches
    for (int i = first_fill; i < count; ++i)
      l2_prefetch(p.b + (static_cast<size_t>(kb_begin + i) * p.N + n0) * 128, rows_w * 128);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer ----------------
      for (int i = 0; i < first_fill; ++i)   // activation tiles of the stages whose weights are on their way
        tma_load_2d(smem_base + i * C::kStageBytes + kWTileBytes, &tmap_x, (kb_begin + i) * 128, 0, full_bar(i));
      for (int i = first_fill; i < count; ++i) {
        const int s = i % stages;
        const uint32_t j = i - stages;
        if (!mbar_wait(done_bar(j % kDone), (j / kDone) & 1, abort_flag, p.err, kErrWaitSmemEmpty))
          break;
        const int kb = kb_begin + i;
        const uint32_t sw = smem_base + s * C::kStageBytes;
        mbar_arrive_expect_tx(full_bar(s), rows_w * 128 + C::kXTileBytes);
        bulk_load(sw, p.b + (static_cast<size_t>(kb) * p.N + n0) * 128, rows_w * 128, full_bar(s));
        tma_load_2d(sw + kWTileBytes, &tmap_x, kb * 128, 0, full_bar(s));
      }
    }
    __syncwarp();
    cluster_sync_all();   // (exchange barrier, see the epilogue)
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(128, NT);
      for (int i = 0; i < count; ++i) {
        const int s = i % stages;
        const int buf = i % kAccBufs;
        if (!mbar_wait(tempty_bar(buf), ((i / kAccBufs) & 1) ^ 1, abort_flag, p.err,
                       kErrWaitTmemEmpty) ||
            !mbar_wait(full_bar(s), (i / stages) & 1, abort_flag, p.err, kErrWaitSmemFull))
          break;
        tc_fence_after();
        const uint32_t sw = smem_base + s * C::kStageBytes;
        const uint64_t wdesc = umma_desc_sw128(sw);
        const uint64_t xdesc = umma_desc_sw128(sw + kWTileBytes);
        const uint32_t d = tmem_base + buf * NT;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tc_mma_f8(d, wdesc + 2 * k, xdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
        tc_commit(done_bar(i % kDone));
      }
    }
    __syncwarp();
    cluster_sync_all();   // (exchange barrier, see the epilogue)
  } else {
    // ---------------- epilogue: 128 threads, thread = output column n (accumulator lane) ----------
    const int et = threadIdx.x - 64;            // 0..127
    const int quad = warp & 3;                  // TMEM lane quadrant of this warp
    const int n_loc = quad * 32 + lane;         // weight row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    // scales of this CTA's K range -> shared memory (sa: per token, sb: one per K block)
    for (int idx = et; idx < count * NT; idx += 128) {
      const int kbl = idx / NT, j = idx - kbl * NT;
      const size_t src = p.pertoken ? static_cast<size_t>(j) : static_cast<size_t>(kb_begin + kbl) * p.M + j;
      sa_s[idx] = (j < p.M) ? __ldg(p.scale_a + src) : 0.f;
    }
    // per-token mode: the token's scale rides along every K block, the channel's scale is applied
    // once after the K loop
    for (int kbl = et; kbl < count; kbl += 128)
      sb_s[kbl] = p.pertoken ? 1.f : __ldg(p.scale_b + static_cast<size_t>(n_tile) * KBt + kb_begin + kbl);
    asm volatile("bar.sync 1, 128;" ::: "memory");

    float acc[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j] = 0.f;
    bool alive = true;
    for (int i = 0; i < count && alive; ++i) {
      const int buf = i % kAccBufs;
      const bool got = mbar_wait(done_bar(i % kDone), (i / kDone) & 1, abort_flag, p.err,
                                 kErrWaitTmemFull);
      if (!__all_sync(0xffffffffu, got)) {
        alive = false;
        break;
      }
      tc_fence_after();
      uint32_t v[NT];
      const uint32_t t0 = tmem_base + lane_base + buf * NT;
      if constexpr (NT == 64) {
        tmem_ld<32>(t0, v);
        tmem_ld<32>(t0 + 32, v + 32);
        tmem_wait_dep<32>(v);
        tmem_wait_dep<32>(v + 32);
      } else {
        tmem_ld<NT>(t0, v);
        tmem_wait_dep<NT>(v);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
      const float sb = sb_s[i];
      const float4* sa4 = reinterpret_cast<const float4*>(sa_s + i * NT);
#pragma unroll
      for (int j4 = 0; j4 < NT / 4; ++j4) {
        const float4 s = sa4[j4];  // same address in every lane: broadcast
        acc[4 * j4 + 0] = fmaf(__uint_as_float(v[4 * j4 + 0]), s.x * sb, acc[4 * j4 + 0]);
        acc[4 * j4 + 1] = fmaf(__uint_as_float(v[4 * j4 + 1]), s.y * sb, acc[4 * j4 + 1]);
        acc[4 * j4 + 2] = fmaf(__uint_as_float(v[4 * j4 + 2]), s.z * sb, acc[4 * j4 + 2]);
        acc[4 * j4 + 3] = fmaf(__uint_as_float(v[4 * j4 + 3]), s.w * sb, acc[4 * j4 + 3]);
      }
    }
    // Split-K exchange. The token columns are dealt out to the CTAs of the cluster (owner of
    // column j = j / cpc). Partials go to this CTA's own shared memory as [j][n] (the pipeline
    // stages are free by now: every MMA of this CTA has completed), then one bulk copy per owner
    // moves that owner's column slice into its receive area, slot [sender][local column][n].
    // Exchange barrier: the send and receive areas live in the pipeline ring, so no copy may start
    // before every CTA of the cluster has consumed its last stage (the epilogue has seen the commit
    // of its last K block by now; the other warps arrive as soon as they have issued their work).
    // The send area is this CTA's own (only its finished MMAs read it), so it is written between
    // the arrival and the wait.
    if (p.pertoken) {
      const int n = n_tile * 128 + n_loc;
      const float sbn = n < p.N ? __ldg(p.scale_b + n) : 0.f;
#pragma unroll
      for (int j = 0; j < NT; ++j) acc[j] *= sbn;
    }
    __syncwarp();
    cluster_arrive();
    float* send = reinterpret_cast<float*>(smem_al);
#pragma unroll
    for (int j = 0; j < NT; ++j)
      if (j < p.M) send[j * 128 + n_loc] = acc[j];
    cluster_wait();
    fence_proxy_async_smem();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int cpc = (p.M + p.splits - 1) / p.splits;
    if (et == 0 && alive) {
      for (int o = 0; o < p.splits; ++o) {
        const int lo = o * cpc;
        const int cols = min(p.M, lo + cpc) - lo;
        if (cols > 0)
          bulk_copy_to_cta(map_to_cta(recv_base + static_cast<uint32_t>(split * cpc) * 512u, o),
                           smem_base + static_cast<uint32_t>(lo) * 512u,
                           static_cast<uint32_t>(cols) * 512u, map_to_cta(recv_bar, o));
      }
    }
    // this CTA's slice: wait for every sender's copy, add in rank order, store
    const int j_lo = split * cpc;
    const int j_hi = min(p.M, j_lo + cpc);
    if (j_hi > j_lo && alive) {
      const bool got = mbar_wait(recv_bar, 0, abort_flag, p.err, kErrWaitExchange);
      if (__all_sync(0xffffffffu, got)) {
        OutT* const out = reinterpret_cast<OutT*>(p.out);
        // eight columns at a time so that their shared-memory loads are in flight together
        for (int jb = j_lo; jb < j_hi; jb += 8) {
          float sum[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) sum[u] = 0.f;
          for (int c = 0; c < p.splits; ++c) {  // fixed rank order: deterministic
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (jb + u < j_hi) sum[u] += recv[(c * cpc + (jb - j_lo) + u) * 128 + n_loc];
          }
          if (n0 + n_loc < p.N) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              if (jb + u < j_hi) {
                const size_t o = static_cast<size_t>(jb + u) * p.N + n0 + n_loc;
                if constexpr (sizeof(OutT) == 2) {
                  const uint32_t pk = pack2(sum[u], 0.f, OutT());  // one rounding from the fp32 sum
                  reinterpret_cast<unsigned short*>(out)[o] = static_cast<unsigned short>(pk & 0xFFFFu);
                } else {
                  out[o] = sum[u];
                }
              }
            }
          }
        }
      }
    }
  }
  // Nobody leaves before every bulk copy that reads its shared memory has been consumed: the owners
  // arrive here only after their receive barrier completed.
  __syncwarp();
  cluster_sync_all();

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------- host ----------------------------------------------------------
int make_tensor_map_2d(CUtensorMap* map, const void* base, int rows, int cols, int elem_bytes,
                       int box_rows);  // blockscale_gemm.cu

struct DecodePlan {
  int nt, splits, kbps, stages, ctas_per_sm;
  long rounds;  // waves of CTAs over the SMs; the decode kernel only pays off with one
};

static DecodePlan plan_decode(int M, int N, int K, int sms, int force_splits) {
  DecodePlan best{};
  const int nt = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  const int n_tiles = (N + 127) / 128;
  const int KBt = K / 128;
  const int stage_bytes = kWTileBytes + nt * 128;
  double best_cost = 1e30;
  for (int s = 1; s <= 8; ++s) {
    if (force_splits > 0 && s != force_splits) continue;
    const int kbps = (KBt + s - 1) / s;
    const int s_eff = (KBt + kbps - 1) / kbps;
    if (s_eff != s && force_splits <= 0) continue;  // same plan as a smaller s
    int stages = kbps < kDecMaxStages ? kbps : kDecMaxStages;
    if (stages < 2) stages = 2;  // the stage area doubles as the send buffer of the exchange
    const int fixed = kbps * (nt + 1) * 4 + 64 + 2048;
    const int exchange = (2 * nt + 8) * 512;   // send + receive areas, inside the ring
    // Three stages: with more, the CTAs of a deep-K plan (seven K blocks each at K = 7168) no longer
    // fit three to an SM and the launch needs a second wave (13.5 -> 11.1 us at M=32, N=4096).
    if (stages > 3) stages = 3;
    while (stages > 2 && stages * stage_bytes + fixed > 232448) --stages;
    const int ring = stages * stage_bytes > exchange ? stages * stage_bytes : exchange;
    const int smem = ring + fixed;
    if (smem > 232448) continue;
    int cps = 232448 / (smem + 1024);
    const int tmem_cols = nt * 4 < 32 ? 32 : nt * 4;
    if (cps > 512 / tmem_cols) cps = 512 / tmem_cols;
    if (cps > 4) cps = 4;
    if (cps < 1) continue;
    const long ctas = static_cast<long>(n_tiles) * s_eff;
    // the K split is chosen as if two CTAs shared an SM (more splits only lengthen the exchange);
    // the rest of the SM is left to the next launch
    const long slots = static_cast<long>(sms) * (cps > 2 ? 2 : cps);
    const long rounds = (ctas + slots - 1) / slots;
    // a round costs the MMA-issue time of its K blocks (~0.2 us each; two co-resident CTAs share
    // the SM) plus a fixed ~1 us (fill latency, reduction, store)
    const double cost = rounds * (kbps * 0.2 * (cps > 1 && ctas > sms ? 1.5 : 1.0) + 1.0);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = DecodePlan{nt, s_eff, kbps, stages, cps, rounds};
    }
  }
  return best;
}

template <int NT, typename OutT>
static int launch_decode(const CUtensorMap& tmap, const DecodeParams& p, int n_tiles,
                         cudaStream_t stream) {
  auto kern = bs_gemm_decode_kernel<NT, OutT>;
  const int smem = DecCfg<NT>::smem_bytes(p.stages, p.kbps);
  if (smem > 232448)
    return set_error(FLYB200_ERR_UNSUPPORTED, "decode plan needs %d bytes of shared memory", smem);
  static thread_local int configured_dev = -1;
  int dev = 0;
  FLYB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    FLYB200_CUDA_CHECK(
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(n_tiles * p.splits), 1, 1);
  cfg.blockDim = dim3(kDecThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = static_cast<unsigned>(p.splits);
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 2;
  FLYB200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmap, p));
  return FLYB200_OK;
}

// Whether the automatic dispatch should take the decode kernel (measured on B200): it wins when all
// of its CTAs are resident at once (one wave) -- with more than 32 tokens only if K is deep enough
// (>= 32 blocks) for split-K to matter; wide-N shapes that need several waves run faster on the
// persistent tiled kernel.
bool decode_path_pays_off(int M, int N, int K) {
  const int sms = sm_count();
  if (sms <= 0 || M > 64) return false;
  const DecodePlan plan = plan_decode(M, N, K, sms, 0);
  if (plan.splits < 1 || plan.rounds != 1) return false;
  if (M > 32 && K / 128 < 32) return false;
  return true;
}

// Entry used by flyb200_blockscale_gemm for M <= 64.
int launch_decode_gemm(void* c, const void* a, const void* b_repacked, const float* scale_a_t,
                       const float* scale_b, int M, int N, int K, int out_dtype, int force_splits,
                       cudaStream_t stream, bool pertoken) {
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const DecodePlan plan = plan_decode(M, N, K, sms, force_splits);
  if (plan.splits < 1)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "no decode plan for M=%d N=%d K=%d", M, N, K);
  DecodeParams p{};
  p.b = reinterpret_cast<const uint8_t*>(b_repacked);
  p.scale_a = scale_a_t;
  p.scale_b = scale_b;
  p.out = c;
  p.err = device_error_word();
  if (!p.err) return FLYB200_ERR_CUDA;
  p.M = M; p.N = N; p.K = K;
  p.splits = plan.splits; p.kbps = plan.kbps; p.stages = plan.stages;
  p.pertoken = pertoken ? 1 : 0;
  CUtensorMap tmap;
  int rc = make_tensor_map_2d(&tmap, a, M, K, 1, plan.nt);
  if (rc) return rc;
  const int n_tiles = (N + 127) / 128;
  const bool bf16 = out_dtype == FLYB200_BF16;
  switch (plan.nt) {
    case 16:
      return bf16 ? launch_decode<16, __nv_bfloat16>(tmap, p, n_tiles, stream)
                  : launch_decode<16, __half>(tmap, p, n_tiles, stream);
    case 32:
      return bf16 ? launch_decode<32, __nv_bfloat16>(tmap, p, n_tiles, stream)
                  : launch_decode<32, __half>(tmap, p, n_tiles, stream);
    default:
      return bf16 ? launch_decode<64, __nv_bfloat16>(tmap, p, n_tiles, stream)
                  : launch_decode<64, __half>(tmap, p, n_tiles, stream);
  }
}

}  // namespace flyb200
