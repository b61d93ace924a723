// Weight-only int4 x bf16 GEMM for decode-size M (<= 64 tokens): C[M, N] = A[M, K] * dequant(W)[N, K]^T,
// W signed 4-bit with one bf16 scale per (row, 128-wide K group). HBM-bound on the packed weights
// (N*K/2 bytes), so the kernel streams them once and does everything else on chip:
//
//   * swap-AB like the fp8 decode kernel: the 128-row weight tile is the MMA "A" operand
//     (accumulator lane = output column n), the tokens are the MMA "B" operand (NT = 16/32/64).
//   * the packed weights (8 KB per 128-row x 128-K group, contiguous) are fetched by bulk copies into
//     a ring of eight shared-memory slots that runs well ahead of the consumers: 64 KB in flight per
//     CTA keeps the HBM queue full (prefetching one group ahead in registers was latency-bound at
//     1.2 TB/s).
//   * four dequantiser warps turn each packed 128-row x 128-K group (8 KB) into EXACT integer-valued
//     bf16 (-8..7) in the 128-byte-swizzled K-major image the tensor core reads (two 64-K sub-tiles):
//     nibble n = q + 8; (n | 0x4300) is bf16 128 + n; minus 136 gives q. Three integer/half2
//     instructions per two weights, no scale applied yet.
//   * tcgen05.mma kind::f16 (bf16 x bf16 -> f32), 128 x NT x 16, eight per K group, each group into a
//     fresh TMEM accumulator buffer.
//   * the epilogue applies the group scale per accumulator lane in fp32 --
//     acc[n][m] += scale[n][g] * sum_k q[n][k] * a[m][k] -- the same promotion structure as the
//     block-scale kernels; this equals dequantise-then-matmul with the products q*a summed exactly
//     in fp32 before scaling.
//   * split-K over a thread-block cluster with the partials exchanged by bulk copies through
//     distributed shared memory and summed in rank order (deterministic), as in decode_gemm.cu.
//
// The reference has no kernel for this exact format (its nearest code is the W4A16 path of
// kernels/moe_gemm_2stage.py:607-630 and the int4 unpack of kernels/mfma_preshuffle_pipeline.py:
// 202-222); the contract is "dequantise, then matmul".
//
// Packed layout (flyb200_int4_repack): wq [K/128][N/8][4][8][16 bytes] -- per 128-K group and block
// of 8 rows, four 16-byte chunks (32 K elements each), each chunk holding its 8 rows back to back,
// so that a warp reading one chunk of 8 consecutive rows touches 128 contiguous bytes. The 8 nibbles
// of each 32-bit word hold 8 consecutive K elements in the order e0 e2 e4 e6 e1 e3 e5 e7 (low nibble
// first), so that (word >> 4q) & 0x000F000F yields the pair (e_2q, e_2q+1) in the two 16-bit
// halves. Scales [K/128][N] bf16.
#include "common.cuh"
#include "cluster.cuh"

namespace flyb200 {

constexpr int kI4DqWarps = 8;       // dequantiser warps (two per SM sub-partition)
constexpr int kI4Threads = 192 + 32 * kI4DqWarps + 32;   // warp 0 token TMA, warp 1 MMA, warps 2-5 epilogue,
                                    // warps 6-13 dequantise, warp 14 packed-weight and scale copies
constexpr int kI4PackedSlots = 8;   // ring of packed 8 KB groups
constexpr int kI4PackedBytes = 128 * 64;
constexpr int kI4MaxStages = 6;
constexpr int kI4WBytes = 2 * 128 * 128;   // two 64-K bf16 sub-tiles of 128 rows

struct Int4Params {
  const uint8_t* wq;               // [K/128][N/8][4][8][16]
  const __nv_bfloat16* scales_t;   // [K/128][N]
  void* out;                       // [M, N] bf16
  int* err;
  int M, N, K;
  int splits, kbps, stages;
};

__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// bf16 x bf16 -> f32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_bf16_f32(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

template <int NT>
struct I4Cfg {
  static constexpr int kXBytes = 2 * NT * 128;               // two 64-K sub-tiles of NT token rows
  static constexpr int kStageBytes = kI4WBytes + kXBytes;
  static constexpr int kAccBufs = (256 / NT) > 8 ? 8 : (256 / NT);
  static constexpr int kTmemCols = NT * kAccBufs < 32 ? 32 : NT * kAccBufs;
  static constexpr int kPartialBytes = (NT + 8) * 128 * 4;   // [sender][local column][128] fp32
  static constexpr int kMiscBytes = 1024;
  // + the group scales of the CTA's K range: [kbps][128] bf16
  static int smem_bytes(int stages, int kbps) {
    return stages * kStageBytes + kI4PackedSlots * kI4PackedBytes + kPartialBytes + kbps * 256 + kMiscBytes + 1024;
  }
};

template <int NT>
__global__ void __launch_bounds__(kI4Threads)
int4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const Int4Params p) {
  using C = I4Cfg<NT>;
  constexpr int kAccBufs = C::kAccBufs;
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int kDone = stages + kAccBufs;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t packed_off = stages * C::kStageBytes;                       // ring of packed groups
  const uint32_t recv_off = packed_off + kI4PackedSlots * kI4PackedBytes;
  const uint32_t recv_base = smem_base + recv_off;
  float* recv = reinterpret_cast<float*>(smem_al + recv_off);
  const uint32_t scale_off = recv_off + C::kPartialBytes;                    // [kbps][128] bf16
  const __nv_bfloat16* sc_s = reinterpret_cast<const __nv_bfloat16*>(smem_al + scale_off);
  const uint32_t misc_off = scale_off + static_cast<uint32_t>(p.kbps) * 256u;
  const uint32_t bar_base = smem_base + misc_off;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto done_bar = [&](uint32_t i) { return bar_base + 8u * (kI4MaxStages + i); };               // < 6 + 8
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kI4MaxStages + 8 + b); };
  const uint32_t recv_bar = bar_base + 8u * (2 * kI4MaxStages + 16);
  auto pk_full_bar = [&](int s) { return bar_base + 8u * (2 * kI4MaxStages + 17 + s); };
  auto pk_empty_bar = [&](int s) { return bar_base + 8u * (2 * kI4MaxStages + 17 + kI4PackedSlots + s); };
  const uint32_t scale_bar = bar_base + 8u * (2 * kI4MaxStages + 17 + 2 * kI4PackedSlots);
  constexpr int kBars = 2 * kI4MaxStages + 18 + 2 * kI4PackedSlots;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_al + misc_off + 8 * kBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_al + misc_off + 8 * kBars + 4);

  const int split = static_cast<int>(cluster_ctarank());
  const int n_tile = blockIdx.x / p.splits;
  const int n0 = n_tile * 128;
  const int KBt = p.K / 128;
  const int kb_begin = split * p.kbps;
  const int kb_end = min(KBt, kb_begin + p.kbps);
  const int count = max(0, kb_end - kb_begin);

  if (warp == 0) {
    // operands of a stage: the token TMA (one arrival + bytes) and the four dequantiser warps
    if (lane < stages) mbar_init(full_bar(lane), 1 + kI4DqWarps);
    if (lane < kDone) mbar_init(done_bar(lane), 1);
    if (lane < kAccBufs) mbar_init(tempty_bar(lane), 4);
    if (lane < kI4PackedSlots) {
      mbar_init(pk_full_bar(lane), 1);
      mbar_init(pk_empty_bar(lane), kI4DqWarps);   // one arrival per dequantiser warp
    }
    if (lane == 0) {
      mbar_init(recv_bar, 1);
      mbar_init(scale_bar, 1);
      *abort_flag = 0;
      prefetch_tensormap(&tmap_x);
    }
    fence_proxy_async_smem();
    fence_barrier_init();
    if (lane == 0) {
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
  cluster_sync_all();   // the receive barriers of the whole cluster exist before anybody signals them

  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  auto wait_stage_free = [&](int i, int code) -> bool {
    if (i < stages) return true;
    const uint32_t j = i - stages;
    return mbar_wait(done_bar(j % kDone), (j / kDone) & 1, abort_flag, p.err, code);
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- token tiles by TMA ----------------
      for (int i = 0; i < count; ++i) {
        const int s = i % stages;
        if (!wait_stage_free(i, kErrWaitSmemEmpty)) break;
        const uint32_t sx = smem_base + s * C::kStageBytes + kI4WBytes;
        mbar_arrive_expect_tx(full_bar(s), C::kXBytes);
        const int k0 = (kb_begin + i) * 128;
        tma_load_2d(sx, &tmap_x, k0, 0, full_bar(s));
        tma_load_2d(sx + NT * 128, &tmap_x, k0 + 64, 0, full_bar(s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = umma_idesc_bf16_f32(128, NT);
      for (int i = 0; i < count; ++i) {
        const int s = i % stages;
        const int buf = i % kAccBufs;
        if (!mbar_wait(tempty_bar(buf), ((i / kAccBufs) & 1) ^ 1, abort_flag, p.err, kErrWaitTmemEmpty) ||
            !mbar_wait(full_bar(s), (i / stages) & 1, abort_flag, p.err, kErrWaitSmemFull))
          break;
        tc_fence_after();
        const uint32_t sw = smem_base + s * C::kStageBytes;
        const uint32_t d = tmem_base + buf * NT;
        constexpr int kSubTiles = 2;
#pragma unroll
        for (int h = 0; h < kSubTiles; ++h) {
          const uint64_t wdesc = umma_desc_sw128(sw + h * (128 * 128));
          const uint64_t xdesc = umma_desc_sw128(sw + kI4WBytes + h * (NT * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_bf16(d, wdesc + 2 * k, xdesc + 2 * k, idesc, (h | k) ? 1u : 0u);
        }
        tc_commit(done_bar(i % kDone));
      }
    }
  } else if (warp == 6 + kI4DqWarps) {
    if (lane == 0) {
      // ---------------- group scales of the whole K range (256 bytes per group), all in flight at
      // once: read one by one in the promotion loop they cost a DRAM latency per group ----------------
      if (count > 0) {
        mbar_arrive_expect_tx(scale_bar, static_cast<uint32_t>(count) * 256u);
        for (int i = 0; i < count; ++i)
          bulk_load(smem_base + scale_off + i * 256,
                    p.scales_t + static_cast<size_t>(kb_begin + i) * p.N + n0, 256, scale_bar);
      }
      // ---------------- packed weights: bulk copies, up to eight groups ahead ----------------
      for (int i = 0; i < count; ++i) {
        const int ps = i % kI4PackedSlots;
        if (i >= kI4PackedSlots &&
            !mbar_wait(pk_empty_bar(ps), ((i / kI4PackedSlots) & 1) ^ 1, abort_flag, p.err, kErrWaitSmemEmpty))
          break;
        mbar_arrive_expect_tx(pk_full_bar(ps), kI4PackedBytes);
        bulk_load(smem_base + packed_off + ps * kI4PackedBytes,
                  p.wq + (static_cast<size_t>(kb_begin + i) * p.N + n0) * 64, kI4PackedBytes, pk_full_bar(ps));
      }
    }
  } else if (warp >= 6) {
    // ---------------- dequantiser: packed int4 -> integer-valued bf16, swizzled K-major ----------
    // The group's packed tile is 512 16-byte vectors (row = v / 4, K quarter = v % 4); thread t takes
    // vectors t, t+256 (eight warps) of the shared-memory slot (conflict-free: a warp reads 512
    // contiguous bytes per instruction). One vector = 32 weights = four 16-byte chunks of the bf16 image.
    constexpr int kDqThreads = 32 * kI4DqWarps;
    constexpr int kVecs = 512 / kDqThreads;          // 16-byte vectors per thread per group
    const int dt = threadIdx.x - 192;   // 0..kDqThreads-1
    for (int i = 0; i < count; ++i) {
      const int ps = i % kI4PackedSlots;
      const bool have = mbar_wait(pk_full_bar(ps), (i / kI4PackedSlots) & 1, abort_flag, p.err, kErrWaitSmemFull);
      if (!__all_sync(0xffffffffu, have)) break;
      uint4 cur[kVecs];
      const uint32_t pk = smem_base + packed_off + ps * kI4PackedBytes + dt * 16;
#pragma unroll
      for (int j = 0; j < kVecs; ++j)
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(cur[j].x), "=r"(cur[j].y), "=r"(cur[j].z), "=r"(cur[j].w)
                     : "r"(pk + j * (kDqThreads * 16))
                     : "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(pk_empty_bar(ps));   // the slot may be refilled
      const int s = i % stages;
      const bool ok = wait_stage_free(i, kErrWaitGather);
      if (!__all_sync(0xffffffffu, ok)) break;
      const uint32_t sw = smem_base + s * C::kStageBytes;
#pragma unroll
      for (int j = 0; j < kVecs; ++j) {
        const int vec = j * kDqThreads + dt;        // position in the packed tile: [row / 8][part][row % 8]
        const int r = ((vec >> 5) << 3) | (vec & 7), part = (vec >> 3) & 3;
        const uint32_t row_base = sw + (part >> 1) * (128 * 128) + r * 128;
        const uint32_t w[4] = {cur[j].x, cur[j].y, cur[j].z, cur[j].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {        // word q = 8 weights = one 16-byte chunk
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t t = ((w[q] >> (4 * e)) & 0x000F000Fu) | 0x43004300u;
            __nv_bfloat162 h2 = *reinterpret_cast<const __nv_bfloat162*>(&t);
            const uint32_t c136 = 0x43084308u;
            h2 = __hsub2(h2, *reinterpret_cast<const __nv_bfloat162*>(&c136));
            o[e] = *reinterpret_cast<const uint32_t*>(&h2);
          }
          const int chunk = (part & 1) * 4 + q;
          const uint32_t addr = row_base + ((chunk ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[0]), "r"(o[1]),
                       "r"(o[2]), "r"(o[3])
                       : "memory");
        }
      }
      fence_proxy_async_smem();   // generic-proxy writes -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(full_bar(s));
    }
  } else {
    // ---------------- epilogue: thread = output column n (accumulator lane) ----------------
    const int et = threadIdx.x - 64;            // 0..127
    const int quad = warp & 3;                  // TMEM lane quadrant this warp may read
    const int n_loc = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    float acc[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j] = 0.f;
    bool alive = true;
    if (count > 0) {
      const bool have = mbar_wait(scale_bar, 0, abort_flag, p.err, kErrWaitSmemFull);
      alive = __all_sync(0xffffffffu, have);
    }
    for (int i = 0; i < count && alive; ++i) {
      const float sg = __bfloat162float(sc_s[i * 128 + n_loc]);
      const int buf = i % kAccBufs;
      const bool got = mbar_wait(done_bar(i % kDone), (i / kDone) & 1, abort_flag, p.err, kErrWaitTmemFull);
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
#pragma unroll
      for (int j = 0; j < NT; ++j) acc[j] = fmaf(__uint_as_float(v[j]), sg, acc[j]);
    }
    // split-K exchange (same scheme as the fp8 decode kernel): partials as [token][n] into the free
    // stage area, one bulk copy per owner CTA, owners add in rank order and store.
    float* send = reinterpret_cast<float*>(smem_al);
#pragma unroll
    for (int j = 0; j < NT; ++j)
      if (j < p.M) send[j * 128 + n_loc] = acc[j];
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
    const int j_lo = split * cpc;
    const int j_hi = min(p.M, j_lo + cpc);
    if (j_hi > j_lo && alive) {
      const bool got = mbar_wait(recv_bar, 0, abort_flag, p.err, kErrWaitExchange);
      if (__all_sync(0xffffffffu, got)) {
        __nv_bfloat16* const out = reinterpret_cast<__nv_bfloat16*>(p.out);
        for (int jb = j_lo; jb < j_hi; jb += 8) {
          float sum[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) sum[u] = 0.f;
          for (int c = 0; c < p.splits; ++c) {  // fixed rank order: deterministic
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (jb + u < j_hi) sum[u] += recv[(c * cpc + (jb - j_lo) + u) * 128 + n_loc];
          }
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (jb + u < j_hi)
              out[static_cast<size_t>(jb + u) * p.N + n0 + n_loc] = __float2bfloat16_rn(sum[u]);
        }
      }
    }
  }

  // Nobody leaves before every bulk copy that reads its shared memory has been consumed.
  __syncwarp();
  cluster_sync_all();

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

// values [N, K] int8 in [-8, 7] + scales [N, K/128] bf16 -> the packed layout above
__global__ void __launch_bounds__(256)
int4_repack_kernel(const int8_t* __restrict__ q, const __nv_bfloat16* __restrict__ scales,
                   uint32_t* __restrict__ wq, __nv_bfloat16* __restrict__ scales_t, int N, int K) {
  const int KB = K / 128;
  const long long words = static_cast<long long>(KB) * N * 16;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < words;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int wi = static_cast<int>(i & 15);
    const long long rn = i >> 4;
    const int n = static_cast<int>(rn % N);
    const int kb = static_cast<int>(rn / N);
    const int8_t* src = q + static_cast<size_t>(n) * K + kb * 128 + wi * 8;
    uint32_t w = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const uint32_t nib = static_cast<uint32_t>(src[e] + 8) & 0xFu;
      const int pos = (e & 1) ? 4 + (e >> 1) : (e >> 1);   // e0 e2 e4 e6 e1 e3 e5 e7
      w |= nib << (4 * pos);
    }
    // [kb][n / 8][chunk = wi / 4][row = n % 8][word = wi % 4]: a warp reading one chunk of eight
    // consecutive rows touches 128 contiguous bytes of the shared-memory copy (no bank conflicts)
    wq[(((static_cast<long long>(kb) * (N / 8) + n / 8) * 4 + (wi >> 2)) * 8 + (n & 7)) * 4 + (wi & 3)] = w;
    if (wi == 0) scales_t[static_cast<size_t>(kb) * N + n] = scales[static_cast<size_t>(n) * KB + kb];
  }
}

int make_tensor_map_2d(CUtensorMap* map, const void* base, int rows, int cols, int elem_bytes,
                       int box_rows);  // blockscale_gemm.cu

struct I4Plan {
  int nt, splits, kbps, stages;
};

static I4Plan plan_int4(int M, int N, int K, int sms, int force_splits) {
  I4Plan best{0, 0, 0, 0};
  const int nt = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  const int n_tiles = N / 128;
  const int KBt = K / 128;
  const int stage_bytes = kI4WBytes + 2 * nt * 128;
  double best_cost = 1e30;
  for (int s = 1; s <= 8; ++s) {
    if (force_splits > 0 && s != force_splits) continue;
    const int kbps = (KBt + s - 1) / s;
    const int s_eff = (KBt + kbps - 1) / kbps;
    if (s_eff != s && force_splits <= 0) continue;
    int stages = kbps < kI4MaxStages ? kbps : kI4MaxStages;
    if (stages < 2) stages = 2;   // the stage area doubles as the send buffer of the exchange
    const int fixed = (nt + 8) * 512 + 2048 + kI4PackedSlots * kI4PackedBytes + kbps * 256;
    while (stages > 2 && stages * stage_bytes + fixed > 232448) --stages;
    if (stages * stage_bytes + fixed > 232448) continue;
    const long ctas = static_cast<long>(n_tiles) * s_eff;
    const long rounds = (ctas + sms - 1) / sms;
    // a round streams kbps groups (dequantisation ~0.15 us each) plus a fixed ~1.5 us
    const double cost = rounds * (kbps * 0.15 + 1.5);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = I4Plan{nt, s_eff, kbps, stages};
    }
  }
  return best;
}

template <int NT>
static int launch_int4(const CUtensorMap& tmap, const Int4Params& p, cudaStream_t stream) {
  auto kern = int4_gemm_kernel<NT>;
  const int smem = I4Cfg<NT>::smem_bytes(p.stages, p.kbps);
  if (smem > 232448) return set_error(FLYB200_ERR_UNSUPPORTED, "int4 plan needs %d bytes of shared memory", smem);
  static thread_local int configured_dev = -1;
  int dev = 0;
  FLYB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    FLYB200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>((p.N / 128) * p.splits), 1, 1);
  cfg.blockDim = dim3(kI4Threads, 1, 1);
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

}  // namespace flyb200

namespace flyb200 {
int launch_int4_stream(void* c, const void* a, const void* wq, const void* scales_t, int M, int N, int K,
                       int force_splits, cudaStream_t stream);  // int4_stream.cu
}

using namespace flyb200;

extern "C" int flyb200_int4_repack(const int8_t* q, const void* scales, int32_t N, int32_t K, void* wq_out,
                                   void* scales_t_out, void* stream) {
  if (!q || !scales || !wq_out || !scales_t_out)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "int4_repack: NULL buffer");
  if (N < 8 || N % 8 || K < 128 || K % 128 || reinterpret_cast<uintptr_t>(wq_out) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "int4_repack: K %% 128 == 0, N %% 8 == 0 and a 16-byte aligned output");
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  int4_repack_kernel<<<sms * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      q, static_cast<const __nv_bfloat16*>(scales), static_cast<uint32_t*>(wq_out),
      static_cast<__nv_bfloat16*>(scales_t_out), N, K);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

extern "C" int flyb200_int4_gemm(void* c, const void* a, const void* wq, const void* scales_t, int32_t M,
                                 int32_t N, int32_t K, const flyb200_gemm_cfg* cfg, void* stream) {
  if (!c || !a || !wq || !scales_t) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "int4_gemm: NULL buffer");
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(wq)) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "int4_gemm: a and wq must be 16-byte aligned");
  if (M < 1 || M > 64) return set_error(FLYB200_ERR_UNSUPPORTED, "int4_gemm: 1 <= M <= 64 (got %d)", M);
  if (N < 128 || N % 128 || K < 128 || K % 128)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "int4_gemm: N and K must be multiples of 128 (N=%d K=%d)", N, K);
  // cfg.path: 1 = the register-dequantising mma.sync kernel (int4_stream.cu), 2 = the tcgen05 kernel
  // of this file, 0 = whichever was measured faster: up to 32 tokens the former (21.5 / 26.9 us
  // against 32.3 / 33.5 us at N = K = 8192), above that the latter (35.6 against 38.4 us at 64)
  const int path = (cfg && cfg->path) ? cfg->path : (M <= 32 ? 1 : 2);
  if (path != 2)
    return launch_int4_stream(c, a, wq, scales_t, M, N, K, cfg ? cfg->split_k : 0,
                              reinterpret_cast<cudaStream_t>(stream));
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const I4Plan plan = plan_int4(M, N, K, sms, cfg ? cfg->split_k : 0);
  if (plan.splits < 1) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "int4_gemm: no plan for M=%d N=%d K=%d", M, N, K);
  Int4Params p{};
  p.wq = static_cast<const uint8_t*>(wq);
  p.scales_t = static_cast<const __nv_bfloat16*>(scales_t);
  p.out = c;
  p.err = device_error_word();
  if (!p.err) return FLYB200_ERR_CUDA;
  p.M = M; p.N = N; p.K = K;
  p.splits = plan.splits; p.kbps = plan.kbps; p.stages = plan.stages;
  CUtensorMap tmap;
  int rc = make_tensor_map_2d(&tmap, a, M, K, 2, plan.nt);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (plan.nt) {
    case 16: return launch_int4<16>(tmap, p, st);
    case 32: return launch_int4<32>(tmap, p, st);
    default: return launch_int4<64>(tmap, p, st);
  }
}
