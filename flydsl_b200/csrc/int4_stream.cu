// Weight-only int4 x bf16 GEMM for decode-size M (<= 64), register-dequantising kernel: the default
// path of flyb200_int4_gemm (int4_gemm.cu keeps the tcgen05 variant and the packed layout's
// description; both read the same packed weights and give the same arithmetic contract).
//
// Why not tcgen05 here: with 16-64 tokens the tensor work is negligible and the kernel lives or dies
// by how cheaply 4-bit weights become MMA operands at HBM speed. tcgen05.mma reads its operands
// from shared memory, so every weight takes a round trip nibble -> bf16 -> shared memory (4x the
// packed bytes, written and read again: ~660 cycles of shared-memory bandwidth per 8 KB group), and
// one thread issues eight K=16 instructions per group at ~60 cycles each plus the commit (~690
// cycles per group, measured) where the SM's share of HBM bandwidth allows ~330. mma.sync takes the
// weight operand from REGISTERS: a thread unpacks exactly the nibbles of its own B fragment (shift,
// and/or, subtract: three instructions per two weights), every warp issues its own MMAs, and shared
// memory only carries the packed bytes once.
//
//   * CTA = one 128-row weight tile x one K range (split-K over a thread-block cluster, partial sums
//     exchanged through distributed shared memory and added in rank order, as in decode_gemm.cu).
//   * warp 8 (one thread): ring of slots, each = one packed 128 x 128 group (8 KB, one bulk copy)
//     + the tokens' 128 K columns (two TMA tiles of 64 K, 128-byte swizzle); group scales of the whole
//     K range in one go.
//   * warps 0-7: warp w owns weight rows [16w, 16w+16) = two n-blocks of mma.m16n8k16 (tokens are
//     the M=16 side). Per group: 8 x 16-byte loads of its rows' packed words (the four threads of a
//     quad read the same row: a broadcast), per K step one ldmatrix.x4 of the token fragment and two
//     MMAs into a per-group accumulator, then acc += group_sum * scale[n][group] in fp32 -- the same
//     promotion structure as the block-scale kernels: equals dequantise-then-matmul with the products
//     q*a summed in fp32 before scaling. (The template also builds with four n-blocks per warp and
//     with the K steps of a group dealt out to two or four warps; neither was faster.)
//
// Where the time goes (ncu, M=16, N=K=8192): the schedulers issue on 43 % of the cycles, the integer
// ALU pipe is the busiest at 41 %, the legacy tensor pipe 22 %, DRAM 17 %: the unpack instructions
// (three per two weights) bound the kernel at ~960 cycles per 8 KB group against ~330 for the SM's
// share of HBM bandwidth.
//
// Packed layout (flyb200_int4_repack): wq [K/128][N/8][4][8][16 bytes] (see int4_gemm.cu); word j of
// a row holds K elements 8j..8j+7 as nibbles q+8 in the order e0 e2 e4 e6 e1 e3 e5 e7, so
// (word >> 4t) & 0x000F000F is the
// pair (e_2t, e_2t+1) in the two 16-bit halves: exactly the (k, k+1) pair that thread t of a quad
// holds in the B fragment (words 2s and 2s+1 give the fragment's two registers for K step s).
// (n | 0x4300) is the bf16 value 128 + n; minus 136 gives q exactly.
#include "common.cuh"
#include "cluster.cuh"

namespace flyb200 {

// consumer warps: 16 / NB row groups (NB n-blocks of 8 weight rows each) x KS parts of each group's
// K steps; + one producer warp
constexpr int s4_threads(int nb, int ks) { return 32 * ((16 / nb) * ks + 1); }
constexpr int kS4MaxSlots = 16;
constexpr int kS4PackedBytes = 128 * 64;

struct Int4StreamParams {
  const uint8_t* wq;               // [K/128][N/8][4][8][16]
  const __nv_bfloat16* scales_t;   // [K/128][N]
  __nv_bfloat16* out;              // [M, N]
  int* err;
  int M, N, K;
  int splits, kbps, slots;
};

template <int MB>
struct S4Cfg {
  static constexpr int kTokens = 16 * MB;
  static constexpr int kXSub = kTokens * 128;                 // one 64-K sub-tile of the tokens
  static constexpr int kSlotBytes = kS4PackedBytes + 2 * kXSub;
  static constexpr int kRecvBytes = (kTokens + 8) * 128 * 4;  // [sender][local token][128] fp32
  static int smem_bytes(int slots, int kbps) {
    int ring = slots * kSlotBytes;
    const int send = kTokens * 512;                           // the ring doubles as the send buffer
    if (ring < send) ring = send;
    return ring + kRecvBytes + kbps * 256 + 1024 + 1024;
  }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two nibbles (already shifted to bits 0-3 and 16-19) -> two exact bf16 integers in [-8, 7]
__device__ __forceinline__ uint32_t dq_pair(uint32_t shifted) {
  const uint32_t t = (shifted & 0x000F000Fu) | 0x43004300u;   // bf16 (128 + n), twice
  const uint32_t c136 = 0x43084308u;
  __nv_bfloat162 h = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&t),
                             *reinterpret_cast<const __nv_bfloat162*>(&c136));
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int MB, int NB, int KS>
__global__ void __launch_bounds__(s4_threads(NB, KS), 1)
int4_stream_kernel(const __grid_constant__ CUtensorMap tmap_x, const Int4StreamParams p) {
  using C = S4Cfg<MB>;
  constexpr int kRowGroups = 16 / NB;
  constexpr int kConsumers = kRowGroups * KS;
  constexpr int kSteps = 8 / KS;      // K steps of a group per consumer warp
  constexpr int kWords = 16 / KS;     // packed words of a row per consumer warp
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slots = p.slots;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  int ring_bytes = slots * C::kSlotBytes;
  if (ring_bytes < C::kTokens * 512) ring_bytes = C::kTokens * 512;
  const uint32_t recv_off = static_cast<uint32_t>(ring_bytes);
  const uint32_t recv_base = smem_base + recv_off;
  const float* recv = reinterpret_cast<const float*>(smem_al + recv_off);
  const uint32_t scale_off = recv_off + C::kRecvBytes;                       // [kbps][128] bf16
  const uint32_t misc_off = scale_off + static_cast<uint32_t>(p.kbps) * 256u;
  const uint32_t bar_base = smem_base + misc_off;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kS4MaxSlots + s); };
  const uint32_t recv_bar = bar_base + 8u * (2 * kS4MaxSlots);
  const uint32_t scale_bar = bar_base + 8u * (2 * kS4MaxSlots + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_al + misc_off + 8 * (2 * kS4MaxSlots + 2));

  const int split = static_cast<int>(cluster_ctarank());
  const int n_tile = blockIdx.x / p.splits;
  const int n0 = n_tile * 128;
  const int KBt = p.K / 128;
  const int kb_begin = split * p.kbps;
  const int kb_end = min(KBt, kb_begin + p.kbps);
  const int count = max(0, kb_end - kb_begin);
  const int cpc = (p.M + p.splits - 1) / p.splits;   // tokens each CTA of the cluster reduces and stores

  if (warp == 0) {
    if (lane < slots) {
      mbar_init(full_bar(lane), 1);
      mbar_init(empty_bar(lane), kConsumers);
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
      const int own = min(p.M, (split + 1) * cpc) - split * cpc;
      if (own > 0) mbar_arrive_expect_tx(recv_bar, static_cast<uint32_t>(own * p.splits) * 512u);
    }
  }
  __syncthreads();
  cluster_sync_all();   // the receive barriers of the whole cluster exist before anybody signals them

  // Programmatic dependent launch: the packed weights and group scales of the first ring fill are
  // requested BEFORE the dependency wait -- they are parameters, never the result of the kernel that
  // runs just before (a kernel of this library that lets its dependents start early writes no
  // weights; any other kernel has exited before this one starts) -- so that back-to-back launches
  // stream weights while the previous one still reduces and stores. The tokens are read after it.
  const int first_fill = count < slots ? count : slots;
  if (warp == kConsumers && lane == 0 && count > 0) {
    mbar_arrive_expect_tx(scale_bar, static_cast<uint32_t>(count) * 256u);
    for (int i = 0; i < count; ++i)
      bulk_load(smem_base + scale_off + i * 256, p.scales_t + static_cast<size_t>(kb_begin + i) * p.N + n0,
                256, scale_bar);
    for (int i = 0; i < first_fill; ++i) {
      mbar_arrive_expect_tx(full_bar(i), C::kSlotBytes);
      bulk_load(smem_base + i * C::kSlotBytes, p.wq + (static_cast<size_t>(kb_begin + i) * p.N + n0) * 64,
                kS4PackedBytes, full_bar(i));
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == kConsumers) {
    if (lane == 0 && count > 0) {
      // ---------------- producer ----------------
      for (int i = 0; i < first_fill; ++i) {   // tokens of the slots whose weights are on their way
        const uint32_t base = smem_base + i * C::kSlotBytes;
        const int k0 = (kb_begin + i) * 128;
        tma_load_2d(base + kS4PackedBytes, &tmap_x, k0, 0, full_bar(i));
        tma_load_2d(base + kS4PackedBytes + C::kXSub, &tmap_x, k0 + 64, 0, full_bar(i));
      }
      for (int i = first_fill; i < count; ++i) {
        const int s = i % slots;
        if (i >= slots &&
            !mbar_wait(empty_bar(s), ((i / slots) & 1) ^ 1, abort_flag, p.err, kErrWaitSmemEmpty))
          break;
        const uint32_t base = smem_base + s * C::kSlotBytes;
        mbar_arrive_expect_tx(full_bar(s), C::kSlotBytes);
        bulk_load(base, p.wq + (static_cast<size_t>(kb_begin + i) * p.N + n0) * 64, kS4PackedBytes, full_bar(s));
        const int k0 = (kb_begin + i) * 128;
        tma_load_2d(base + kS4PackedBytes, &tmap_x, k0, 0, full_bar(s));
        tma_load_2d(base + kS4PackedBytes + C::kXSub, &tmap_x, k0 + 64, 0, full_bar(s));
      }
    }
  } else {
    // ---------------- consumers ----------------
    const int gid = lane >> 2, tig = lane & 3;
    const uint32_t sh = 4u * tig;
    const int wr = warp % kRowGroups;   // row group: weight rows [8 NB wr, 8 NB (wr + 1))
    const int kh = warp / kRowGroups;   // which part of every group's K steps
    float acc[MB][NB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mb][nb][e] = 0.f;
    bool alive = true;
    if (count > 0) {
      const bool have = mbar_wait(scale_bar, 0, abort_flag, p.err, kErrWaitSmemFull);
      alive = __all_sync(0xffffffffu, have);
    }
    // ldmatrix row address of this lane inside a token sub-tile: matrix mi = lane / 8 covers token
    // rows 8 (mi & 1) .. +7 and the 16-byte K chunk (mi >> 1) of the K step
    const int lm_row = (lane & 7) + 8 * ((lane >> 3) & 1);
    const int lm_chunk = lane >> 4;
    // byte offset of that row's chunk for K step a of a 64-K sub-tile (128-byte swizzle: chunk ^ row % 8;
    // the m-block and sub-tile offsets are multiples of 1024 and do not change row % 8)
    uint32_t lm_off[4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
      lm_off[a] = static_cast<uint32_t>(lm_row * 128 + (((2 * a + lm_chunk) ^ (lane & 7)) << 4));
    for (int i = 0; i < count && alive; ++i) {
      const int s = i % slots;
      const bool got = mbar_wait(full_bar(s), (i / slots) & 1, abort_flag, p.err, kErrWaitSmemFull);
      if (!__all_sync(0xffffffffu, got)) {
        alive = false;
        break;
      }
      const uint32_t base = smem_base + s * C::kSlotBytes;
      // packed words of this thread's two weight rows (64 bytes each)
      // packed tile: [row / 8][chunk][row % 8][16 bytes]; the 8 rows of a chunk are 128 contiguous
      // bytes (the four threads of a quad read the same 16 bytes: a broadcast)
      uint32_t w[NB][kWords];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const uint32_t blk = base + static_cast<uint32_t>(wr * NB + nb) * 512u + gid * 16u;
#pragma unroll
        for (int v = 0; v < kWords / 4; ++v)
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(w[nb][4 * v]), "=r"(w[nb][4 * v + 1]), "=r"(w[nb][4 * v + 2]), "=r"(w[nb][4 * v + 3])
                       : "r"(blk + 128u * (kh * (kWords / 4) + v)));
      }
      float tmp[MB][NB][4];
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int e = 0; e < 4; ++e) tmp[mb][nb][e] = 0.f;
      const uint32_t xs = base + kS4PackedBytes;
#pragma unroll
      for (int kl = 0; kl < kSteps; ++kl) {
        const int ks = kh * kSteps + kl;
        uint32_t a[MB][4];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          ldmatrix_x4(xs + (ks >> 2) * C::kXSub + mb * 2048 + lm_off[ks & 3], a[mb]);
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const uint32_t b0 = dq_pair(w[nb][2 * kl] >> sh);
          const uint32_t b1 = dq_pair(w[nb][2 * kl + 1] >> sh);
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) mma_bf16_16816(tmp[mb][nb], a[mb], b0, b1);
        }
      }
      // the slot has been read (the packed words sit in registers, the token fragments were consumed)
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(s));
      // promotion: columns (2 tig, 2 tig + 1) of each n-block carry their own group scale
      const __nv_bfloat16* sc = reinterpret_cast<const __nv_bfloat16*>(smem_al + scale_off) + i * 128 + wr * (8 * NB);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(sc + nb * 8 + 2 * tig);
        const float s0 = __bfloat162float(s2.x), s1 = __bfloat162float(s2.y);
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          acc[mb][nb][0] = fmaf(tmp[mb][nb][0], s0, acc[mb][nb][0]);
          acc[mb][nb][1] = fmaf(tmp[mb][nb][1], s1, acc[mb][nb][1]);
          acc[mb][nb][2] = fmaf(tmp[mb][nb][2], s0, acc[mb][nb][2]);
          acc[mb][nb][3] = fmaf(tmp[mb][nb][3], s1, acc[mb][nb][3]);
        }
      }
    }

    // ---------------- split-K exchange ----------------
    // Partials as [token][n] fp32 into the ring (every slot has been consumed: all consumers pass
    // the barrier below after their last group), one bulk copy per owner CTA into its receive area
    // [sender][local token][128]; owners add in rank order and store.
    auto consumer_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(32 * kConsumers) : "memory"); };
    consumer_sync();
    float* send = reinterpret_cast<float*>(smem_al);
#pragma unroll
    for (int part = 0; part < KS; ++part) {   // the warps of K part 0 write, those of part 1 add
      if (kh == part) {
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
          for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int tok = mb * 16 + gid + ((e & 2) ? 8 : 0);
              const int n_loc = (wr * NB + nb) * 8 + 2 * tig + (e & 1);
              if (tok < p.M) {
                float* dst = send + tok * 128 + n_loc;
                *dst = part == 0 ? acc[mb][nb][e] : *dst + acc[mb][nb][e];   // fixed order: deterministic
              }
            }
      }
      if (part + 1 < KS) consumer_sync();
    }
    fence_proxy_async_smem();
    consumer_sync();
    if (threadIdx.x == 0 && alive) {
      for (int o = 0; o < p.splits; ++o) {
        const int lo = o * cpc;
        const int cols = min(p.M, lo + cpc) - lo;
        if (cols > 0)
          bulk_copy_to_cta(map_to_cta(recv_base + static_cast<uint32_t>(split * cpc) * 512u, o),
                           smem_base + static_cast<uint32_t>(lo) * 512u, static_cast<uint32_t>(cols) * 512u,
                           map_to_cta(recv_bar, o));
      }
    }
    const int j_lo = split * cpc;
    const int j_hi = min(p.M, j_lo + cpc);
    if (j_hi > j_lo && alive) {
      const bool got = mbar_wait(recv_bar, 0, abort_flag, p.err, kErrWaitExchange);
      if (__all_sync(0xffffffffu, got)) {
        // thread t sums column pair (t & 63) of tokens j_lo + (t >> 6), + kConsumers / 2, ...
        const int cp = threadIdx.x & 63;
        static_assert(kConsumers % 2 == 0, "whole groups of 64 threads");
        for (int j = j_lo + (threadIdx.x >> 6); j < j_hi; j += kConsumers / 2) {
          float2 sum = make_float2(0.f, 0.f);
          for (int c = 0; c < p.splits; ++c) {   // fixed rank order: deterministic
            const float2 v = *reinterpret_cast<const float2*>(recv + (c * cpc + (j - j_lo)) * 128 + 2 * cp);
            sum.x += v.x;
            sum.y += v.y;
          }
          *reinterpret_cast<__nv_bfloat162*>(p.out + static_cast<size_t>(j) * p.N + n0 + 2 * cp) =
              __floats2bfloat162_rn(sum.x, sum.y);
        }
      }
    }
  }

  // Nobody leaves before every bulk copy that reads its shared memory has been consumed.
  __syncwarp();
  cluster_sync_all();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
}

// ---------------------------------- host ----------------------------------------------------------
int make_tensor_map_2d(CUtensorMap* map, const void* base, int rows, int cols, int elem_bytes,
                       int box_rows);  // blockscale_gemm.cu

struct S4Plan {
  int mb, ks, splits, kbps, slots;
};

// K splits (cluster size) and ring depth. One CTA streams kbps groups; the SMs' load is what counts
// (two CTAs may share an SM when M <= 32), plus a fixed cost per wave and a little per split for the
// exchange.
static S4Plan plan_int4_stream(int M, int N, int K, int sms, int force_splits) {
  S4Plan best{0, 0, 0, 0, 0};
  const int mb = M <= 16 ? 1 : (M <= 32 ? 2 : 4);
  const int ks = 1;
  const int n_tiles = N / 128;
  const int KBt = K / 128;
  const int slot = kS4PackedBytes + 2 * 16 * mb * 128;
  double best_cost = 1e30;
  for (int s = 1; s <= 8; ++s) {
    if (force_splits > 0 && s != force_splits) continue;
    const int kbps = (KBt + s - 1) / s;
    const int s_eff = (KBt + kbps - 1) / kbps;
    if (s_eff != s && force_splits <= 0) continue;
    const long ctas = static_cast<long>(n_tiles) * s_eff;
    const long per_sm = (ctas + sms - 1) / sms;
    // up to 32 tokens a CTA takes at most half of an SM's shared memory, so that the CTAs of the
    // next launch are resident (and prefetching) while this one computes
    const int cps = mb <= 2 ? 2 : 1;
    const int fixed = (16 * mb + 8) * 512 + kbps * 256 + 2048;
    int slots = (232448 / cps - 1024 - fixed) / slot;
    if (slots > kS4MaxSlots) slots = kS4MaxSlots;
    if (slots > kbps) slots = kbps;
    if (slots < 2) slots = 2;   // the ring doubles as the send buffer of the exchange
    if (slots * slot + fixed > 232448) continue;
    const long waves = (ctas + sms - 1) / sms;
    const double cost = static_cast<double>(per_sm) * kbps + 6.0 * waves + 0.5 * s_eff;
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = S4Plan{mb, ks, s_eff, kbps, slots};
    }
  }
  return best;
}

template <int MB, int NB, int KS>
static int launch_int4_stream_mb(const CUtensorMap& tmap, const Int4StreamParams& p, cudaStream_t stream) {
  auto kern = int4_stream_kernel<MB, NB, KS>;
  const int smem = S4Cfg<MB>::smem_bytes(p.slots, p.kbps);
  if (smem > 232448)
    return set_error(FLYB200_ERR_UNSUPPORTED, "int4 plan needs %d bytes of shared memory", smem);
  static thread_local int configured_dev = -1;
  int dev = 0;
  FLYB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    FLYB200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>((p.N / 128) * p.splits), 1, 1);
  cfg.blockDim = dim3(s4_threads(NB, KS), 1, 1);
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

// Entry used by flyb200_int4_gemm (arguments already validated there).
int launch_int4_stream(void* c, const void* a, const void* wq, const void* scales_t, int M, int N, int K,
                       int force_splits, cudaStream_t stream) {
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const S4Plan plan = plan_int4_stream(M, N, K, sms, force_splits);
  if (plan.splits < 1)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "int4_gemm: no plan for M=%d N=%d K=%d", M, N, K);
  Int4StreamParams p{};
  p.wq = static_cast<const uint8_t*>(wq);
  p.scales_t = static_cast<const __nv_bfloat16*>(scales_t);
  p.out = static_cast<__nv_bfloat16*>(c);
  p.err = device_error_word();
  if (!p.err) return FLYB200_ERR_CUDA;
  p.M = M; p.N = N; p.K = K;
  p.splits = plan.splits; p.kbps = plan.kbps; p.slots = plan.slots;
  CUtensorMap tmap;
  const int rc = make_tensor_map_2d(&tmap, a, M, K, 2, 16 * plan.mb);
  if (rc) return rc;
  switch (plan.mb) {
    // Eight consumer warps of two n-blocks each, every warp all K steps of a group: measured at
    // M=16, N=K=8192 against 16 warps taking half the K steps each (21.5 / 23.5 us) and against four
    // n-blocks per warp with two or four K parts (22.8 / 24.5 us).
    case 1: return launch_int4_stream_mb<1, 2, 1>(tmap, p, stream);
    case 2: return launch_int4_stream_mb<2, 2, 1>(tmap, p, stream);
    default: return launch_int4_stream_mb<4, 2, 1>(tmap, p, stream);
  }
}

}  // namespace flyb200
