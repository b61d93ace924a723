// Per-token / per-channel scaled FP8 GEMM on CTA pairs: C = (A * B^T) * scale_a[m] * scale_b[n].
//
// The single-CTA per-token kernel (blockscale_gemm.cu, mode kDensePT) is bounded by operand bytes in
// flight: a 128 x 256 tile needs 48 KB per K block and only four such stages fit in shared memory.
// Here two CTAs of a cluster share a 256 x 256 tile: tcgen05.mma.cta_group::2 (M = 256, issued by the
// pair's leader) reads each CTA's own 128 rows of A and HALF of the weight tile from each CTA, so a
// stage is 32 KB per CTA, six stages fit, and every weight byte crosses L2 -> SM once per pair
// instead of once per CTA. No multicast loads: every CTA fetches its own operands.
//
// Roles per CTA (384 threads): warp 0 producer, warp 1 MMA issuer (leader) + TMEM allocation, warp 2
// store thread, warp 3 relay (tells the leader when the peer's stage has landed), warps 4-11 epilogue.
// Every wait is bounded; on expiry the role records a code in the device error word and all roles
// leave through the common teardown (both CTAs always reach the final cluster barrier).
// Reference: kernels/preshuffle_gemm.py:206-1266 (in_dtype fp8); contract run_torch of
// tests/kernels/test_preshuffle_gemm.py:55-66.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "cluster.cuh"
#include "common.cuh"
#include "flyb200.h"

namespace flyb200 {

int make_tensor_map_2d(CUtensorMap* map, const void* base, int rows, int cols, int elem_bytes, int box_rows);

namespace {

constexpr int kPairThreads = 384;
constexpr int kPBK = 128;                       // K bytes per stage row
constexpr int kPStages = 6;
constexpr int kPStageBytes = 2 * 128 * kPBK;    // A 128 rows + B 128 rows
constexpr int kPRegionBytes = 128 * 128;        // 128 rows x 64 bf16
constexpr int kPStagingBytes = 2 * kPRegionBytes;   // half a tile: 128 rows x 128 columns
constexpr int kPMisc = 2048;
constexpr int kPSmem = kPStages * kPStageBytes + kPStagingBytes + kPMisc + 1024;
constexpr int kPAccBufs = 2;
constexpr int kPEpiWarps = 8;

struct PairParams {
  const uint8_t* b;
  const float* scale_a;
  const float* scale_b;
  int* err;
  int M, N, K;
  int group_m;   // pair-row blocks per group of the tile order (0 = one group)
};

__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// completion of all MMAs issued so far -> one arrival on a barrier of the issuing (leader) CTA; the
// leader's relay thread passes it on to the peer
__device__ __forceinline__ void tc_commit2(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f8_2(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on an mbarrier of another CTA of the cluster. Relaxed: the arriving threads publish no
// data of their own (they pass on a completion they have observed on a local barrier); with release
// semantics at cluster scope each such arrival took ~700-900 cycles and was the bottleneck of the loop.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t local_bar, uint32_t rank) {
  const uint32_t remote = map_to_cta(local_bar, rank);
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

struct PairTile {
  int pm, n;   // pair-row block (256 rows), column tile (256 columns)
};

template <typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
pt_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_c,
               const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  const uint32_t cstage_base = smem_base + kPStages * kPStageBytes;
  uint8_t* misc = smem_al + kPStages * kPStageBytes + kPStagingBytes;
  const uint32_t bar_base = smem_base + kPStages * kPStageBytes + kPStagingBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };   // own loads landed (leader: and the peer's)
  auto sfree_bar = [&](int s) { return bar_base + 8u * (2 * kPStages + s); };        // stage consumed
  auto tfull_bar = [&](int b) { return bar_base + 8u * (3 * kPStages + b); };        // tile accumulated
  auto tempty_bar = [&](int b) { return bar_base + 8u * (3 * kPStages + kPAccBufs + b); };  // leader: drained
  const uint32_t cfull_bar = bar_base + 8u * (3 * kPStages + 2 * kPAccBufs);
  const uint32_t cfree_bar = cfull_bar + 8u;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(misc + 512);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 516);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(full_bar(s), leader ? 2 : 1);   // leader: + the peer relay's arrival
      mbar_init(sfree_bar(s), 1);
    }
    for (int b = 0; b < kPAccBufs; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 2 * kPEpiWarps);   // the epilogue warps of both CTAs
    }
    mbar_init(cfull_bar, kPEpiWarps);
    mbar_init(cfree_bar, 1);
    *abort_flag = 0;
    fence_proxy_async_smem();
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anybody signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int KB = p.K / kPBK;
  const int num_pm = (p.M + 255) / 256;
  const int num_n = p.N / 256;
  const int total = num_pm * num_n;
  const int pair = static_cast<int>(blockIdx.x >> 1);
  const int npairs = static_cast<int>(gridDim.x >> 1);
  const int gm = (p.group_m > 0 && p.group_m < num_pm) ? p.group_m : num_pm;
  auto decode = [&](int t) {
    PairTile o;
    const int per_group = gm * num_n;
    const int g = t / per_group;
    const int r = t - g * per_group;
    const int rows_here = min(gm, num_pm - g * gm);
    o.n = r / rows_here;
    o.pm = g * gm + (r - o.n * rows_here);
    return o;
  };

  if (warp < 4) {
    reg_dealloc<40>();
    if (warp == 0 && lane == 0) {
      // ---------------- producer: this CTA's 128 rows of A and its half of the weight tile ----------------
      uint32_t it = 0;
      bool alive = true;
      for (int t = pair; t < total && alive; t += npairs) {
        const PairTile tl = decode(t);
        const int row0 = tl.pm * 256 + static_cast<int>(rank) * 128;
        const uint8_t* wsrc = p.b + static_cast<size_t>(tl.n * 256 + static_cast<int>(rank) * 128) * kPBK;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kPStages;
          if (!mbar_wait(sfree_bar(s), ((it / kPStages) & 1) ^ 1, abort_flag, p.err, kErrWaitSmemEmpty)) {
            alive = false;
            break;
          }
          const uint32_t sa = smem_base + s * kPStageBytes;
          mbar_arrive_expect_tx(full_bar(s), kPStageBytes);
          tma_load_2d(sa, &tmap_a, kb * kPBK, row0, full_bar(s));
          bulk_load(sa + 128 * kPBK, wsrc + static_cast<size_t>(kb) * p.N * kPBK, 128 * kPBK, full_bar(s));
        }
      }
    } else if (warp == 1 && lane == 0 && leader) {
      // ---------------- MMA issuer (leader): 256 x 256 x 32 over both CTAs ----------------
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(256, 256);
      uint32_t it = 0, tiles = 0;
      bool alive = true;
      for (int t = pair; t < total && alive; t += npairs, ++tiles) {
        const int buf = static_cast<int>(tiles % kPAccBufs);
        if (!mbar_wait(tempty_bar(buf), ((tiles / kPAccBufs) & 1) ^ 1, abort_flag, p.err, kErrWaitTmemEmpty)) break;
        const uint32_t d = tmem_base + buf * 256;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kPStages;
          const uint32_t ph = (it / kPStages) & 1;
          const uint32_t sa = smem_base + s * kPStageBytes;
          const uint64_t adesc = umma_desc_sw128(sa);
          const uint64_t bdesc = umma_desc_sw128(sa + 128 * kPBK);
          // one barrier per stage collects both CTAs' operands: the leader's own loads (its
          // producer's arrival + their bytes) and the peer relay's arrival
          if (!mbar_wait(full_bar(s), ph, abort_flag, p.err, kErrWaitSmemFull)) {
            alive = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kPBK / 32; ++k)
            tc_mma_f8_2(d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) ? 1u : 0u);
          tc_commit2(sfree_bar(s));   // the stage may be refilled (the relay tells the peer)
        }
        if (!alive) break;
        tc_commit2(tfull_bar(buf));   // the tile is complete in both CTAs' tensor memory
      }

    } else if (warp == 2 && lane == 0) {
      // ---------------- store thread: staged half tiles -> TMA stores ----------------
      uint32_t n = 0;
      bool ok = true;
      for (int t = pair; t < total && ok; t += npairs) {
        const PairTile tl = decode(t);
        const int row0 = tl.pm * 256 + static_cast<int>(rank) * 128;
        for (int h = 0; h < 2; ++h, ++n) {
          if (!mbar_wait(cfull_bar, n & 1, abort_flag, p.err, kErrWaitEpilogue)) {
            ok = false;
            break;
          }
          if (row0 < p.M) {
#pragma unroll
            for (int reg = 0; reg < 2; ++reg)
              tma_store_2d(&tmap_c, cstage_base + reg * kPRegionBytes, tl.n * 256 + h * 128 + reg * 64, row0);
            bulk_commit_group();
            bulk_wait_group_read0();
          }
          mbar_arrive(cfree_bar);
        }
      }
      bulk_wait_group0();
    } else if (warp == 3 && lane == 0 && leader) {
      // ---------------- relay (leader): stage consumed / tile complete -> tell the peer ----------------
      uint32_t it = 0, tiles = 0;
      bool alive = true;
      for (int t = pair; t < total && alive; t += npairs, ++tiles) {
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kPStages;
          if (!mbar_wait(sfree_bar(s), (it / kPStages) & 1, abort_flag, p.err, kErrWaitSmemEmpty)) {
            alive = false;
            break;
          }
          mbar_arrive_remote(sfree_bar(s), 1);
        }
        if (!alive) break;
        const int buf = static_cast<int>(tiles % kPAccBufs);
        if (!mbar_wait(tfull_bar(buf), (tiles / kPAccBufs) & 1, abort_flag, p.err, kErrWaitTmemFull)) break;
        mbar_arrive_remote(tfull_bar(buf), 1);
      }
    } else if (warp == 3 && lane == 0 && !leader) {
      // ---------------- relay (peer): my stage has landed -> tell the leader ----------------
      uint32_t it = 0;
      bool alive = true;
      for (int t = pair; t < total && alive; t += npairs) {
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % kPStages;
          if (!mbar_wait(full_bar(s), (it / kPStages) & 1, abort_flag, p.err, kErrWaitSmemFull)) {
            alive = false;
            break;
          }
          mbar_arrive_remote(full_bar(s), 0);
        }
      }
    }
  } else {
    reg_alloc<232>();
    // ---------------- epilogue: this CTA's 128 rows x 256 columns of the pair's tile ----------------
    const int ew = warp - 4;
    const int quad = ew & 3, half = ew >> 2;
    const int r = quad * 32 + lane;   // row inside the CTA's 128 rows = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t tiles = 0, passes = 0;
    bool alive = true;
    for (int t = pair; t < total && alive; t += npairs, ++tiles) {
      const PairTile tl = decode(t);
      const int buf = static_cast<int>(tiles % kPAccBufs);
      const bool got = mbar_wait(tfull_bar(buf), (tiles / kPAccBufs) & 1, abort_flag, p.err, kErrWaitTmemFull);
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
      const int row = tl.pm * 256 + static_cast<int>(rank) * 128 + r;
      const float sa = row < p.M ? __ldg(p.scale_a + row) : 0.f;
      for (int h = 0; h < 2 && alive; ++h, ++passes) {
        // this thread's 64 columns of the half tile: tile columns h*128 + half*64 ...
        const int cbase = h * 128 + half * 64;
        const float* sbp = p.scale_b + tl.n * 256 + cbase;
        uint32_t v[64];
#pragma unroll
        for (int q = 0; q < 4; ++q) tmem_ld<16>(tmem_base + lane_base + buf * 256 + cbase + q * 16, v + q * 16);
#pragma unroll
        for (int q = 0; q < 4; ++q) tmem_wait_dep<16>(v + q * 16);
        if (h == 1) {
          // both halves have been read: hand the buffer back to the leader's issuer
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (leader) mbar_arrive(tempty_bar(buf));
            else mbar_arrive_remote(tempty_bar(buf), 0);
          }
        }
        if (passes > 0) {
          const bool ok = mbar_wait(cfree_bar, (passes - 1) & 1, abort_flag, p.err, kErrWaitEpilogue);
          if (!__all_sync(0xffffffffu, ok)) {
            alive = false;
            break;
          }
        }
#pragma unroll
        for (int j = 0; j < 64; j += 8) {
          uint32_t w[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float s0 = sa * __ldg(sbp + j + 2 * q);
            const float s1 = sa * __ldg(sbp + j + 2 * q + 1);
            w[q] = pack2(__uint_as_float(v[j + 2 * q]) * s0, __uint_as_float(v[j + 2 * q + 1]) * s1, OutT());
          }
          const int col = half * 64 + j;   // column inside the staged half tile
          const uint32_t addr = cstage_base + (col >> 6) * kPRegionBytes + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                       "r"(w[3])
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(cfull_bar);
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();   // nobody frees tensor memory or leaves while the partner may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

template <typename OutT>
int launch_pair(const CUtensorMap& tmap_a, const CUtensorMap& tmap_c, const PairParams& p, int pairs,
                cudaStream_t stream) {
  auto kern = pt_pair_kernel<OutT>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  FLYB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    FLYB200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPSmem));
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = kPSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  FLYB200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmap_a, tmap_c, p));
  return FLYB200_OK;
}

}  // namespace

// Entry used by flyb200_pertoken_gemm (cfg.path 3, or by default for shapes it is built for):
// N % 256 == 0, K % 128 == 0, M >= 256.
int launch_pertoken_pair_gemm(void* c, const void* a, const void* b_repacked, const float* scale_a,
                              const float* scale_b, int M, int N, int K, int out_dtype, int max_ctas, int group_m,
                              cudaStream_t stream) {
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  PairParams p{};
  p.b = static_cast<const uint8_t*>(b_repacked);
  p.scale_a = scale_a;
  p.scale_b = scale_b;
  p.err = device_error_word();
  if (!p.err) return FLYB200_ERR_CUDA;
  p.M = M; p.N = N; p.K = K;
  p.group_m = group_m / 2;
  int pairs = sms / 2;
  if (max_ctas > 1 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  const long tiles = static_cast<long>((M + 255) / 256) * (N / 256);
  if (tiles < pairs) pairs = static_cast<int>(tiles);
  CUtensorMap tmap_a, tmap_c;
  int rc;
  if ((rc = make_tensor_map_2d(&tmap_a, a, M, K, 1, 128))) return rc;
  if ((rc = make_tensor_map_2d(&tmap_c, c, M, N, 2, 128))) return rc;
  if (out_dtype == FLYB200_BF16) return launch_pair<__nv_bfloat16>(tmap_a, tmap_c, p, pairs, stream);
  return launch_pair<__half>(tmap_a, tmap_c, p, pairs, stream);
}

}  // namespace flyb200
