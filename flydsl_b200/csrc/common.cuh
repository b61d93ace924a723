// Shared device helpers for libflyb200: mbarrier, TMA (bulk and tensor), tcgen05 (TMEM alloc, MMA,
// commit, load) and the bounded-wait / error-word protocol. sm_100a only.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flyb200.h"

namespace flyb200 {

// ---- host-side error plumbing (api.cu) -------------------------------------------------------
int set_error(int status, const char* fmt, ...);
int* device_error_word();  // address of the current device's error word (cached per device)
int sm_count();            // SM count of the current device (cached per device)

#define FLYB200_CUDA_CHECK(expr)                                                               \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      return ::flyb200::set_error(FLYB200_ERR_CUDA, "%s failed: %s", #expr,                    \
                                  cudaGetErrorString(_e));                                     \
  } while (0)

// Device error codes written to the error word (first writer wins).
enum DeviceError : int {
  kErrNone = 0,
  kErrWaitSmemEmpty = 1,  // producer gave up waiting for a free shared-memory stage
  kErrWaitSmemFull = 2,   // MMA issuer gave up waiting for operands
  kErrWaitTmemEmpty = 3,  // MMA issuer gave up waiting for a free accumulator buffer
  kErrWaitTmemFull = 4,   // epilogue gave up waiting for an accumulator
  kErrWaitGather = 5,     // gather warps gave up waiting for a free stage
  kErrWaitEpilogue = 6,   // an epilogue warp gave up waiting for the other epilogue warps
  kErrWaitExchange = 7,   // decode kernel: split-K partials of a cluster neighbour never arrived
  kErrWaitPeer = 8,       // expert-parallel barrier: a peer rank's flag never arrived
};

// ---- shared-memory address / mbarrier --------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Every wait in these kernels is bounded. A role that runs out of patience raises the CTA-wide
// abort flag (shared memory) and records why in the device error word; every other role sees the
// flag on its next wait and leaves its loop, so the CTA reaches its teardown (TMEM release) and the
// context stays usable. The limit is far above any legitimate wait (a whole launch lasts < 10 ms).
constexpr long long kWaitLimitCycles = 1500000000LL;  // ~0.8 s at 1.9 GHz

__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            int* err_word, int code) {
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = 1;
      atomicCAS(err_word, 0, code | (static_cast<int>(blockIdx.x) << 8));
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* err_word, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, err_word, code);
}

// ---- TMA -------------------------------------------------------------------------------------
// 2-D tiled tensor load, completion counted on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}
// Same copy with an L2 eviction policy (from l2_policy_evict_first / createpolicy).
__device__ __forceinline__ void bulk_load_hint(uint32_t dst, const void* src, uint32_t bytes,
                                               uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
          "r"(dst),
      "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
// Ask L2 to fetch [src, src + bytes) from HBM; nothing lands in the SM. 16-byte granularity.
__device__ __forceinline__ void l2_prefetch(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- cp.async (row gather for the MoE stages) --------------------------------------------------
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tcgen05 -----------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, fp8/fp6/fp4 operand kind, one CTA. K = 32 per instruction.
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor: K-major operand, rows of 128 bytes, 128-byte swizzle, 8-row
// groups 1024 bytes apart (tile base 1024-byte aligned). A K step of 32 bytes inside the swizzled
// row is taken by adding 2 (32 >> 4) to the descriptor's address field.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address  [0,14)
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused) [16,30)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset [32,46)
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                      // layout: SWIZZLE_128B
  return d;
}
// Instruction descriptor: e4m3 x e4m3 -> f32, both operands K-major, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3_f32(int m, int n) {
  return (1u << 4)                              // D format f32
         | (0u << 7) | (0u << 10)               // A, B format e4m3
         | (0u << 15) | (0u << 16)              // A, B K-major
         | (static_cast<uint32_t>(n >> 3) << 17)  // N / 8
         | (static_cast<uint32_t>(m >> 4) << 24); // M / 16
}

// TMEM -> registers: thread i of the warp reads lane (base lane + i), N consecutive 32-bit columns.
#define FLYB200_TMEM_LD_X8(taddr, r)                                                             \
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"           \
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),         \
                 "=r"(r[6]), "=r"(r[7])                                                          \
               : "r"(taddr))
#define FLYB200_TMEM_LD_X16(taddr, r)                                                            \
  asm volatile(                                                                                  \
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "                                                  \
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"                          \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),      \
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),  \
        "=r"(r[14]), "=r"(r[15])                                                                 \
      : "r"(taddr))
#define FLYB200_TMEM_LD_X32(taddr, r)                                                            \
  asm volatile(                                                                                  \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                  \
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"                                  \
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"                 \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),      \
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),  \
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),            \
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),            \
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])             \
      : "r"(taddr))

template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t* r) {
  static_assert(N == 8 || N == 16 || N == 32, "chunk width");
  if constexpr (N == 8) FLYB200_TMEM_LD_X8(taddr, r);
  if constexpr (N == 16) FLYB200_TMEM_LD_X16(taddr, r);
  if constexpr (N == 32) FLYB200_TMEM_LD_X32(taddr, r);
}

// tcgen05.wait::ld that also names the loaded registers as read-write operands, so the compiler
// cannot schedule a use of them ahead of the wait.
#define FLYB200_R8(r, o) "+r"(r[o]), "+r"(r[o + 1]), "+r"(r[o + 2]), "+r"(r[o + 3]), "+r"(r[o + 4]), \
                         "+r"(r[o + 5]), "+r"(r[o + 6]), "+r"(r[o + 7])
template <int N>
__device__ __forceinline__ void tmem_wait_dep(uint32_t* r) {
  static_assert(N == 8 || N == 16 || N == 32, "chunk width");
  if constexpr (N == 8)
    asm volatile("tcgen05.wait::ld.sync.aligned;" : FLYB200_R8(r, 0)::"memory");
  if constexpr (N == 16)
    asm volatile("tcgen05.wait::ld.sync.aligned;" : FLYB200_R8(r, 0), FLYB200_R8(r, 8)::"memory");
  if constexpr (N == 32)
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : FLYB200_R8(r, 0), FLYB200_R8(r, 8), FLYB200_R8(r, 16), FLYB200_R8(r, 24)::"memory");
}

// TMA tensor store shared -> global (bulk async-group completion). Clips rows/columns outside the
// tensor. x is the innermost (column) coordinate and must be 16-byte aligned in bytes.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_group_read0() {  // sources may be overwritten
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_group0() {  // writes complete
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// Register re-balancing between warpgroups (producer/MMA warps need few, epilogue warps many).
template <int R>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R));
}
template <int R>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R));
}

// ---- output packing ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack2(float a, float b, __nv_bfloat16) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __half) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace flyb200
