// Expert-parallel token exchange over peer memory (NVLink / NVSwitch), one process per GPU.
//
// Every rank owns one device buffer that its peers map (CUDA IPC): a receive area of W x T packed
// token rows, an area of W x T partial output rows, and W barrier flags. One MoE step is then
//
//   plan + push    each source rank writes its token rows STRAIGHT into the destination's receive
//                  area (plain 16-byte peer stores); only rows that are needed travel
//   barrier        flag exchange, bounded spin
//   local experts  sort / gather / two GEMM stages on local memory; the top-k reduce writes each
//                  partial row straight into the back area of the rank that owns the token (peer
//                  stores, issued as soon as this rank is done)
//   barrier
//   sum            each source rank adds its tokens' partial rows from its own back area in rank
//                  order, fp32 (flyb200_ep_combine)
//   (variant: partial rows stay local and the source ranks pull them, flyb200_ep_pull_combine)
//
// so there is no packed send buffer, no receive-side copy and no gathered intermediate, and only the
// rows that are needed cross NVLink. Loads and stores to peer memory are ordinary ld/st; nothing here
// uses multicast or multimem. The reference is single-GPU and has no counterpart.
//
// Row format (as in ep_pack.cu): [H fp8 | H/128 f32 scales | k i32 expert ids | k f32 route weights];
// receive row of (source rank s, slot j) = s*T + j; unused slots carry expert id -1 everywhere.
#include "common.cuh"
#include "ep_plan.cuh"

namespace flyb200 {

constexpr int kMaxPeers = 16;
struct PeerPtrs {
  uint8_t* p[kMaxPeers];
};

// One warp per (destination rank r, slot s).
__global__ void __launch_bounds__(256)
ep_push_kernel(const uint8_t* __restrict__ x, const float* __restrict__ x_scale,
               const int* __restrict__ topk_ids, const float* __restrict__ topk_w,
               const int* __restrict__ src, PeerPtrs peers, long long recv_off, int T, int H, int k, int W,
               int rank) {
  const int nscale = H / 128;
  const int row_bytes = H + 4 * nscale + 8 * k;
  const int lane = threadIdx.x & 31;
  const int warp0 = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int rows = W * T;
  for (int i = warp0; i < rows; i += nwarps) {
    const int r = i / T, s = i - r * T;
    const int t = src[i];
    uint8_t* dst = peers.p[r] + recv_off + (static_cast<size_t>(rank) * T + s) * row_bytes;
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

// Thread r tells rank r "rank `rank` has reached `epoch`" and waits until rank r has said the same.
// Everything this rank wrote before (peer stores of earlier kernels on the stream included) is
// ordered before the flag by the system-scope fence + release; the acquire orders the kernels that
// follow after the peers' writes. The wait is bounded: on expiry the error word is set and the
// kernel returns (what follows then reads incomplete data, but nothing hangs).
__global__ void ep_barrier_kernel(PeerPtrs peers, long long flag_off, int W, int rank, unsigned epoch,
                                  long long limit_cycles, int* err) {
  const int r = threadIdx.x;
  if (r >= W) return;
  __threadfence_system();
  unsigned* remote = reinterpret_cast<unsigned*>(peers.p[r] + flag_off) + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const unsigned* local = reinterpret_cast<const unsigned*>(peers.p[rank] + flag_off) + r;
  const long long t0 = clock64();
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local) : "memory");
    if (static_cast<int>(v - epoch) >= 0) break;
    if (clock64() - t0 > limit_cycles) {
      atomicCAS(err, 0, kErrWaitPeer | (r << 8));
      break;
    }
    __nanosleep(100);
  }
}

// out[t] = sum over ranks r (ascending) of the partial row that rank r computed for token t, read
// from rank r's partial area at row rank*T + slot[t][r]; fp32 accumulate; one 16-byte vector per
// thread, all of a token's loads issued before the first add.
template <typename T_>
__global__ void __launch_bounds__(256)
ep_pull_kernel(PeerPtrs peers, long long part_off, const uint8_t* __restrict__ need,
               const int* __restrict__ slot, T_* __restrict__ out, int T, int W, int H, int rank) {
  constexpr int VEC = 16 / sizeof(T_);
  const int vec_per_row = H / VEC;
  const long long total = static_cast<long long>(T) * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_row);
    const int v = static_cast<int>(i - static_cast<long long>(t) * vec_per_row);
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    for (int r0 = 0; r0 < W; r0 += 8) {
      uint4 raw[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int r = r0 + q;
        raw[q] = make_uint4(0u, 0u, 0u, 0u);
        if (r < W && need[t * W + r]) {
          const T_* base = reinterpret_cast<const T_*>(peers.p[r] + part_off);
          const long long row = static_cast<long long>(rank) * T + slot[t * W + r];
          raw[q] = *reinterpret_cast<const uint4*>(base + row * H + static_cast<long long>(v) * VEC);
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const T_* e = reinterpret_cast<const T_*>(&raw[q]);
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[j] += static_cast<float>(e[j]);
      }
    }
    uint4 o;
    T_* po = reinterpret_cast<T_*>(&o);
#pragma unroll
    for (int j = 0; j < VEC; ++j) po[j] = static_cast<T_>(acc[j]);
    *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H + static_cast<long long>(v) * VEC) = o;
  }
}

// Top-k reduce of the local experts' route rows, written STRAIGHT into the memory of the rank that
// owns the token: row i of this rank's received rows came from source rank i / T, slot i % T; its
// partial sum (the valid routes in slot order, fp32 -- the arithmetic of the masked moe_reduce
// kernel) goes to that rank's back area at row rank*T + slot. Rows without a local route are not
// sent. The source rank then sums its back area locally (flyb200_ep_combine), so the only NVLink
// traffic of the combine is this kernel's stores, issued as soon as a rank finishes its experts.
template <typename T_>
__global__ void __launch_bounds__(256)
ep_reduce_push_kernel(const T_* __restrict__ routes, const uint8_t* __restrict__ valid, PeerPtrs peers,
                      long long back_off, int R, int T, int k, int H, int rank) {
  constexpr int VEC = 16 / sizeof(T_);
  const int vec_per_row = H / VEC;
  const long long total = static_cast<long long>(R) * vec_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx / vec_per_row);
    const int v = static_cast<int>(idx - static_cast<long long>(i) * vec_per_row);
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    bool any = false;
    for (int s = 0; s < k; ++s) {
      if (valid[i * k + s] == 0) continue;
      any = true;
      const uint4 raw = *reinterpret_cast<const uint4*>(
          routes + (static_cast<long long>(i) * k + s) * H + static_cast<long long>(v) * VEC);
      const T_* e = reinterpret_cast<const T_*>(&raw);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] += static_cast<float>(e[j]);
    }
    if (!any) continue;
    uint4 o;
    T_* po = reinterpret_cast<T_*>(&o);
#pragma unroll
    for (int j = 0; j < VEC; ++j) po[j] = static_cast<T_>(acc[j]);
    const int src = i / T, slot = i - src * T;
    T_* dst = reinterpret_cast<T_*>(peers.p[src] + back_off) +
              (static_cast<long long>(rank) * T + slot) * H + static_cast<long long>(v) * VEC;
    *reinterpret_cast<uint4*>(dst) = o;
  }
}

static bool load_peers(const void* const* peers, int W, PeerPtrs& pp) {
  if (!peers || W < 1 || W > kMaxPeers) return false;
  for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = nullptr;
  for (int i = 0; i < W; ++i) {
    if (!peers[i] || reinterpret_cast<uintptr_t>(peers[i]) % 16) return false;
    pp.p[i] = static_cast<uint8_t*>(const_cast<void*>(peers[i]));
  }
  return true;
}

}  // namespace flyb200

using namespace flyb200;

extern "C" int flyb200_ep_buffer_create(int64_t bytes, void** ptr_out, void* ipc_handle_out) {
  if (bytes < 1 || !ptr_out || !ipc_handle_out)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_buffer_create: bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
  void* ptr = nullptr;
  FLYB200_CUDA_CHECK(cudaMalloc(&ptr, static_cast<size_t>(bytes)));
  cudaError_t e = cudaMemset(ptr, 0, static_cast<size_t>(bytes));
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) {
    cudaFree(ptr);
    return set_error(FLYB200_ERR_CUDA, "ep_buffer_create: %s", cudaGetErrorString(e));
  }
  memcpy(ipc_handle_out, &h, sizeof(h));
  *ptr_out = ptr;
  return FLYB200_OK;
}

extern "C" int flyb200_ep_buffer_open(const void* ipc_handle, void** ptr_out) {
  if (!ipc_handle || !ptr_out) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_buffer_open: NULL argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  void* ptr = nullptr;
  FLYB200_CUDA_CHECK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr_out = ptr;
  return FLYB200_OK;
}

extern "C" int flyb200_ep_buffer_close(void* opened_ptr) {
  if (!opened_ptr) return FLYB200_OK;
  FLYB200_CUDA_CHECK(cudaIpcCloseMemHandle(opened_ptr));
  return FLYB200_OK;
}

extern "C" int flyb200_ep_buffer_destroy(void* ptr) {
  if (!ptr) return FLYB200_OK;
  FLYB200_CUDA_CHECK(cudaFree(ptr));
  return FLYB200_OK;
}

extern "C" int flyb200_ep_barrier(const void* const* peers, int32_t W, int32_t rank, int64_t flag_off,
                                  uint32_t epoch, int32_t limit_ms, void* stream) {
  PeerPtrs pp;
  if (!load_peers(peers, W, pp) || rank < 0 || rank >= W || flag_off < 0 || flag_off % 16 || limit_ms < 1)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_barrier: bad arguments (at most %d ranks)", kMaxPeers);
  int* err = device_error_word();
  if (!err) return FLYB200_ERR_CUDA;
  const long long limit = static_cast<long long>(limit_ms) * 2000000LL;  // about 2 GHz
  ep_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pp, flag_off, W, rank, epoch, limit,
                                                                         err);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

extern "C" int flyb200_ep_push(const void* x, const float* x_scale, const int32_t* topk_ids,
                               const float* topk_weights, int32_t T, int32_t H, int32_t k, int32_t W,
                               int32_t rank, int32_t experts_per_rank, const void* const* peers,
                               int64_t recv_off, uint8_t* need_out, int32_t* slot_out, int32_t* src_out,
                               void* stream) {
  PeerPtrs pp;
  if (!x || !x_scale || !topk_ids || !topk_weights || !need_out || !slot_out || !src_out ||
      !load_peers(peers, W, pp))
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_push: NULL buffer or more than %d ranks", kMaxPeers);
  if (reinterpret_cast<uintptr_t>(x) % 16 || recv_off < 0 || recv_off % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_push: x and the receive area must be 16-byte aligned");
  if (T < 1 || H < 128 || H % 128 || k < 1 || (8 * k) % 16 || rank < 0 || rank >= W || experts_per_rank < 1 ||
      (H + 4 * (H / 128) + 8 * k) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "ep_push: bad sizes (H %% 128 == 0, k even, packed row H + 4*(H/128) + 8*k a multiple of 16)");
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  ep_plan_kernel<<<W, kPlanThreads, 0, st>>>(topk_ids, T, k, W, experts_per_rank, need_out, slot_out, src_out);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  const int rows = W * T;
  int blocks = (rows + 7) / 8;
  if (blocks > sms * 8) blocks = sms * 8;
  ep_push_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint8_t*>(x), x_scale, topk_ids, topk_weights,
                                         src_out, pp, recv_off, T, H, k, W, rank);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

extern "C" int flyb200_ep_pull_combine(const void* const* peers, int64_t part_off, const uint8_t* need,
                                       const int32_t* slot, void* out, int32_t T, int32_t W, int32_t H,
                                       int32_t rank, int32_t dtype, void* stream) {
  PeerPtrs pp;
  if (!need || !slot || !out || !load_peers(peers, W, pp))
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_pull_combine: NULL buffer or more than %d ranks",
                     kMaxPeers);
  if (reinterpret_cast<uintptr_t>(out) % 16 || part_off < 0 || part_off % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_pull_combine: buffers must be 16-byte aligned");
  if (T < 1 || H < 8 || H % 8 || rank < 0 || rank >= W || (dtype != FLYB200_BF16 && dtype != FLYB200_F16))
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_pull_combine: bad sizes or dtype");
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const long long total = static_cast<long long>(T) * (H / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > static_cast<long long>(sms) * 16) blocks = static_cast<long long>(sms) * 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == FLYB200_BF16)
    ep_pull_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(
        pp, part_off, need, slot, static_cast<__nv_bfloat16*>(out), T, W, H, rank);
  else
    ep_pull_kernel<__half><<<static_cast<int>(blocks), 256, 0, st>>>(
        pp, part_off, need, slot, static_cast<__half*>(out), T, W, H, rank);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}

extern "C" int flyb200_ep_reduce_push(const void* routes, const uint8_t* valid, const void* const* peers,
                                      int64_t back_off, int32_t T, int32_t W, int32_t k, int32_t H,
                                      int32_t rank, int32_t dtype, void* stream) {
  PeerPtrs pp;
  if (!routes || !valid || !load_peers(peers, W, pp))
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_reduce_push: NULL buffer or more than %d ranks", kMaxPeers);
  if (reinterpret_cast<uintptr_t>(routes) % 16 || back_off < 0 || back_off % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_reduce_push: buffers must be 16-byte aligned");
  if (T < 1 || k < 1 || H < 8 || H % 8 || rank < 0 || rank >= W || (dtype != FLYB200_BF16 && dtype != FLYB200_F16))
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "ep_reduce_push: bad sizes or dtype");
  const int sms = sm_count();
  if (sms <= 0) return FLYB200_ERR_CUDA;
  const int R = W * T;
  const long long total = static_cast<long long>(R) * (H / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > static_cast<long long>(sms) * 16) blocks = static_cast<long long>(sms) * 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == FLYB200_BF16)
    ep_reduce_push_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(routes), valid, pp, back_off, R, T, k, H, rank);
  else
    ep_reduce_push_kernel<__half><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const __half*>(routes), valid, pp, back_off, R, T, k, H, rank);
  FLYB200_CUDA_CHECK(cudaGetLastError());
  return FLYB200_OK;
}
