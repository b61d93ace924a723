// Stage 2 of the block-scale MoE in its deterministic "reduce" form as one C-ABI call: the stage-2
// GEMM stores one row per (token, slot) route into a scratch buffer and the top-k reduce adds a
// token's rows in slot order. The reference does the same in Python and allocates the scratch per
// call (_MoeGemm2ReduceWrapper, kernels/moe_blockscale_2stage.py:2642-2737); here the caller owns it.
#include "common.cuh"

using namespace flyb200;

static size_t elem_bytes(int dtype) { return dtype == FLYB200_F32 ? 4 : 2; }

extern "C" size_t flyb200_moe_gemm2_reduce_workspace_bytes(int32_t T, int32_t k, int32_t H,
                                                           int32_t out_dtype) {
  if (T < 0 || k < 0 || H < 0) return 0;
  return static_cast<size_t>(T) * k * H * elem_bytes(out_dtype);
}

extern "C" int flyb200_moe_gemm2_reduce(void* out, const void* a2, const void* w_repacked,
                                        const float* scale_x, const float* scale_w,
                                        const int32_t* sorted_ids, const int32_t* expert_ids,
                                        const float* sorted_weights, const int32_t* num_valid_ids,
                                        const uint8_t* valid_mask, int32_t T, int32_t H, int32_t I,
                                        int32_t num_blocks, int32_t E, int32_t k, int32_t tile_m,
                                        int32_t doweight, int32_t out_dtype,
                                        const flyb200_gemm_cfg* cfg, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  if (out_dtype != FLYB200_BF16 && out_dtype != FLYB200_F16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "moe_gemm2_reduce: out_dtype must be BF16 or F16 (per-route rows are 16-bit)");
  if (!workspace) return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_gemm2_reduce: workspace is NULL");
  if (reinterpret_cast<uintptr_t>(workspace) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT, "moe_gemm2_reduce: workspace must be 16-byte aligned");
  const size_t need = flyb200_moe_gemm2_reduce_workspace_bytes(T, k, H, out_dtype);
  if (workspace_bytes < need)
    return set_error(FLYB200_ERR_WORKSPACE, "moe_gemm2_reduce: workspace has %zu bytes, needs %zu",
                     workspace_bytes, need);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // Without a mask every (token, slot) row is read by the reduce, so rows that no routing block
  // covers must read as zero (the reference wrapper zero-fills for the same reason, :2716-2717).
  if (!valid_mask) FLYB200_CUDA_CHECK(cudaMemsetAsync(workspace, 0, need, st));
  int rc = flyb200_moe_gemm2(workspace, a2, w_repacked, scale_x, scale_w, sorted_ids, expert_ids,
                             sorted_weights, num_valid_ids, T, H, I, num_blocks, E, k, tile_m,
                             doweight, /*accumulate=*/0, out_dtype, cfg, stream);
  if (rc) return rc;
  return flyb200_moe_reduce(workspace, out, valid_mask, T, k, H, out_dtype, stream);
}

// The per-token-scale sibling (scale_x [T*k], scale_w [E*H]); `zero_fill` = 0 skips the clearing of
// the per-route rows when the caller knows that every (token, slot) has a routing position
// (zero_intermediate of the reference's wrapper, kernels/moe_gemm_2stage.py:2689-2780).
extern "C" int flyb200_moe_gemm2_reduce_pertoken(void* out, const void* a2, const void* w_repacked,
                                                 const float* scale_x, const float* scale_w,
                                                 const int32_t* sorted_ids, const int32_t* expert_ids,
                                                 const float* sorted_weights, const int32_t* num_valid_ids,
                                                 const uint8_t* valid_mask, int32_t T, int32_t H, int32_t I,
                                                 int32_t num_blocks, int32_t E, int32_t k, int32_t tile_m,
                                                 int32_t doweight, int32_t out_dtype,
                                                 const flyb200_gemm_cfg* cfg, void* workspace,
                                                 size_t workspace_bytes, int32_t zero_fill, void* stream) {
  if (out_dtype != FLYB200_BF16 && out_dtype != FLYB200_F16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "moe_gemm2_reduce_pertoken: out_dtype must be BF16 or F16 (per-route rows are 16-bit)");
  if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "moe_gemm2_reduce_pertoken: workspace must be non-NULL and 16-byte aligned");
  const size_t need = flyb200_moe_gemm2_reduce_workspace_bytes(T, k, H, out_dtype);
  if (workspace_bytes < need)
    return set_error(FLYB200_ERR_WORKSPACE, "moe_gemm2_reduce_pertoken: workspace has %zu bytes, needs %zu",
                     workspace_bytes, need);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!valid_mask && zero_fill) FLYB200_CUDA_CHECK(cudaMemsetAsync(workspace, 0, need, st));
  int rc = flyb200_moe_gemm2_pertoken(workspace, a2, w_repacked, scale_x, scale_w, sorted_ids, expert_ids,
                                      sorted_weights, num_valid_ids, T, H, I, num_blocks, E, k, tile_m,
                                      doweight, /*accumulate=*/0, out_dtype, cfg, stream);
  if (rc) return rc;
  return flyb200_moe_reduce(workspace, out, valid_mask, T, k, H, out_dtype, stream);
}

// ---------------------------------------------------------------------------------------------
// The same operation for callers that have no way to hand over scratch memory.
//
// Who that is: code that drives this library from a place where it holds no device allocator -- a
// C/C++ serving loop that binds the ABI directly (no PyTorch caching allocator behind it), a plug-in
// callback that is only given its input and output buffers, or a host application that budgets
// device memory up front and forbids cudaMalloc afterwards (cudaMalloc also synchronises the whole
// device, which such a loop cannot afford per step). For them the per-route rows live in a
// fixed-size array that is part of the library image.
//
// Cost and limits: every GPU that loads libflyb200 keeps kStaticScratchBytes of device memory for
// this array until the process exits, used or not. Requests that need more are refused. All calls on
// a device share the one array, so (a) two calls whose kernels may overlap on the GPU (different
// streams, or graphs replayed concurrently) race on it -- keep them on one stream or order them
// yourself; (b) the array still holds the previous call's rows: the part this call reads without
// having written it is cleared first (no mask: the whole [T*k, H] range; with a mask the reduce
// never reads an unwritten row).
constexpr size_t kStaticScratchBytes = 16u << 20;  // 16 MiB: e.g. 1170 (token, slot) rows at H = 7168
static __device__ __align__(256) unsigned char g_gemm2_reduce_scratch[kStaticScratchBytes];

// Device address of the array for the current device. Inside host code the symbol's name is only a
// host-side handle, so the address is asked from the runtime once per device (with that device
// current) and cached. This set-up runs inside the first call on each device; make that first call
// outside any stream capture.
static int static_scratch_ptr(void** out_ptr) {
  constexpr int kMaxDevices = 64;
  static void* cache[kMaxDevices] = {nullptr};
  int dev = 0;
  FLYB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices)
    return set_error(FLYB200_ERR_CUDA, "device index %d out of range", dev);
  if (!cache[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_gemm2_reduce_scratch);
    if (e != cudaSuccess || !ptr)
      return set_error(FLYB200_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed: %s",
                       cudaGetErrorString(e));
    cache[dev] = ptr;
  }
  *out_ptr = cache[dev];
  return FLYB200_OK;
}

extern "C" size_t flyb200_moe_gemm2_reduce_noalloc_max_bytes(void) { return kStaticScratchBytes; }

extern "C" int flyb200_moe_gemm2_reduce_noalloc(
    void* out, const void* a2, const void* w_repacked, const float* scale_x, const float* scale_w,
    const int32_t* sorted_ids, const int32_t* expert_ids, const float* sorted_weights,
    const int32_t* num_valid_ids, const uint8_t* valid_mask, int32_t T, int32_t H, int32_t I,
    int32_t num_blocks, int32_t E, int32_t k, int32_t tile_m, int32_t doweight, int32_t out_dtype,
    const flyb200_gemm_cfg* cfg, void* stream) {
  if (out_dtype != FLYB200_BF16 && out_dtype != FLYB200_F16)
    return set_error(FLYB200_ERR_INVALID_ARGUMENT,
                     "moe_gemm2_reduce_noalloc: out_dtype must be BF16 or F16");
  const size_t need = flyb200_moe_gemm2_reduce_workspace_bytes(T, k, H, out_dtype);
  if (need > kStaticScratchBytes)
    return set_error(FLYB200_ERR_WORKSPACE,
                     "moe_gemm2_reduce_noalloc: T*k*H needs %zu bytes of scratch but the built-in "
                     "array holds %zu; use flyb200_moe_gemm2_reduce with your own workspace",
                     need, kStaticScratchBytes);
  void* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!valid_mask && need) FLYB200_CUDA_CHECK(cudaMemsetAsync(scratch, 0, need, st));
  rc = flyb200_moe_gemm2(scratch, a2, w_repacked, scale_x, scale_w, sorted_ids, expert_ids,
                         sorted_weights, num_valid_ids, T, H, I, num_blocks, E, k, tile_m, doweight,
                         /*accumulate=*/0, out_dtype, cfg, stream);
  if (rc) return rc;
  return flyb200_moe_reduce(scratch, out, valid_mask, T, k, H, out_dtype, stream);
}
