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
