/*
 * flyb200.h — C ABI of libflyb200.so: FP8 (e4m3) block-scale GEMM and two-stage block-scale MoE
 * kernels for NVIDIA B200 (sm_100a).
 *
 * Every entry point
 *   - takes plain device pointers, sizes and a CUDA stream handle (cudaStream_t passed as void*;
 *     NULL = the legacy default stream),
 *   - enqueues work on that stream and returns without synchronising it,
 *   - returns FLYB200_OK (0) or a negative flyb200_status; flyb200_last_error_string() describes
 *     the last failure on the calling thread,
 *   - allocates no device memory (workspaces, where needed, are caller-provided).
 *
 * Each declaration names the interface of the reference project (FlyDSL, paths relative to its
 * root) that it stands in for.
 *
 * Conventions shared by all GEMM entry points (identical to the reference kernels):
 *   activations   fp8 e4m3fn, row-major [rows, K]
 *   act. scales   fp32, TRANSPOSED [K/128, rows]  (one scale per row per 128-wide K block)
 *   weights       fp8 e4m3fn, repacked by flyb200_repack_weight_fp8 (NOT the reference's AMD layout)
 *   weight scales fp32, [ceil(N/128), K/128] row-major (experts concatenated along N)
 *   result        C[m,n] = sum_kb ( sum_{k in kb} A[m,k] * B[n,k] ) * sa[kb,m] * sb[n/128,kb]
 *                 accumulated in fp32, rounded once to the output type.
 */
#ifndef FLYB200_H_
#define FLYB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum flyb200_status {
  FLYB200_OK = 0,
  FLYB200_ERR_INVALID_ARGUMENT = -1, /* null pointer, misaligned pointer, bad size            */
  FLYB200_ERR_UNSUPPORTED = -2,      /* legal in the reference but not built here             */
  FLYB200_ERR_CUDA = -3,             /* a CUDA runtime / driver call failed                   */
  FLYB200_ERR_WORKSPACE = -4,        /* caller workspace too small                            */
  FLYB200_ERR_DEVICE_TIMEOUT = -5    /* a kernel gave up on a bounded wait (device error word) */
} flyb200_status;

typedef enum flyb200_dtype {
  FLYB200_BF16 = 0,
  FLYB200_F16 = 1,
  FLYB200_F32 = 2
} flyb200_dtype;

/* Optional tuning knobs; a NULL pointer or zero fields select the built-in heuristic
 * (role of select_tile_config, tests/kernels/test_blockscale_preshuffle_gemm.py:52-83). */
typedef struct flyb200_gemm_cfg {
  int32_t block_n;  /* MMA N / CTA tile width: 32, 64, 128 or 256; 0 = auto */
  int32_t max_ctas; /* cap on the persistent grid; 0 = one CTA per SM       */
  int32_t path;     /* dense GEMM: 0 = auto, 1 = tiled kernel, 2 = decode kernel (M <= 64).
                     * int4 GEMM: see flyb200_int4_gemm.
                     * MoE stages: bit 0 = activations already in routing order (TMA-fed),
                     *             bit 1 = stage-1 output in routing order                   */
  int32_t split_k;  /* decode kernel: K splits per weight tile (cluster size, 1..8); 0 = auto    */
} flyb200_gemm_cfg;

/* Weight repack [batch, N, K] (row-major fp8 bytes) -> per batch [K/128][N/8][8 rows][128 B], the
 * 128-byte-swizzled K-major shared-memory image that tcgen05.mma consumes, so a CTA fetches a
 * (rows x 128 B) weight tile with one bulk copy. Same byte count in and out. N % 8 == 0,
 * K % 128 == 0. Replaces shuffle_weight (tests/utils.py:76-96). */
int flyb200_repack_weight_fp8(void* dst, const void* src, int64_t batch, int64_t N, int64_t K,
                              void* stream);

/* Dense block-scale GEMM. Replaces the launcher returned by compile_blockscale_preshuffle_gemm
 * (kernels/blockscale_preshuffle_gemm.py:39-52, launch_gemm :842-876, kernel_gemm :161-839).
 * c [M,N] out_dtype (BF16|F16); a [M,K]; b_repacked [N,K] repacked; scale_a_t [K/128, M];
 * scale_b [ceil(N/128), K/128]. Any M >= 1; N % 16 == 0; K % 128 == 0. */
int flyb200_blockscale_gemm(void* c, const void* a, const void* b_repacked, const float* scale_a_t,
                            const float* scale_b, int32_t M, int32_t N, int32_t K,
                            int32_t out_dtype, const flyb200_gemm_cfg* cfg, void* stream);

/* Dense FP8 GEMM with one scale per token and one per output channel:
 * c[m,n] = (sum_k a[m,k] * b[n,k]) * scale_a[m] * scale_b[n], the whole K range accumulated in fp32
 * before scaling. Replaces the launcher returned by compile_preshuffle_gemm_a8 with in_dtype "fp8"
 * (kernels/preshuffle_gemm.py:39-52, launch_gemm :1269-1303, kernel_gemm :206-1266); the contract is
 * run_torch of tests/kernels/test_preshuffle_gemm.py:55-66. c [M,N] out_dtype (BF16|F16); a [M,K];
 * b_repacked [N,K] from flyb200_repack_weight_fp8; scale_a [M]; scale_b [N]. Any M >= 1;
 * N % 16 == 0; K % 128 == 0. cfg: max_ctas; path 0 = auto, 1 = single-CTA tiles, 2 = decode kernel,
 * 3 = CTA pairs (256 x 256 tiles over two SMs; M >= 256, N % 256 == 0; auto takes it from M = 1024);
 * split_k as for flyb200_blockscale_gemm (M <= 64
 * goes to the swap-AB split-K decode kernel when that pays off: there the token's scale rides along
 * every K block and the channel's scale is applied once after the K loop). */
int flyb200_pertoken_gemm(void* c, const void* a, const void* b_repacked, const float* scale_a,
                          const float* scale_b, int32_t M, int32_t N, int32_t K, int32_t out_dtype,
                          const flyb200_gemm_cfg* cfg, void* stream);

/* MoE routing sort. Bit-exact stand-in for moe_sorting_torch_native
 * (tests/kernels/test_moe_gemm.py:97-161) and the sorter half of build_routing_buffers (:223-295).
 * topk_ids i32 [T,k]; topk_weights f32 [T,k]; expert_mask i32 [E] or NULL; num_local_tokens: < 0
 * means all T tokens. Outputs: sorted_ids i32 [T*k + E*block_m - k] = (slot<<24)|token, padding =
 * (k<<24)|T; sorted_weights f32 same length (padding rows get 0.0); sorted_expert_ids i32
 * [ceil(len/block_m)] (-1 beyond the used blocks); num_valid_ids i32 [2] = {padded rows, T}. */
int flyb200_moe_sort(const int32_t* topk_ids, const float* topk_weights, int32_t T, int32_t k,
                     int32_t E, int32_t block_m, const int32_t* expert_mask,
                     int32_t num_local_tokens, int32_t* sorted_ids, float* sorted_weights,
                     int32_t* sorted_expert_ids, int32_t* num_valid_ids, void* stream);

/* flyb200_moe_sort fused with the permute of the activations into routing order (what
 * flyb200_moe_gather_rows does in a second launch): x fp8 [T, K] and x_scale_t f32 [K/128, T] are
 * copied to x_sorted [T*k + E*block_m - k, K] and x_scale_sorted_t [K/128, same rows], row i = the
 * token of sorted position i, zeros on padding rows (rows at or beyond num_valid_ids[0] are left
 * untouched). The reference gathers inside its stage kernels
 * (kernels/moe_blockscale_2stage.py:394-439). K % 128 == 0. */
int flyb200_moe_sort_permute(const int32_t* topk_ids, const float* topk_weights, int32_t T, int32_t k,
                             int32_t E, int32_t block_m, const int32_t* expert_mask,
                             int32_t num_local_tokens, int32_t* sorted_ids, float* sorted_weights,
                             int32_t* sorted_expert_ids, int32_t* num_valid_ids, const void* x,
                             const float* x_scale_t, void* x_sorted, float* x_scale_sorted_t, int32_t K,
                             void* stream);

/* Router: topk_ids[t] = the k experts with the largest logits[t] in descending order (slot order),
 * topk_weights[t] = softmax over those k values. Replaces the reference test's
 * torch.topk + torch.softmax (tests/kernels/test_moe_blockscale.py:228-230). logits f32 [T, E],
 * E <= 1024; ties go to the lower expert id; NaN scores are never selected. */
int flyb200_moe_route_topk(const float* logits, int32_t T, int32_t E, int32_t k, int32_t* topk_ids,
                           float* topk_weights, void* stream);

/* MoE stage 1: gather rows by sorted id, X * W1^T (gate rows [0,I), up rows [I,2I) per expert),
 * out[(t*k+s), col] = silu(gate) * up [* route weight]. Replaces
 * launch_moe_blockscale_gemm1 (kernels/moe_blockscale_2stage.py:1165-1214; factory :74-89).
 * x [T,H]; w repacked [E, 2I, H]; scale_x [H/128, T]; scale_w [E*(2I/128), H/128];
 * out [T,k,I] out_dtype (F16|BF16). tile_m = rows per routing block (<= 128). */
int flyb200_moe_gemm1(void* out, const void* x, const void* w_repacked, const float* scale_x,
                      const float* scale_w, const int32_t* sorted_ids, const int32_t* expert_ids,
                      const float* sorted_weights, const int32_t* num_valid_ids, int32_t T,
                      int32_t I, int32_t H, int32_t num_blocks, int32_t E, int32_t k,
                      int32_t tile_m, int32_t doweight, int32_t out_dtype,
                      const flyb200_gemm_cfg* cfg, void* stream);

/* flyb200_moe_gemm1 with the re-quantisation between the stages fused into its epilogue: instead of
 * the 16-bit out it writes out_q fp8 e4m3fn [rows, I] and out_scale_t f32 [I/128, rows] in routing
 * order (rows = T*k + E*tile_m - k sorted positions) -- bit for bit what flyb200_quant_1x128 makes of
 * the stage-1 output rounded to mid_dtype (F16|BF16), i.e. the reference's host re-quantisation
 * (tests/kernels/test_moe_blockscale.py:346-361) without the intermediate tensor. Needs cfg.path
 * bits 0 and 1 (routing-order input and output); uses 256-wide tiles (128 output columns = one scale
 * group per row). Rows of padding positions are not written. */
int flyb200_moe_gemm1_q8(void* out_q, float* out_scale_t, const void* x, const void* w_repacked,
                         const float* scale_x, const float* scale_w, const int32_t* sorted_ids,
                         const int32_t* expert_ids, const float* sorted_weights,
                         const int32_t* num_valid_ids, int32_t T, int32_t I, int32_t H,
                         int32_t num_blocks, int32_t E, int32_t k, int32_t tile_m, int32_t doweight,
                         int32_t mid_dtype, const flyb200_gemm_cfg* cfg, void* stream);

/* MoE stage 2: gather rows (t*k+s) of a2, A2 * W2^T, [* route weight], then either atomically add
 * into out[t, col] (accumulate != 0; caller zeroes out) or store to out[(t*k+s), col]. Replaces
 * launch_moe_blockscale_gemm2 (kernels/moe_blockscale_2stage.py:2390-2440; factory :1219-1238).
 * a2 [T*k, I]; w repacked [E, H, I]; scale_x [I/128, T*k]; scale_w [E*(H/128), I/128];
 * out out_dtype (F16|BF16|F32). */
int flyb200_moe_gemm2(void* out, const void* a2, const void* w_repacked, const float* scale_x,
                      const float* scale_w, const int32_t* sorted_ids, const int32_t* expert_ids,
                      const float* sorted_weights, const int32_t* num_valid_ids, int32_t T,
                      int32_t H, int32_t I, int32_t num_blocks, int32_t E, int32_t k,
                      int32_t tile_m, int32_t doweight, int32_t accumulate, int32_t out_dtype,
                      const flyb200_gemm_cfg* cfg, void* stream);

/* The two MoE stages with per-token activation scales and per-channel weight scales (fp8 operands):
 * replace launch_moe_gemm1 (kernels/moe_gemm_2stage.py:1215-1262; factory :93-107) and launch_moe_gemm2
 * (kernels/moe_gemm_2stage.py:2431-2478; factory :1267-1282) for in_dtype "fp8". Arguments as in
 * flyb200_moe_gemm1 / flyb200_moe_gemm2 except the scales: scale_x one f32 per activation row ([T]
 * for stage 1; [T*k], row t*k+s, for stage 2 -- or one per routing-order row with cfg.path bit 0),
 * scale_w one f32 per output channel of every expert ([E*2I], gate channels then up channels per
 * expert, for stage 1; [E*H] for stage 2). The whole K range of a tile is accumulated in tensor
 * memory and scaled once. cfg.block_n must be 0 or 256. */
int flyb200_moe_gemm1_pertoken(void* out, const void* x, const void* w_repacked, const float* scale_x,
                               const float* scale_w, const int32_t* sorted_ids, const int32_t* expert_ids,
                               const float* sorted_weights, const int32_t* num_valid_ids, int32_t T,
                               int32_t I, int32_t H, int32_t num_blocks, int32_t E, int32_t k,
                               int32_t tile_m, int32_t doweight, int32_t out_dtype,
                               const flyb200_gemm_cfg* cfg, void* stream);
int flyb200_moe_gemm2_pertoken(void* out, const void* a2, const void* w_repacked, const float* scale_x,
                               const float* scale_w, const int32_t* sorted_ids, const int32_t* expert_ids,
                               const float* sorted_weights, const int32_t* num_valid_ids, int32_t T,
                               int32_t H, int32_t I, int32_t num_blocks, int32_t E, int32_t k,
                               int32_t tile_m, int32_t doweight, int32_t accumulate, int32_t out_dtype,
                               const flyb200_gemm_cfg* cfg, void* stream);
/* Per-token stage 2 in reduce mode: per-route rows into `workspace` (cleared first when there is no
 * mask and zero_fill != 0), then the top-k reduction: the wrapper of compile_moe_gemm2_ex(mode=
 * "reduce") (kernels/moe_gemm_2stage.py:2689-2780). workspace as for flyb200_moe_gemm2_reduce. */
int flyb200_moe_gemm2_reduce_pertoken(void* out, const void* a2, const void* w_repacked,
                                      const float* scale_x, const float* scale_w,
                                      const int32_t* sorted_ids, const int32_t* expert_ids,
                                      const float* sorted_weights, const int32_t* num_valid_ids,
                                      const uint8_t* valid_mask, int32_t T, int32_t H, int32_t I,
                                      int32_t num_blocks, int32_t E, int32_t k, int32_t tile_m,
                                      int32_t doweight, int32_t out_dtype, const flyb200_gemm_cfg* cfg,
                                      void* workspace, size_t workspace_bytes, int32_t zero_fill,
                                      void* stream);

/* Y[t,d] = sum_s X[t,s,d] (fp32 accumulate, slot order 0..k-1), optional u8 mask [T,k].
 * Replaces the launcher of compile_moe_reduction (kernels/moe_blockscale_2stage.py:2446-2638). */
int flyb200_moe_reduce(const void* x, void* y, const uint8_t* valid_mask, int32_t T, int32_t k,
                       int32_t H, int32_t dtype, void* stream);

/* Stage 2 in its deterministic "reduce" form as one call: the GEMM stores one row per (token, slot)
 * route into `workspace` ([T*k, H] of out_dtype, BF16|F16), then the top-k reduce adds a token's
 * rows in slot order into out [T, H]. valid_mask u8 [T,k] or NULL (NULL: the workspace is zeroed
 * first). Replaces _MoeGemm2ReduceWrapper.__call__ (kernels/moe_blockscale_2stage.py:2642-2737),
 * which allocates that intermediate itself on every call; here the caller owns it. */
int flyb200_moe_gemm2_reduce(void* out, const void* a2, const void* w_repacked,
                             const float* scale_x, const float* scale_w, const int32_t* sorted_ids,
                             const int32_t* expert_ids, const float* sorted_weights,
                             const int32_t* num_valid_ids, const uint8_t* valid_mask, int32_t T,
                             int32_t H, int32_t I, int32_t num_blocks, int32_t E, int32_t k,
                             int32_t tile_m, int32_t doweight, int32_t out_dtype,
                             const flyb200_gemm_cfg* cfg, void* workspace, size_t workspace_bytes,
                             void* stream);

/* Bytes flyb200_moe_gemm2_reduce needs in `workspace`: T*k*H*sizeof(out_dtype). */
size_t flyb200_moe_gemm2_reduce_workspace_bytes(int32_t T, int32_t k, int32_t H, int32_t out_dtype);

/* flyb200_moe_gemm2_reduce for callers that cannot supply scratch memory (no counterpart in the
 * reference, whose wrapper simply allocates): a bare C/C++ serving loop or plug-in callback that
 * holds no device allocator, or a host that forbids cudaMalloc after start-up. The per-route rows go
 * to a fixed array inside the library image instead of `workspace`; the call allocates nothing.
 *   - Limit: T*k*H*sizeof(out_dtype) <= flyb200_moe_gemm2_reduce_noalloc_max_bytes() (16 MiB);
 *     larger requests return FLYB200_ERR_WORKSPACE. Every GPU that loads the library holds those
 *     16 MiB until the process exits.
 *   - The array is shared by all calls on a device: calls whose kernels can overlap on the GPU race
 *     on it; serialise them. Stale rows of an earlier call are cleared where this call would read
 *     them.
 *   - The first call on each device looks up the array's device address; make that first call
 *     outside any stream capture.
 * Arguments and result are those of flyb200_moe_gemm2_reduce without workspace/workspace_bytes. */
int flyb200_moe_gemm2_reduce_noalloc(void* out, const void* a2, const void* w_repacked,
                                     const float* scale_x, const float* scale_w,
                                     const int32_t* sorted_ids, const int32_t* expert_ids,
                                     const float* sorted_weights, const int32_t* num_valid_ids,
                                     const uint8_t* valid_mask, int32_t T, int32_t H, int32_t I,
                                     int32_t num_blocks, int32_t E, int32_t k, int32_t tile_m,
                                     int32_t doweight, int32_t out_dtype,
                                     const flyb200_gemm_cfg* cfg, void* stream);

/* Size of the built-in scratch array used by flyb200_moe_gemm2_reduce_noalloc, in bytes. */
size_t flyb200_moe_gemm2_reduce_noalloc_max_bytes(void);

/* 1x128 group quantiser: x [rows, cols] (in_dtype) -> q fp8 e4m3fn [rows, cols] and
 * scale_t f32 [cols/128, rows]; scale = amax/448 (0 -> 1). Replaces the host re-quantisation between
 * the MoE stages (tests/kernels/test_moe_blockscale.py:346-361, pertoken_quant tests/utils.py:29-73). */
int flyb200_quant_1x128(const void* x, void* q, float* scale_t, int64_t rows, int32_t cols,
                        int32_t in_dtype, void* stream);

/* Activations into routing order (a helper with no reference counterpart: the reference gathers rows
 * inside its stage kernels, kernels/moe_blockscale_2stage.py:394-439). Row i < num_valid_ids[0] of
 * x_out is the source row of sorted position i -- token t (by_slot = 0) or route t*topk+slot
 * (by_slot != 0) -- zero for padding; scale_out_t [K/128, rows_out] likewise. x [rows_in, K] fp8,
 * scale_t [K/128, rows_in]. With inputs prepared this way flyb200_moe_gemm1/2 take cfg.path bit 0
 * (A fetched by TMA) and stage 1 may write in routing order with cfg.path bit 1. */
int flyb200_moe_gather_rows(const void* x, const float* scale_t, const int32_t* sorted_ids,
                            const int32_t* num_valid_ids, void* x_out, float* scale_out_t,
                            int32_t rows_in, int32_t K, int32_t topk, int32_t rows_out,
                            int32_t by_slot, void* stream);
/* The same permutation for the per-token-scale MoE: ONE scale per row, scale [rows_in] ->
 * scale_out [rows_out] (K a multiple of 16). */
int flyb200_moe_gather_rows_pertoken(const void* x, const float* scale, const int32_t* sorted_ids,
                                     const int32_t* num_valid_ids, void* x_out, float* scale_out,
                                     int32_t rows_in, int32_t K, int32_t topk, int32_t rows_out,
                                     int32_t by_slot, void* stream);

/* Whole-row quantiser, bit for bit the reference's pertoken_quant (tests/utils.py:29-73) on 16-bit
 * rows: scale[r] = amax(|x[r, :]|)/448 (0 -> 1; NaN -> 0 and +-Inf -> +-448 first), q = x/scale as
 * fp8 e4m3. It is what the reference test runs on the host between the stages of the per-token-scale
 * MoE (tests/kernels/test_moe_gemm.py:1296-1300). x [rows, cols] in_dtype (F16|BF16), cols % 8 == 0;
 * num_rows_dev (may be NULL): device int32 holding the number of leading rows to process, at most
 * `rows` (the padded route count of the sorter). */
int flyb200_quant_pertoken(const void* x, void* q, float* scale, const int32_t* num_rows_dev,
                           int64_t rows, int32_t cols, int32_t in_dtype, void* stream);

/* flyb200_quant_1x128 over the first num_rows_dev[0] rows only (row count known on the device, e.g.
 * the sorter's padded route count); scale_t is [cols/128, rows_alloc]. Input BF16|F16. */
int flyb200_quant_1x128_devrows(const void* x, void* q, float* scale_t, const int32_t* num_rows_dev,
                                int64_t rows_alloc, int32_t cols, int32_t in_dtype, void* stream);

/* Expert-parallel dispatch preparation (new multi-GPU layer, no reference counterpart). For local
 * tokens x [T,H] fp8 with token-major scales x_scale [T,H/128], topk_ids i32 [T,k], topk_weights f32
 * [T,k] and W ranks owning experts_per_rank consecutive experts each: need_out u8 [T,W] (token t
 * visits rank r), slot_out i32 [T,W] (its row slot inside rank r's block), src_out i32 [W*T] (token
 * feeding each send row, -1 = unused) and the packed send buffer send_out [W*T, H + 4*H/128 + 8*k]
 * bytes = [fp8 row | scales | expert ids | route weights], unused rows with ids -1. k must be even. */
int flyb200_ep_plan_pack(const void* x, const float* x_scale, const int32_t* topk_ids,
                         const float* topk_weights, int32_t T, int32_t H, int32_t k, int32_t W,
                         int32_t experts_per_rank, uint8_t* need_out, int32_t* slot_out,
                         int32_t* src_out, void* send_out, void* stream);

/* Expert-parallel receive side: flyb200_moe_gather_rows reading straight from a packed receive
 * buffer (rows_in rows in the flyb200_ep_plan_pack row format) -- x_out [rows_out, H] in routing
 * order, scale_out_t [H/128, rows_out]. No reference counterpart. */
int flyb200_ep_gather_packed(const void* packed, const int32_t* sorted_ids,
                             const int32_t* num_valid_ids, void* x_out, float* scale_out_t,
                             int32_t rows_in, int32_t H, int32_t k, int32_t rows_out, void* stream);

/* Expert-parallel receive side: the [rows, k] expert ids and route weights of a packed receive buffer
 * as dense tensors, plus valid[r][j] = 1 iff that expert lives on `rank` (ids / experts_per_rank ==
 * rank; -1 marks an unused slot) -- the sorter's inputs and the valid_mask of flyb200_moe_reduce.
 * local_ids != 0: ids_out holds ids relative to the rank's first expert and -1 for every route that
 * is not this rank's, so that the sort runs over experts_per_rank experts. No reference counterpart. */
int flyb200_ep_unpack_meta(const void* packed, int32_t rows, int32_t H, int32_t k,
                           int32_t experts_per_rank, int32_t rank, int32_t local_ids,
                           int32_t* ids_out, float* weights_out, uint8_t* valid_out, void* stream);

/* Expert-parallel final sum: out[t] = sum over ranks r, ascending, of back[r*T + slot[t][r]] where
 * need[t][r] (fp32 accumulate; back/out BF16|F16 [*, H]). No reference counterpart. */
int flyb200_ep_combine(const void* back, const uint8_t* need, const int32_t* slot, void* out, int32_t T,
                       int32_t W, int32_t H, int32_t dtype, void* stream);

/* ---- Expert-parallel exchange over peer memory (one process per GPU, NVLink). No reference
 * counterpart: the reference is single-GPU. Every rank creates one exchange buffer, passes the 64-byte
 * handle to its peers (any host channel) and opens theirs; peers[r] below is rank r's buffer as mapped
 * in THIS process (peers[rank] = the own buffer). These four calls allocate / map device memory and
 * belong at start-up. ---- */
int flyb200_ep_buffer_create(int64_t bytes, void** ptr_out, void* ipc_handle_out /* 64 bytes */);
int flyb200_ep_buffer_open(const void* ipc_handle, void** ptr_out);
int flyb200_ep_buffer_close(void* opened_ptr);
int flyb200_ep_buffer_destroy(void* ptr);

/* All-rank barrier on the stream: flags (W x u32, zero at creation) live at flag_off in every buffer;
 * epoch must grow by one per call, the same on every rank. A rank waits at most limit_ms for each
 * peer, then records FLYB200_ERR_DEVICE_TIMEOUT in the device error word and goes on. */
int flyb200_ep_barrier(const void* const* peers, int32_t W, int32_t rank, int64_t flag_off,
                       uint32_t epoch, int32_t limit_ms, void* stream);

/* flyb200_ep_plan_pack whose rows go straight into the destinations' receive areas (at recv_off in
 * each buffer; row of (source rank s, slot j) = s*T + j) instead of a send buffer. */
int flyb200_ep_push(const void* x, const float* x_scale, const int32_t* topk_ids,
                    const float* topk_weights, int32_t T, int32_t H, int32_t k, int32_t W, int32_t rank,
                    int32_t experts_per_rank, const void* const* peers, int64_t recv_off,
                    uint8_t* need_out, int32_t* slot_out, int32_t* src_out, void* stream);

/* flyb200_ep_combine reading each partial row from the rank that computed it: rank r's partial area
 * (at part_off in its buffer, [W*T, H] BF16|F16) holds the row of this rank's token t at
 * rank*T + slot[t][r]. */
int flyb200_ep_pull_combine(const void* const* peers, int64_t part_off, const uint8_t* need,
                            const int32_t* slot, void* out, int32_t T, int32_t W, int32_t H, int32_t rank,
                            int32_t dtype, void* stream);

/* ---- Weight-only int4 x bf16 GEMM for decode-size M (the "dequantise, then matmul" contract; the
 * reference has no kernel of this exact format -- nearest: the W4A16 path of
 * kernels/moe_gemm_2stage.py:607-630 and the int4 unpack of kernels/mfma_preshuffle_pipeline.py:202-222). ---- */

/* q int8 [N, K] with values in [-8, 7] and scales bf16 [N, K/128] -> wq_out uint8
 * [K/128][N/8][4][8][16]: per 128-K group and block of 8 rows, four 16-byte chunks (32 K elements
 * each), each chunk holding its 8 rows back to back (nibble = q + 8; the eight nibbles of a 32-bit
 * word hold K elements e0 e2 e4 e6 e1 e3 e5 e7), and scales_t_out bf16 [K/128][N].
 * K % 128 == 0, N % 8 == 0. */
int flyb200_int4_repack(const int8_t* q, const void* scales, int32_t N, int32_t K, void* wq_out,
                        void* scales_t_out, void* stream);

/* c bf16 [M, N] = a bf16 [M, K] * dequant(W)^T, W as produced by flyb200_int4_repack; fp32
 * accumulation, the group scale applied per 128-K group in fp32. 1 <= M <= 64; N, K % 128 == 0.
 * cfg (optional): split_k forces the split-K factor (cluster size, 1..8); path picks the kernel:
 * 1 = weights unpacked in registers and fed to mma.sync (faster up to 32 tokens), 2 = weights
 * unpacked through shared memory for tcgen05.mma, 0 = by token count. Same arithmetic either way. */
int flyb200_int4_gemm(void* c, const void* a, const void* wq, const void* scales_t, int32_t M, int32_t N,
                      int32_t K, const flyb200_gemm_cfg* cfg, void* stream);

/* Masked top-k reduce of the local experts' route rows (the arithmetic of flyb200_moe_reduce with a
 * valid_mask) whose result rows go straight into the owners' memory: row i of routes' [W*T, k, H]
 * belongs to source rank i / T, slot i % T and is stored at row rank*T + slot of that rank's back area
 * (back_off in its buffer, [W*T, H]). Rows without a valid route are not sent. The owner then calls
 * flyb200_ep_combine on its own back area. */
int flyb200_ep_reduce_push(const void* routes, const uint8_t* valid, const void* const* peers,
                           int64_t back_off, int32_t T, int32_t W, int32_t k, int32_t H, int32_t rank,
                           int32_t dtype, void* stream);

/* Reads and clears the device error word of the current device after synchronising `stream`.
 * *code_out = 0 when no kernel reported a problem. The reference only prints GPU errors
 * (lib/Runtime/FlyRocmRuntimeWrappers.cpp:22-30); this is the status-returning equivalent. */
int flyb200_query_device_error(void* stream, int32_t* code_out);

/* Text for the last non-OK status returned on this thread ("" if none). */
const char* flyb200_last_error_string(void);

/* Library version, major*10000 + minor*100 + patch. */
int flyb200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FLYB200_H_ */
