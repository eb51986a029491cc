/*
 * fso_b200: the C ABI of the B200 (sm_100a) MXFP8 dense / MoE path.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream (cudaStream_t passed as void*), launches on
 * that stream and returns without synchronizing. Nothing here allocates device memory: outputs, workspaces and
 * scratch are the caller's. Return value: 0 on success, a positive cudaError_t when a CUDA call failed, a
 * negative FSO_ERR_* code otherwise; fso_b200_last_error() gives the text of the last failure on the calling
 * host thread. A refused call (FSO_ERR_INVALID) has launched nothing.
 *
 * Layouts (identical to the reference's sm_100 forms, python/fish_scales_ops/include/fso/activation_contract.h):
 *   quantized tensor  e4m3 bytes [rows, K], row-major, 16-byte aligned, K % 128 == 0
 *   scale words       int32, align(rows,128) * K/128 of them; word(m, kp) packs the UE8M0 bytes of the 32-element
 *                     blocks 4kp..4kp+3 of row m (lowest block in the lowest byte) and sits at
 *                     ((m/128) * (K/128) + kp) * 128 + (m%32) * 4 + (m%128)/32; the padded rows' words are zero.
 *
 * Each declaration names the reference interface it replaces (path inside the reference project : line).
 */
#ifndef FSO_B200_H
#define FSO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FSO_ERR_INVALID (-1)       /* malformed argument; nothing was launched */
#define FSO_ERR_UNSUPPORTED (-2)   /* this device or shape is not served */
#define FSO_ERR_INTERNAL (-3)

int fso_b200_version(void);
const char* fso_b200_last_error(void);

/* Reads (and clears) the device-side status word of the current device: 0, or the code of a bounded wait that ran
 * out inside a kernel. Synchronizes the device; meant for tests and health checks, never for the hot path. */
int fso_b200_device_status(int* status);

/* Health check of the bounded device-side waits: launches one thread that waits, for at most limit_cycles SM cycles
 * (0 < limit_cycles <= 2e9), on an mbarrier nothing arrives at; when the wait has run out the thread records the
 * status 0x700 (read it with fso_b200_device_status) and the kernel returns. The device context stays usable.
 * No counterpart in the reference, whose device waits are unbounded (e.g. the work-stealing scheduler's spin,
 * csrc/gemm/include/blockscale_gemm/arch/sm100/mxfp8/slot_work_stealing.cuh). */
int fso_b200_selftest_wait_expires(int64_t limit_cycles, void* stream);

/* bf16 [M, K] -> e4m3 [M, K] + scale words (1x32 MXFP8 rule, bit-exact with the reference).
 * interleave_i > 0: x is G stacked [2*I, K] expert matrices in [gate; up] row order and output rows 2j / 2j+1 of
 * each expert take its rows j / I+j (the fused-FC1 weight order).
 * Replaces: op quantize_1x32_packed, csrc/gemm/ops/mxfp8.cu:279-321 -> fp8bs_quantize_1x32_packed,
 * csrc/gemm/ops/quant_kernels.cu:776-820; expert form python/fish_scales_ops/gemm/mxfp8.py:1511-1582. */
int fso_quantize_1x32(const void* x_bf16, void* xq, void* sf, int64_t m, int64_t k, int64_t interleave_i,
                      void* stream);

/* The activation form of fso_quantize_1x32 (no row interleave): the same bytes, and the kernel lets a decode-sized
 * fso_gemm_mxfp8 launched behind it on the stream start loading its weights while it runs (programmatic dependent
 * launch; the GEMM waits for this kernel before it reads xq / sf). Do not use it to produce a tensor that the next
 * kernel on the stream reads as a weight. Replaces: dense_quantize_activation,
 * python/fish_scales_ops/dense/__init__.py:1068-1099 (and the quantize step inside dense_linear, :911-932). */
int fso_quantize_activation_1x32(const void* x, void* xq, void* sf, int64_t m, int64_t k, void* stream);

/* One empty plain launch: everything enqueued before it has completed before anything enqueued after it starts,
 * including kernels that use programmatic dependent launch. fso.dense.prepare_weight ends with it, so that a linear
 * issued right after prepare never reads weight bytes that are still being written.
 * Replaces: _complete_handle, python/fish_scales_ops/dense/__init__.py:605-620. */
int fso_stream_fence(void* stream);

/* The step between the gate_up and the down projection of a SwiGLU MLP: gu bf16 [M, 2*INTER] (columns [0, INTER)
 * gate, [INTER, 2*INTER) up) -> h = silu(gate) * up quantized with the 1x32 rule, xq e4m3 [M, INTER] and sf in the
 * layout of fso_quantize_1x32, without h reaching memory. silu uses the hardware tanh approximation, so the bytes
 * are defined up to that approximation (output tolerance). Launched with programmatic dependent launch like the
 * activation quantizer. gu 32-byte aligned. Replaces: silu_chunk_mul_quantize_1x32,
 * python/fish_scales_ops/gemm/mxfp8.py:216-236 (csrc/gemm/ops/quant_kernels.cu:690-727). */
int fso_silu_mul_quantize_1x32(const void* gu, void* xq, void* sf, int64_t m, int64_t inter, void* stream);

/* Block-FP8 checkpoint (e4m3 [N, K] + one fp32 scale per 128x128 tile, [N/128, K/128]) -> MXFP8: each value is
 * bf16_rne(float(fp8) * scale) and then goes through the 1x32 rule. N % 128 == 0. interleave_i as in
 * fso_quantize_1x32 (stacked experts, I % 128 == 0; the tile scale follows the source row).
 * Replaces: _dequantize_block_fp8 + _requantize_block_fp8, python/fish_scales_ops/dense/__init__.py:422-462,
 * and python/fish_scales_ops/moe/__init__.py:400-407 for experts. */
int fso_requant_bs128_to_mx(const void* wq, const float* s128, void* out_q, void* out_sf, int64_t n, int64_t k,
                            int64_t interleave_i, void* stream);

/* Checkpoint UE8M0 bytes uint8 [G, N, K/32] -> scale words, one atom slab of align(N,128)*K/128 words per group;
 * interleave_i as in fso_quantize_1x32 (applied to the rows of every group).
 * Replaces: _ue8m0_scale_handle, python/fish_scales_ops/gemm/mxfp8.py:718-768. */
int fso_pack_ue8m0(const void* sf_u8, void* out_sf, int64_t g, int64_t n, int64_t k, int64_t interleave_i,
                   void* stream);

/* Dense GEMM D[M, N] (bf16) = A[M, K] * W[N, K]^T over MXFP8 operands with fp32 accumulation.
 * fso_gemm_mxfp8_ws_bytes gives the workspace the split-K route of this shape needs (0 when it takes none);
 * ws may be NULL when that is 0. N % 128 == 0, K % 128 == 0.
 * Replaces: linear_mxfp8_raw, csrc/gemm/ops/mxfp8.cu:432-541 -> launch_sm100_mxfp8_dispatch (mxfp8.cu:48-51) ->
 * gemm_dispatch_sm100_mxfp8, csrc/gemm/include/blockscale_gemm/arch/sm100/mxfp8/dispatch.cuh:1430-1443. */
int fso_gemm_mxfp8_ws_bytes(int64_t m, int64_t n, int64_t k, int64_t* bytes);
/* The route fso_gemm_mxfp8 takes for one shape, as host arithmetic only (no launch, no device needed when
 * sm_count_or_0 > 0; 0 = the current device's SM count): out6 = { 1 when the weight rows sit on MMA-M (decode-sized
 * M), MMA-N tile width, K slices, 128-wide K blocks per slice, 1 when the CTA-pair kernel runs it, output tiles }.
 * The reference decides the same things inside its dispatch cascade and prints them under FSO_PRINT_TILE_INFO
 * (csrc/gemm/include/blockscale_gemm/arch/sm100/mxfp8/dispatch.cuh:1430-1443, grouped_dispatch.cuh:162-176); it has
 * no query of its own. */
int fso_gemm_mxfp8_describe(int64_t m, int64_t n, int64_t k, int64_t sm_count_or_0, int32_t* out6);
int fso_gemm_mxfp8(const void* a, const void* sfa, const void* w, const void* sfw, void* d, int64_t m, int64_t n,
                   int64_t k, void* ws, int64_t ws_bytes, void* stream);

/* fso_gemm_mxfp8 with the dense epilogue applied to the fp32 accumulator (after any split-K sum) before the one
 * rounding: d = bf16( act(acc + bias[n]) + residual[m, n] ). bias bf16 [N] (a +0.0 bias element counts as -0.0, so
 * that a zero bias gives the bytes of no bias), residual bf16 [M, N], either may be NULL; activation 0 = identity,
 * 1 = erf-GELU 0.5 v (1 + erf(v / sqrt 2)) in fp32. With all three absent the call is fso_gemm_mxfp8.
 * Replaces: the DenseEpilogue argument of linear_mxfp8_raw, csrc/gemm/include/blockscale_gemm/common/epilogue.cuh:1-30
 * (python/fish_scales_ops/gemm/_epilogue.py:1-30). */
int fso_gemm_mxfp8_epilogue(const void* a, const void* sfa, const void* w, const void* sfw, void* d, int64_t m,
                            int64_t n, int64_t k, const void* bias, const void* residual, int64_t activation,
                            void* ws, int64_t ws_bytes, void* stream);

/* The same GEMM with its output in the activation contract instead of bf16: out_q e4m3 [M, N] and out_sf the scale
 * words of an [M, N] activation (align(M,128) * N/128 words, rows past M zero), bit for bit what
 * fso_quantize_activation_1x32 gives on the bf16 output of fso_gemm_mxfp8_epilogue(bias, activation): the epilogue
 * rounds act(acc + bias) to bf16 first and then applies the 1x32 rule per row and 32 columns, one launch and no
 * bf16 round trip through memory. Served for the shapes fso_gemm_mxfp8_fuses_quantized_output answers 1 for (normal
 * orientation, no split-K); FSO_ERR_UNSUPPORTED otherwise, and the caller runs the two launches.
 * Replaces: op linear_mxfp8_quantized_raw and its epilogue, csrc/gemm/include/blockscale_gemm/common/epilogue.cuh:14,
 * 47-57, arch/sm100/mxfp8/dense_epi_math.cuh:203-214; python/fish_scales_ops/dense/__init__.py:1004-1047. */
int fso_gemm_mxfp8_fuses_quantized_output(int64_t m, int64_t n, int64_t k, int* yes);
int fso_gemm_mxfp8_quantized(const void* a, const void* sfa, const void* w, const void* sfw, void* out_q, void* out_sf,
    int64_t m, int64_t n, int64_t k, const void* bias, int64_t activation, void* stream);

/* The gate_up projection of a dense SwiGLU MLP with the activation fused into the GEMM: w e4m3 [2I, K] with its rows
 * interleaved (gate_j, up_j adjacent; fso_quantize_1x32 / fso_requant_bs128_to_mx with interleave_i = I produce
 * that order), dq = silu(gate) * up as e4m3 [M, I], sd its scale words (align(M,128) * I/128, rows past M zero), ready
 * to be the activation of the down projection. 2I % 256 == 0.
 * Replaces the two-kernel chain linear_mxfp8 + silu_chunk_mul_quantize_1x32_fp8
 * (python/fish_scales_ops/gemm/mxfp8.py:216-236, csrc/gemm/ops/quant_kernels.cu:690-727) by the dense form of the
 * fused FC1 epilogue (csrc/gemm/include/blockscale_gemm/arch/sm100/mxfp8/fused_swiglu_store.cuh:266-346). */
int fso_gemm_mxfp8_swiglu(const void* a, const void* sfa, const void* w, const void* sfw, void* dq, void* sd, int64_t m,
    int64_t two_i, int64_t k, void* stream);

/* Host-static sizes of one MoE layer call (functions of the argument shapes only).
 * Replaces: _mxfp8_layer_plan / moe_compact_num_blocks, python/fish_scales_ops/gemm/mxfp8.py:1653-1728, 1228-1239. */
typedef struct fso_moe_plan {
    int64_t pairs;          /* tokens * topk */
    int64_t num_blocks;     /* bound on the 128-row blocks in use */
    int64_t rows;           /* rows of every compact intermediate: 128 * (num_blocks + 1) */
    int64_t route_scratch_bytes;   /* scratch fso_moe_route needs (0 for small calls) */
} fso_moe_plan;
int fso_moe_plan_make(int64_t tokens, int64_t topk, int64_t num_experts, fso_moe_plan* plan);

/* Compact routing. ids int32 [tokens * topk]; ids outside [0, E) are skipped (slot -1).
 * masked_m[E] rows per expert; blk0[E+1] exclusive prefix of ceil(rows/128), blk0[E] = blocks in use;
 * slot_of_flat[tokens*topk] = blk0[e]*128 + rank, rank = position among the expert's pairs in ascending flat
 * index (deterministic); blk_expert[num_blocks] expert of each block, -1 past the blocks in use.
 * Replaces: moe_build_routing_compact, csrc/gemm/ops/moe_glue.cu:2651-2823. */
int fso_moe_route(const int32_t* ids, int64_t tokens, int64_t topk, int64_t num_experts, int64_t num_blocks,
                  int32_t* masked_m, int32_t* blk0, int32_t* slot_of_flat, int32_t* blk_expert, void* scratch,
                  int64_t scratch_bytes, void* stream);

/* fso_moe_route for callers that cannot pass scratch memory and must not allocate (an engine that owns all device
 * memory and forbids allocation in its forward pass, code running where cudaMalloc would stall the stream): the
 * scratch is a 256 KiB array inside the library image, resident on every GPU that loads the library. Same outputs,
 * bit for bit, as fso_moe_route. tokens * topk <= 65536, otherwise FSO_ERR_INVALID. The first call on a device looks
 * up the array's device address (make it outside stream capture); calls share the array, so calls that overlap on
 * the GPU race and must be serialized. Allocates nothing. No counterpart in the reference (its routing op allocates
 * through the torch caching allocator). */
int fso_moe_route_noalloc(const int32_t* ids, int64_t tokens, int64_t topk, int64_t num_experts, int64_t num_blocks,
                          int32_t* masked_m, int32_t* blk0, int32_t* slot_of_flat, int32_t* blk_expert, void* stream);

/* Row gather + 1x32 quantize into the compact buffers: row slot_of_flat[i] of hq / sh takes token i / topk.
 * hq e4m3 [rows, H], sh scale words of a [rows, H] tensor. Rows no pair maps to are not written.
 * Replaces: quantize_1x32_grouped_gather_out, csrc/gemm/ops/mxfp8_compact.cu:206. */
int fso_moe_gather_quant(const void* hidden_bf16, const int32_t* slot_of_flat, int64_t tokens, int64_t topk,
                         int64_t h, int64_t rows, void* hq, void* sh, void* stream);

/* Grouped FC1 with the fused SiLU(gate)*up requantize: for every block b in use, rows [128b, 128b+128) of hq times
 * w13[blk_expert[b]]^T (rows interleaved gate/up) -> dq e4m3 [rows, I] + sd scale words of a [rows, I] tensor.
 * Replaces: linear_mxfp8_grouped_compact_swiglu, csrc/gemm/ops/mxfp8_compact.cu:375 (mxfp8.cu:1456). */
int fso_moe_fc1_swiglu(const void* hq, const void* sh, const void* w13, const void* sw13, const int32_t* blk0,
                       const int32_t* blk_expert, int64_t num_experts, int64_t h, int64_t inter, int64_t num_blocks,
                       int64_t rows, void* dq, void* sd, void* stream);

/* Grouped FC2: dq [rows, I] x w2[e]^T -> dn bf16 [rows, H].
 * Replaces: linear_mxfp8_grouped_compact, csrc/gemm/ops/mxfp8_compact.cu:335 (mxfp8.cu:1411). */
int fso_moe_fc2(const void* dq, const void* sd, const void* w2, const void* sw2, const int32_t* blk0,
                const int32_t* blk_expert, int64_t num_experts, int64_t h, int64_t inter, int64_t num_blocks,
                int64_t rows, void* dn, void* stream);

/* The grouped GEMMs of the layer's decode band (1 to 64 tokens), in the swapped orientation: the weight rows of the
 * experts in use on MMA-M, each expert's few routed rows on MMA-N in tiles of 32 / 64, one tile per (block in use,
 * 128 weight rows); nothing is computed for experts no token chose, and every weight byte is streamed once.
 * out = [rows, n_w], fp32 when out_is_f32 != 0 and bf16 otherwise: for FC1 (weight w13 [E, 2I, H], n_w = 2I, k = H)
 * the fp32 gate / up accumulators in the experts' interleaved column order, for FC2 (weight w2 [E, H, I], n_w = H,
 * k = I) the bf16 down projection. Few live tiles and a long K:
 * K is split inside thread-block clusters (one launch, ordered sum). Every host decision is a function of the shapes,
 * tokens and topk. Between the two calls fso_moe_silu_mul_quantize_rows turns FC1's fp32 output gu into FC2's
 * activation: silu(gate) * up with the 1x32 rule, routed rows only.
 * Replaces the compact slot route: ops linear_mxfp8_grouped_compact[_swiglu] below the band rule of
 * python/fish_scales_ops/gemm/mxfp8.py:540-551, kernels csrc/gemm/include/blockscale_gemm/arch/sm100/mxfp8/
 * grouped_slot_dispatch.cuh:1-110, and the unfused FC1 arm silu_chunk_mul_quantize_1x32_grouped_out
 * (csrc/gemm/ops/mxfp8_compact.cu:258, quant_kernels.cu:2131-2251). The reference's single persistent FC1 + FC2
 * kernel (csrc/gemm/ops/mxfp8.cu:1546, slot_moe_scheduler.cuh) is three launches here, chained with programmatic
 * dependent launch. */
int fso_moe_grouped_gemm_decode(const void* act_q, const void* act_sf, const void* weight, const void* sfw,
    const int32_t* masked_m, const int32_t* blk0, const int32_t* blk_expert, int64_t num_experts, int64_t n_w, int64_t k,
    int64_t num_blocks, int64_t rows, void* out, int64_t out_is_f32, int64_t tokens, int64_t topk, void* stream);
int fso_moe_silu_mul_quantize_rows(const void* gu, const int32_t* masked_m, const int32_t* blk0,
    const int32_t* blk_expert, int64_t num_experts, int64_t rows, int64_t inter, void* dq, void* sd, void* stream);

/* out[t] = bf16( sum_j w[t,j] * dn[slot_of_flat[t*topk+j]] (+ bias_scale[t] * bias[t]) ), fp32, j ascending.
 * bias / bias_scale may be NULL. Replaces: moe_combine, csrc/gemm/ops/moe_glue.cu:2908-3016. */
int fso_moe_combine(const void* dn, const int32_t* slot_of_flat, const float* topk_w, const void* bias,
                    const float* bias_scale, void* out, int64_t tokens, int64_t topk, int64_t h, void* stream);

/* Router: logits [M, ld] (bf16 = 0, fp16 = 1, fp32 = 2; expert dimension contiguous) -> topk_ids int32 [M, topk] in
 * descending weight order (ties to the lower expert id), topk_w fp32 [M, topk] = softmax over the selected k
 * (renormalize != 0) or the plain softmax over all experts. Rows at or past *num_token_non_padded (device int32,
 * may be NULL) get the sentinel id num_experts and weight 0; expert_map (device int32 [num_experts + 1], may be
 * NULL) is applied to every id including the sentinel; shared_gate (fp32 [M], may be NULL) = sigmoid of logit
 * column num_experts. num_experts <= 1024, topk <= 8.
 * Replaces: moe_topk_from_logits, csrc/gemm/ops/moe_glue.cu:3074-3152 (kernel :1370-1465). */
int fso_moe_topk_from_logits(const void* logits, int64_t logit_dtype, int64_t m, int64_t num_experts, int64_t ld,
                             int64_t topk, int64_t renormalize, const int32_t* num_token_non_padded,
                             const int32_t* expert_map, int32_t* topk_ids, float* topk_w, float* shared_gate,
                             void* stream);

/* ---- Expert-parallel exchange over peer memory -------------------------------------------------------------------
 * The reference has no communication code: docs/guide.md:139-141 and python/fish_scales_ops/moe/__init__.py:733-739
 * leave sharding and the exchange to the caller. The entry points below have no counterpart there; they serve
 * this library's expert_parallel_layer helper. They never wait on another GPU: a kernel only stores into peer-mapped
 * buffers, and the caller orders the ranks with a stream-ordered collective before anything reads those buffers. */

/* Plan, step 1: rank_mask[t] bit r = token t has a top-k id in rank r's expert range [r * experts_per_rank, (r + 1) *
 * experts_per_rank); row[r] = number of this rank's tokens bound for rank r, row[world] = tokens. world <= 64. */
int fso_ep_plan_count(const int32_t* topk_ids, int64_t tokens, int64_t topk, int64_t experts_per_rank, int64_t world,
                      uint64_t* rank_mask, int64_t* row, void* stream);

/* Plan, step 2, from the all-gathered rows (table[s * (world + 1) + d] = rows rank s sends to rank d): this rank's
 * send list (send_token / send_rank, grouped by destination, tokens ascending; as many entries as the table says this
 * rank sends), send_off [world], dst_base [world], recv_off [world + 1], back_base [world] as the other entry points
 * take them, and slot int32 [tokens, world] = position of (token, rank) in the send list or -1, which is the slot
 * table of the final fso_moe_combine over the returned partial rows. */
int fso_ep_plan_place(const uint64_t* rank_mask, const int64_t* table, int64_t tokens, int64_t world, int64_t rank,
                      int64_t* send_token, int64_t* send_rank, int64_t* send_off, int64_t* dst_base, int64_t* recv_off,
                      int64_t* back_base, int32_t* slot, void* stream);

/* Dispatch: sent row i is token send_token[i] for rank send_rank[i] (rows grouped by rank, group r starting at
 * send_off[r]); it is stored at row dst_base[r] + (i - send_off[r]) of rank r's receive buffers, whose addresses are
 * peer_q[r] (e4m3 [*, H]), peer_w[r] (uint32 scale words [*, H/128], row-major), peer_ids[r] (int32 [*, topk], ids
 * rewritten to r's local expert range, -1 elsewhere) and peer_wt[r] (fp32 [*, topk]). xq / xs are this rank's
 * tokens as fso_quantize_1x32 wrote them. All index arrays are device memory. */
int fso_ep_dispatch_push(const void* xq, const void* xs, const int32_t* topk_ids, const float* topk_w,
                         const int64_t* send_token, const int64_t* send_rank, const int64_t* send_off,
                         const int64_t* dst_base, const uint64_t* peer_q, const uint64_t* peer_w,
                         const uint64_t* peer_ids, const uint64_t* peer_wt, int64_t rows, int64_t topk, int64_t h,
                         int64_t experts_per_rank, void* stream);

/* Received rows (codes [rows_in, H] and scale words [rows_in, H/128], both row-major) -> the compact slot order:
 * the same outputs as fso_moe_gather_quant for rows that were quantized by their sender. */
int fso_moe_gather_rows(const void* rx_q, const void* rx_w, const int32_t* slot_of_flat, int64_t rows_in,
                        int64_t topk, int64_t h, int64_t rows, void* hq, void* sh, void* stream);

/* fso_moe_combine without bias whose output row t goes to row back_base[s] + (t - recv_off[s]) of the bf16 [*, H]
 * buffer at address peer_back[s], s being the source rank with recv_off[s] <= t < recv_off[s + 1] (recv_off has
 * world + 1 entries). top-k <= 8, H a multiple of 64, dn 32-byte aligned. */
int fso_moe_combine_scatter(const void* dn, const int32_t* slot_of_flat, const float* topk_w, int64_t tokens,
                            int64_t topk, int64_t h, const int64_t* recv_off, const int64_t* back_base,
                            const uint64_t* peer_back, int64_t world, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FSO_B200_H */
