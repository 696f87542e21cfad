/*
 * C ABI of libmegamoe_b200.so -- the B200 (sm_100a) implementation of the W8A8 channelwise Mega MoE layer.
 *
 * These entry points are what a binding of the reference's `megamoe._C` extension module would call for this
 * path; each comment names the reference interface it replaces (paths relative to the reference project).
 * Plain pointers and integers only: no torch types, no C++ exceptions.  Every function returns 0 on success
 * and a non-zero code on failure; mm_last_error() then returns a message (thread-local, valid until the next
 * call on the same thread).  All device work is enqueued on `stream` (a cudaStream_t passed as void*) and the
 * call returns without synchronising, unless stated otherwise.
 */
#ifndef MEGAMOE_B200_H
#define MEGAMOE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MM_ABI_MAX_RANKS 16

/* indices into the `offsets` array filled by mm_symm_buffer_layout */
enum {
    MM_SYM_PEER_PTRS = 0, MM_SYM_SIGNALS, MM_SYM_RUNTIME_NUM_TOKENS, MM_SYM_COUNT_MATRIX,
    MM_SYM_X, MM_SYM_X_SF, MM_SYM_TOPK_IDX, MM_SYM_TOPK_WEIGHTS,
    MM_SYM_POOL_X, MM_SYM_POOL_META, MM_SYM_COMBINE, MM_SYM_POOL_ROWS, MM_SYM_NUM_OFFSETS
};
/* indices into the `offsets` array filled by mm_scratch_layout */
enum {
    MM_SCR_STATUS = 0, MM_SCR_EPOCH, MM_SCR_PLAN, MM_SCR_BLOCK_COUNTS, MM_SCR_DEST_BASE, MM_SCR_EXPERT_TOTAL,
    MM_SCR_EXPERT_OFF, MM_SCR_MBLOCK_EXPERT, MM_SCR_MBLOCK_VALID, MM_SCR_DEST_ROW, MM_SCR_ROW_AMAX,
    MM_SCR_ACT_SCALE, MM_SCR_ACT_BF16, MM_SCR_ACT_FP8, MM_SCR_SEND_BASE, MM_SCR_SEND_LIST, MM_SCR_L1_DONE, MM_SCR_L2_READY,
    MM_SCR_GRID_SYNC, MM_SCR_ACT_SF, MM_SCR_ROUTE_BLOCKS, MM_SCR_NUM_OFFSETS
};
/* stages of one staged layer call, in launch order (indices of mm_get_stage_times) */
enum {
    MM_STAGE_ROUTE_COUNT = 0, MM_STAGE_ROUTE_EXCHANGE, MM_STAGE_ROUTE_PLAN, MM_STAGE_DISPATCH, MM_STAGE_BARRIER_DISPATCH,
    MM_STAGE_GEMM1, MM_STAGE_REQUANT, MM_STAGE_GEMM2, MM_STAGE_BARRIER_COMBINE, MM_STAGE_REDUCE,
    MM_STAGE_FUSED /* the single launch of MM_MODE_FUSED */, MM_NUM_STAGES
};
/* execution variants of mm_fp8_w8a8_mega_moe */
enum { MM_MODE_STAGED = 0, MM_MODE_FUSED = 1, MM_MODE_STAGED_SPLIT = 2, MM_MODE_STAGED_UE8M0 = 3 };

/* Message of the last failure on this thread. */
const char* mm_last_error(void);

/* Token-count alignment of the symmetric buffer (384).
 * Replaces get_token_alignment_for_mega_moe, csrc/apis/mega_dcu.hpp:24-26. */
int mm_token_alignment(void);

/* Byte offsets of every region of the symmetric buffer and its total size.
 * Replaces get_symm_buffer_size_for_mega_moe and its slice function, csrc/apis/mega_dcu.hpp:93-154.
 * R ranks, E experts in total, T max tokens per rank, K top-k, H hidden, I intermediate. */
int mm_symm_buffer_layout(int R, int E, int T, int K, int H, int I, int64_t* offsets, int64_t* total_bytes);

/* Byte offsets of every region of the local (non-symmetric) scratch buffer and its total size.
 * Replaces get_mega_moe_route_scratch_size_for_mega_moe, csrc/apis/mega_dcu.hpp:156-169. */
int mm_scratch_layout(int R, int E, int T, int K, int H, int I, int64_t* offsets, int64_t* total_bytes);

/* Peer-mappable device memory: allocate and export / import / unmap / free.  The handle is 64 bytes.
 * Replace allocate_hip_ipc_buffer, open_hip_ipc_handles, close_hip_ipc_handles, free_hip_ipc_buffer,
 * csrc/python_api_hip.cpp:38-101.  These calls synchronise. */
int mm_ipc_alloc(int64_t bytes, void** dev_ptr, void* handle64);
int mm_ipc_open(const void* handle64, void** dev_ptr);
int mm_ipc_close(void* dev_ptr);
int mm_ipc_free(void* dev_ptr);

/* Zero the control regions of both buffers (signals, count matrix, epochs, status, row amax) and write the
 * peer pointer table into the symmetric buffer header.  Call once after allocation, and again (after a host
 * barrier across ranks) to recover from a reported error.
 * Replaces set_mega_moe_peer_ptrs, csrc/apis/mega_dcu.hpp:171-210 (and the buffer.zero_() before it). */
int mm_init_buffers(void* sym_base, void* scratch, const uint64_t* peer_ptrs, int rank,
                    int R, int E, int T, int K, int H, int I, void* stream);

/* Per-row FP8 e4m3 quantisation of a bf16 matrix [rows, k] (k % 8 == 0): scale = max(amax,1e-4)/448.
 * Replaces cast_to_fp8_channelwise, megamoe/__init__.py:51-56 (bit-exact codes and scales). */
int mm_quant_per_token(const void* x_bf16, int64_t rows, int k, void* out_fp8, float* out_scale, void* stream);

/* Router top-k + weight normalisation + per-token FP8 quantisation in one kernel, writing the four input views of the
 * symmetric buffer directly (pass their device addresses).  router_logits f32 [num_tokens, E]; the K largest logits are
 * selected (ties towards the lower index, descending order) and weighted with a softmax over the selected logits.
 * Replaces what the reference leaves to its caller: torch.topk + softmax + cast_to_fp8_channelwise + four copy_ calls
 * (tests/test_mega_moe_dcu.py:491-508, README.md:482-487). */
int mm_router_topk_quant(const void* x_bf16, const float* router_logits, int num_tokens, int E, int K, int H, void* x_fp8,
                         float* x_sf, int64_t* topk_idx, float* topk_weights, void* stream);

/* The layer.  Inputs x / x_sf / topk_idx / topk_weights are read from the symmetric buffer views; y receives
 * bf16 [num_tokens, H].  w1 = fp8 weights [E_loc, 2I, H] (rows [0,I) gate, [I,2I) up) with s1 f32 [E_loc, 2I]; w2 = fp8
 * weights [E_loc, H, I] with s2 f32 [E_loc, H].  Both weight tensors are stored TILED in the order the GEMM kernels
 * stream them: [E_loc][n block][K/128][256 rows][128 bytes], one contiguous 32 KiB block per (output tile, k block).
 * For w1, n block j (j < I/128) holds gate rows [128j,128j+128) followed by up rows [I+128j, I+128j+128); for w2, n block
 * j (j < ceil(H/256)) holds rows [256j, 256j+256), zero rows past H.  (The reference packs 16x16 Marlin tiles for its
 * MMAC units instead, deep_gemm/include/deep_gemm/layout/mega_moe_dcu.cuh:50-66.)  stats (nullable) int32 [E_loc] accumulates rows received per local
 * expert.  peer_ptrs: HOST array of the R ranks' symmetric-buffer device addresses (entry `rank` is sym_base).
 * runtime_num_tokens (nullable): device int32 overriding num_tokens (CUDA-graph bucket mode).
 * activation_clamp: +inf for none.  mode: MM_MODE_FUSED (one launch, small token counts), MM_MODE_STAGED (routing kernels + the
 * layer kernel), MM_MODE_STAGED_SPLIT (separate dispatch / GEMM1 / requantisation / GEMM2 launches), or MM_MODE_STAGED_UE8M0:
 * split launches with the activation recipe of the reference's Blackwell kernel -- e4m3 codes with one power-of-two (UE8M0)
 * scale per (row, 32 columns), produced in the GEMM1 epilogue and applied by a block-scaled MMA in GEMM2
 * (deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:839-870,1023-1057); weights stay FP8 with channelwise scales.
 * Replaces launch_mega_moe_multirank_persistent_hip_w8a8_channelwise, csrc/apis/mega_dcu.hpp:41-55, and the
 * staged driver fp8_mega_moe_large_opt_3stage, megamoe/large_opt.py:367-508. */
int mm_fp8_w8a8_mega_moe(void* y, const void* w1, const float* s1, const void* w2, const float* s2, int* stats,
                         void* sym_base, void* scratch, const uint64_t* peer_ptrs, int rank, int R,
                         int T_max, int E_loc, int num_tokens, int K, int H, int I, float activation_clamp,
                         int mode, const int* runtime_num_tokens, void* stream);

/* Copy the 5-word status {code, phase, rank, expected, observed} of the scratch buffer to the host
 * (synchronises the stream).  code 0 = no bounded wait expired.  The reference aborts the process instead
 * (deep_gemm/include/deep_gemm/comm/mega_moe_dcu.cuh:85-89). */
int mm_read_status(const void* scratch, void* stream, int32_t* out5);

/* Set the limits of the device-side bounded waits (milliseconds): cross-rank barriers and in-kernel pipelines. */
int mm_set_timeouts(int rank_barrier_ms, int pipeline_ms);

/* Tuning switches of the layer kernel, for measurements (no counterpart in the reference, whose tile policy is fixed at
 * compile time, deep_gemm/include/deep_gemm/impls/mega_moe_dcu.cuh:129-137).  policy bits: 1 = both helper warps of a CTA
 * push rows (default: one pushes, one requantises from the start), 2 = epilogue warps help pushing until their first
 * accumulator is complete (default on), 4 = inside a wave pair all GEMM1 tiles come before the GEMM2 tiles (default: they
 * alternate), 8 = tiles assigned round-robin instead of claimed dynamically.  wave_mblocks: m-blocks per wave of the tile
 * order, 0 = default (about two rounds of GEMM1 tiles), negative = one wave.  Defaults come from MEGAMOE_HELPER_POLICY and
 * MEGAMOE_WAVE_MBLOCKS at load time.  All ranks of a group must use the same values. */
int mm_set_tuning(int policy, int wave_mblocks);

/* Test hook (host only, no device work): the layer kernel's tile order.  out3 receives, for tile index t = 0 ..
 * num_mblocks * (gemm1_blocks + gemm2_blocks) - 1, the triple {kind (0 = GEMM1, 1 = GEMM2), m-block, n-block} that the kernel's
 * own order object yields -- the same code the device runs.  The order replaces the reference's wave scheduler
 * (deep_gemm/include/deep_gemm/scheduler/mega_moe.cuh:116-181); the kernel's freedom from deadlock rests on two of its
 * properties, which the CPU tests check: every tile appears exactly once, and every GEMM2 tile of an m-block comes after all
 * GEMM1 tiles of that m-block. */
int mm_tile_order(int num_mblocks, int wave_mblocks, int gemm1_blocks, int gemm2_blocks, int tile_interleave, int32_t* out3);

/* Tuning aid: per-tile cycle stamps of one CTA of the layer kernel.  device_words: max_tiles x 12 int64 words in device
 * memory (zeroed by the caller), filled by later calls: word 0 = tile index | kind << 32 (0 = GEMM1, 1 = GEMM2), then the
 * SM's clock64 when the producer took the tile / saw its dependency met / issued its last copy, when the MMA issuer took
 * it / issued its first / its last MMA, when the first epilogue warp began waiting for the accumulator / saw it complete /
 * released it.  max_tiles = 0 switches the trace off.  Not for production: the stamps cost a few stores per tile. */
int mm_set_tile_trace(void* device_words, int max_tiles, int cta);

/* JSON description of the build.  Replaces get_mega_moe_hip_build_config, csrc/apis/mega_dcu.hpp:28-39. */
int mm_build_config(char* json, int capacity);

/* Number of kernels the library has launched in this process (all entry points). */
int64_t mm_launch_count(void);

/* Size of the work area built into the library for mm_fp8_w8a8_mega_moe_static (bytes, per GPU). */
#define MM_STATIC_WORK_BYTES (64u << 20)

/* The single-rank layer WITHOUT caller-provided work buffers, for hosts that are not allowed to allocate device
 * memory (a serving process whose memory arena owns all of HBM, a code path where cudaMalloc's device-wide
 * synchronisation is unacceptable, a plugin that may only touch the tensors it is handed).  It has no counterpart in
 * the reference, which always allocates its symmetric buffer and route scratch itself (megamoe/__init__.py:172-177).
 * The symmetric and scratch regions live in a device array of MM_STATIC_WORK_BYTES that is part of the library image:
 * every GPU that loads the library holds it until the process exits.  Shapes whose regions do not fit (see
 * mm_symm_buffer_layout / mm_scratch_layout with R = 1 and T = num_tokens rounded up to 384) are rejected with an error.
 * x_fp8 [num_tokens,H], x_sf [num_tokens], topk_idx int64 [num_tokens,K], topk_weights f32 [num_tokens,K] and y bf16
 * [num_tokens,H] are device pointers; weights/scales/stats/clamp as for mm_fp8_w8a8_mega_moe, num_experts = all experts.
 * No cudaMalloc, cudaFree or other allocating call is made.  The first call on each device looks up the address of
 * the built-in area (cudaGetSymbolAddress); make that first call outside any stream capture.  All calls on a device
 * share the area and it keeps the previous call's contents, so each call first clears the words that must start at
 * zero; two calls that overlap on the GPU (different streams) race -- serialise them. */
int mm_fp8_w8a8_mega_moe_static(void* y, const void* x_fp8, const float* x_sf, const int64_t* topk_idx,
                                const float* topk_weights, const void* w1, const float* s1, const void* w2, const float* s2,
                                int* stats, int num_tokens, int num_experts, int K, int H, int I, float activation_clamp,
                                void* stream);

/* Status words {code, phase, rank, expected, observed} of the LAST mm_fp8_w8a8_mega_moe_static call on the current device
 * (they live inside the built-in work area, which the caller cannot address, and the next static call clears them): copies
 * them to the host and synchronises the stream.  code 0 = no bounded wait expired and the receive pool did not overflow;
 * otherwise y of that call is not valid.  No counterpart in the reference (see mm_read_status). */
int mm_fp8_w8a8_mega_moe_static_status(void* stream, int32_t* out5);

/* DeepEP-layout helpers of the reference's split baseline (DeepEP dispatch -> scatter -> grouped GEMM -> gather -> DeepEP
 * combine).  Scatter groups the received tokens by expert: expert_start_loc = exclusive prefix of
 * num_recv_tokens_per_expert; route (token, slot) with expert e gets row expert_start_loc[e] + its rank among e's routes (in
 * route order; the reference's atomicAdd order is unspecified); output_index[route] = row or -1; m_indices[row] = e; the FP8
 * row, its scale and the route weight are copied.  The caller pre-fills output_index and m_indices with -1 and
 * route_weights with 0.  Gather: recv_y[token] = bf16(sum over slots of l2_out[output_index] (* weight)).
 * Replace launch_mega_moe_deepep_scatter_channelwise_hip / ..._gather_..., csrc/kernels/mega_moe_baseline_hip.cu:130-232. */
int mm_deepep_scatter_channelwise(void* grouped_x, float* grouped_x_scale, float* route_weights, int* m_indices, int* output_index,
                                  int* expert_start_loc, const void* recv_x, const float* recv_x_scale, const void* recv_topk_ids,
                                  const float* recv_topk_weights, const int* num_recv_tokens_per_expert, int total_rows,
                                  int recv_rows, int topk, int hidden, int num_experts, int topk_ids_i64, void* stream);
int mm_deepep_gather_channelwise(void* recv_y, const void* l2_out, const void* recv_topk_ids, const float* recv_topk_weights,
                                 const int* output_index, int recv_rows, int topk, int hidden, int topk_ids_i64,
                                 int apply_topk_weights, void* stream);

/* The compute pieces of the reference test's split baseline (tests/test_mega_moe_dcu.py:188-300), so that it can be run
 * on B200 beside the fused layer.
 *
 * mm_m_grouped_fp8_gemm_nt_contiguous: out[row, :] = bf16( (a_fp8[row, :] . w[e, :, :]^T) * a_scale[row] * w_scale[e, :] ),
 *   e = m_indices[row]; stands in for the external deepgemm.m_grouped_fp8_gemm_nt_contiguous that the test calls
 *   (tests/test_mega_moe_dcu.py:245-250, 274-279).  Rows are grouped by expert, every group padded to 128 rows, padding
 *   rows carry m_indices = -1 (left untouched in `out`).  w_tiled: [E][ceil(N/256)][K/128][256][128] e4m3 (rows in natural
 *   order, the "l2" packing of the Python helper pack_weights_tiled).  work: device int32[32 + 2 * rows / 128]; its first
 *   five words are a status record readable with mm_read_status (code 5 = a block mixes experts or has a hole).
 * mm_swiglu_quant_channelwise: the reference's K2 kernel (megamoe/dcu_megamoe_large_opt/K2_fused/k2_fused_ext.cu:254-377;
 *   Python wrapper K2_fused/k2_fused.py:12-58): x bf16 [rows][2*inter] (gate | up) -> e4m3 [rows][inter] + f32 scale [rows],
 *   y = gate * sigmoid(gate) * up * weights[row] (fp32; clamp: up two-sided, gate from above), scale = max(amax, 1e-4) / 448.
 *   weights, row_combine_ptrs and out_bf16 may be null. */
int mm_m_grouped_fp8_gemm_nt_contiguous(const void* a_fp8, const float* a_scale, const void* w_tiled, const float* w_scale,
                                        void* out_bf16, const int* m_indices, int rows, int N, int K, int E, int* work,
                                        void* stream);
int mm_swiglu_quant_channelwise(const void* x_bf16, const float* weights, const int64_t* row_combine_ptrs, void* out_fp8,
                                float* out_scale, void* out_bf16, int rows, int inter, int has_clamp, float clamp_value,
                                void* stream);

/* Measurement aid (no counterpart in the reference, whose test divides by a datasheet figure, tests/test_mega_moe_dcu.py:20-22):
 * launch a kernel that issues `iters` groups of eight dense FP8 MMAs (tcgen05 kind::f8f6f4, M128 x N256 x K32 per SM) from
 * operands resident in shared memory.  *flops_out receives the floating-point operations of the launch; time it with events
 * on `stream` to get the tensor-core rate the GEMM kernels can at best reach.
 *   operands: 0 = every byte 1.0 (few bits toggle: the burst rate), 1 = pseudo-random finite e4m3 values of both signs and
 *             magnitude below 2, 2 = e4m3 codes as per-row quantisation of N(0,1) data produces them (exponent fields 9..14,
 *             random sign and mantissa).  The cycle count per MMA is the same for all three (128); the power draw is not,
 *             and under the board's power cap the clock -- and with it the rate -- falls from 0 to 1 to 2;
 *   cta_pair: 0 = cta_group::1 MMAs, 1 = cta_group::2 MMAs (M256 over two SMs) as the CTA-pair GEMM kernels issue them.
 * status_dev: a zeroed device int. */
int mm_fp8_mma_peak_probe(int iters, int operands, int cta_pair, int* status_dev, void* stream, double* flops_out);

/* Measurement aid (no counterpart in the reference, whose test divides by a datasheet interconnect figure,
 * tests/test_mega_moe_dcu.py:20-22): write bytes_per_dst bytes (a multiple of 512) with plain 16-byte vector stores into
 * each of the n_dst device addresses of the HOST array dst_ptrs.  With peer-mapped addresses (e.g. the receive pool of
 * other ranks' symmetric buffers, between layer calls) and events on `stream` this gives the NVLink store rate that the
 * dispatch push and the GEMM2 combine stores can at best reach.  The destinations' previous contents are lost. */
int mm_peer_store_probe(const uint64_t* dst_ptrs, int n_dst, int64_t bytes_per_dst, void* stream);

/* Per-stage device timing of the layer call (the reference's test prints per-kernel times with a profiler,
 * tests/test_mega_moe_dcu.py:794-834; here CUDA events are recorded on the caller's stream around every launch).
 * mm_set_stage_timing(1) turns recording on for later calls; mm_get_stage_times waits for the last timed call and
 * fills ms[MM_NUM_STAGES] with each stage's duration in milliseconds (-1 for a stage that did not run). */
int mm_set_stage_timing(int enable);
int mm_get_stage_times(float* ms, int n);

#ifdef __cplusplus
}
#endif
#endif
