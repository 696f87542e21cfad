// Memory layout of the Mega MoE layer: one symmetric (peer-mapped) buffer and one local scratch buffer per rank.
// Single source of truth for host code, device code and (through mm_symm_buffer_layout / mm_scratch_layout) Python.
//
// The reference keeps [peer ptrs][signal ptrs][runtime token count] x, x_sf, topk_idx, topk_weights, combine[K][T][H]
// in its symmetric buffer (deep_gemm/include/deep_gemm/layout/mega_moe_dcu.cuh:23-48,116-130) and pulls token rows
// from the source rank.  This layout keeps the same caller-visible views and adds what a push design needs on the
// owning rank: the [R][E] route-count matrix, the per-expert receive pool and its per-row metadata.
#pragma once
#include <stdint.h>

#define MM_MAX_RANKS 16
#define MM_BLOCK_M 128           // rows of one GEMM tile; every expert's pool segment starts on a multiple of it
#define MM_TOKEN_ALIGNMENT 384   // deep_gemm/include/deep_gemm/layout/mega_moe_dcu.cuh:9
#define MM_ROUTE_CHUNK 256       // routes handled by one block of the routing kernels
#define MM_MAX_EXPERTS 1024
#define MM_MAX_TOPK 32

// cross-rank barrier ids (one int32 slot per (barrier, source rank) in the symmetric buffer)
enum { MM_BAR_COUNTS = 0, MM_BAR_DISPATCH = 1, MM_BAR_COMBINE = 2, MM_NUM_BARRIERS = 4 };

// status codes written by bounded device-side waits (0 = ok)
enum {
    MM_OK = 0,
    MM_ERR_RANK_BARRIER_TIMEOUT = 1,
    MM_ERR_PIPE_TIMEOUT = 2,
    MM_ERR_POOL_OVERFLOW = 3,
    MM_ERR_GRID_BARRIER_TIMEOUT = 4,
};

struct MmStatus {       // first bytes of the scratch buffer
    int32_t code, phase, rank, expected, observed;
    int32_t pad[11];
};

struct MmPoolMeta {     // one per receive-pool row, written by the source rank together with the row
    float x_scale;      // per-token activation scale of the source token
    float route_weight; // top-k weight of this route
    int32_t src_token;  // token index on the source rank
    int32_t src_info;   // (source rank << 8) | top-k slot
};

#ifdef __cplusplus
static inline int64_t mm_align(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

struct MmSymLayout {
    int64_t peer_ptrs;          // uint64 [MM_MAX_RANKS]
    int64_t signals;            // int32  [MM_NUM_BARRIERS][MM_MAX_RANKS]
    int64_t runtime_num_tokens; // int32  [1]  (device-side token count used in graph mode)
    int64_t count_matrix;       // int32  [R][E]   row r is written by rank r
    int64_t pool_arrive;        // int32  [pool_rows / MM_BLOCK_M + 1]  rows landed per m-block, last word = all rows (fused variant)
    int64_t x;                  // fp8    [T][H]
    int64_t x_sf;               // f32    [T]
    int64_t topk_idx;           // int64  [T][K]
    int64_t topk_weights;       // f32    [T][K]
    int64_t pool_x;             // fp8    [pool_rows][H]   written by source ranks
    int64_t pool_meta;          // MmPoolMeta [pool_rows]
    int64_t combine;            // bf16   [T][K][H]        written by owner ranks; a token's K slots are adjacent, so the rows of one
                                //                         GEMM2 tile (consecutive tokens of one source rank) land in a few MiB of the peer
    int64_t total;
    int64_t pool_rows;          // capacity in rows (multiple of MM_BLOCK_M)
};

struct MmScratchLayout {
    int64_t status;        // MmStatus
    int64_t epoch;         // int32 [4]: [0] call epoch used by the cross-rank barriers, [1..] grid-barrier words
    int64_t plan;          // int32 [8]: [0] num_mblocks, [1] pool rows in use (padded), [2] m-block pairs, [3] valid routes of this
                           //            rank (length of send_list), [6] rows to receive
    int64_t block_counts;  // int32 [route_blocks][E]   per-block histogram, then exclusive prefix over blocks
    int64_t dest_base;     // int32 [E]   first pool row (on the owner) for this rank's routes to expert e
    int64_t expert_total;  // int32 [E_loc]
    int64_t expert_off;    // int32 [E_loc]
    int64_t mblock_expert; // int32 [pool_rows / MM_BLOCK_M]
    int64_t mblock_valid;  // int32 [pool_rows / MM_BLOCK_M]
    int64_t l1_done;       // int32 [pool_rows / MM_BLOCK_M]      epilogue-warp shares of GEMM1 tiles stored per m-block (layer kernel)
    int64_t l2_ready;      // int32 [pool_rows / MM_BLOCK_M]      quarters of an m-block requantised (layer kernel)
    int64_t grid_sync;     // int32 [8]  [0] CTA arrivals (monotonic), [1] fused calls completed, [2] requantisation units done,
                           //            [3] push cursor into send_list, [4] requantisation-unit cursor
    int64_t dest_row;      // int32 [T][K]   pool row of each local route (-1 invalid); kept for inspection
    int64_t send_base;     // int32 [E]      position in send_list of this rank's first route to expert e
    int64_t send_list;     // int32x4 [T][K] this rank's valid routes in send order (local expert index, then owner rank):
                           //                {route, pool row on the owner, owner rank, token}
    int64_t row_amax;      // u32   [pool_rows]  bit pattern of the non-negative row amax, self-resetting
    int64_t act_scale;     // f32   [pool_rows]
    int64_t act_bf16;      // bf16  [pool_rows][I]
    int64_t act_fp8;       // fp8   [pool_rows][I]
    int64_t act_sf;        // u8    [pool_rows / 128][I / 128][512]  UE8M0 scale bytes of the block-scaled recipe (gemm_ue8m0.cuh)
    int64_t total;
    int64_t route_blocks;
};

static inline int64_t mm_pool_rows(int R, int E, int T, int K) {
    const int64_t e_loc = E / R;
    return mm_align((int64_t)R * T * K + e_loc * (MM_BLOCK_M - 1), MM_BLOCK_M);
}

static inline MmSymLayout mm_sym_layout(int R, int E, int T, int K, int H, int I) {
    (void)I;
    MmSymLayout L;
    int64_t o = 0;
    L.peer_ptrs = o;          o = mm_align(o + 8 * MM_MAX_RANKS, 256);
    L.signals = o;            o = mm_align(o + 4 * MM_NUM_BARRIERS * MM_MAX_RANKS, 256);
    L.runtime_num_tokens = o; o = mm_align(o + 16, 256);
    L.count_matrix = o;       o = mm_align(o + (int64_t)4 * R * E, 256);
    L.pool_rows = mm_pool_rows(R, E, T, K);
    L.pool_arrive = o;        o = mm_align(o + (L.pool_rows / MM_BLOCK_M + 1) * 4, 256);
    L.x = o;                  o = mm_align(o + (int64_t)T * H, 256);
    L.x_sf = o;               o = mm_align(o + (int64_t)T * 4, 256);
    L.topk_idx = o;           o = mm_align(o + (int64_t)T * K * 8, 256);
    L.topk_weights = o;       o = mm_align(o + (int64_t)T * K * 4, 256);
    L.pool_rows = mm_pool_rows(R, E, T, K);
    L.pool_x = o;             o = mm_align(o + L.pool_rows * H, 256);
    L.pool_meta = o;          o = mm_align(o + L.pool_rows * (int64_t)sizeof(MmPoolMeta), 256);
    L.combine = o;            o = mm_align(o + (int64_t)K * T * H * 2, 256);
    L.total = o;
    return L;
}

static inline MmScratchLayout mm_scratch_layout_of(int R, int E, int T, int K, int H, int I) {
    (void)H;
    MmScratchLayout L;
    const int64_t pool_rows = mm_pool_rows(R, E, T, K);
    const int64_t e_loc = E / R;
    L.route_blocks = ((int64_t)T * K + MM_ROUTE_CHUNK - 1) / MM_ROUTE_CHUNK;
    if (L.route_blocks < 1) L.route_blocks = 1;
    int64_t o = 0;
    L.status = o;        o = mm_align(o + (int64_t)sizeof(MmStatus), 256);
    L.epoch = o;         o = mm_align(o + 16, 256);
    L.plan = o;          o = mm_align(o + 32, 256);
    L.block_counts = o;  o = mm_align(o + L.route_blocks * E * 4, 256);
    L.dest_base = o;     o = mm_align(o + (int64_t)E * 4, 256);
    L.expert_total = o;  o = mm_align(o + e_loc * 4, 256);
    L.expert_off = o;    o = mm_align(o + e_loc * 4, 256);
    L.mblock_expert = o; o = mm_align(o + pool_rows / MM_BLOCK_M * 4, 256);
    L.mblock_valid = o;  o = mm_align(o + pool_rows / MM_BLOCK_M * 4, 256);
    L.l1_done = o;       o = mm_align(o + pool_rows / MM_BLOCK_M * 4, 256);
    L.l2_ready = o;      o = mm_align(o + pool_rows / MM_BLOCK_M * 4, 256);
    L.grid_sync = o;     o = mm_align(o + 32, 256);
    L.dest_row = o;      o = mm_align(o + (int64_t)T * K * 4, 256);
    L.send_base = o;     o = mm_align(o + (int64_t)E * 4, 256);
    L.send_list = o;     o = mm_align(o + (int64_t)T * K * 16, 256);
    L.row_amax = o;      o = mm_align(o + pool_rows * 4, 256);
    L.act_scale = o;     o = mm_align(o + pool_rows * 4, 256);
    L.act_bf16 = o;      o = mm_align(o + pool_rows * I * 2, 1024);
    L.act_fp8 = o;       o = mm_align(o + pool_rows * I, 1024);
    L.act_sf = o;        o = mm_align(o + pool_rows / MM_BLOCK_M * (I / 128) * 512, 1024);
    L.total = o;
    return L;
}
#endif
