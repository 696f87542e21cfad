// Grouped FP8 GEMMs on CTA PAIRS (thread-block cluster of 2, tcgen05 cta_group::2) for shapes with many rows per expert.
//
// One pair works on two m-blocks (2 x 128 pool rows) of the SAME expert against one 256-row weight tile:
//   * each CTA loads its own 128 activation rows and only HALF of the weight tile (128 of its 256 rows), so the operand
//     bytes per SM and per k block drop from 48 KiB to 32 KiB (and the L2 -> SM traffic of the launch by a third);
//   * one thread of the pair's leader (cluster rank 0) issues M256 x N256 x K32 MMAs that read both CTAs' shared memory
//     and write each CTA's 128 accumulator rows into that CTA's own TMEM;
//   * tcgen05.commit arrives on the barriers of both CTAs, so each CTA's producer and epilogue warps wait locally;
//     the peer's copies count their bytes on the leader's "operands landed" barrier, and the peer's epilogue warps
//     arrive remotely on the leader's "accumulator free" barrier.
// An expert with an odd number of m-blocks leaves the second CTA of its last pair without rows: that CTA still feeds the
// pipeline (it re-loads the first m-block's rows) and skips the stores.
// Same arithmetic, epilogue and outputs (bit for bit) as gemm.cuh; same bounded waits and status words.
// Measured on B200 (hidden 4096, intermediate 2048): with 192 rows per expert (two m-blocks: every weight tile is streamed
// from HBM once instead of once from HBM and once from L2) both GEMMs are 10 % faster than with the one-CTA kernel; with
// 384 rows (three m-blocks, a half-empty second pair) GEMM1 is 7 % slower, with 768 rows 9 % slower, with 1536 rows it
// ties.  The host code therefore picks this kernel when an expert is expected to hold two m-blocks.
#pragma once
#include "gemm.cuh"

namespace mm {

constexpr int kPairStages = 6;
constexpr int kPairBBytes = kBBytes / 2;                       // each CTA holds 128 of the tile's 256 weight rows
constexpr int kPairStageBytes = kABytes + kPairBBytes;         // 32 KiB
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + kStagingBytes + kScaleBytes + 256 /*barriers*/;
static_assert(kPairSmemBytes <= 232448, "exceeds the 227 KiB of shared memory a CTA can have");

// Walks the experts in order as the pair index grows (a CTA's pair indices are increasing).
struct PairWalker {
    int e = 0, base = 0, n = -1;
    // returns false when `pair` is beyond the last expert
    __device__ __forceinline__ bool seek(const GemmParams& p, int pair) {
        if (n < 0) n = e < p.E_loc ? (((p.expert_total[e] + kBlockM - 1) / kBlockM) + 1) / 2 : 0;
        while (e < p.E_loc && pair >= base + n) {
            base += n;
            ++e;
            n = e < p.E_loc ? (((p.expert_total[e] + kBlockM - 1) / kBlockM) + 1) / 2 : 0;
        }
        return e < p.E_loc;
    }
    // m-block handled by cluster rank r for this pair, or -1 when the expert has no such m-block
    __device__ __forceinline__ int mblock(const GemmParams& p, int pair, int r) const {
        const int j = 2 * (pair - base) + r;
        const int blocks = (p.expert_total[e] + kBlockM - 1) / kBlockM;
        return j < blocks ? p.expert_off[e] / kBlockM + j : -1;
    }
};

template <int kKind>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b_half, GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    uint8_t* smem_gen = smem_raw;
    if ((smem_base & 1023u) != 0u) {                         // same in both CTAs of a pair, so both leave
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, MM_ERR_PIPE_TIMEOUT) == 0) { p.status[1] = 110 + kKind; p.status[2] = blockIdx.x; }
        return;
    }
    const uint32_t staging_u32 = smem_base + kPairStages * kPairStageBytes;
    uint8_t* staging_gen = smem_gen + kPairStages * kPairStageBytes;
    float* scales_gen = reinterpret_cast<float*>(staging_gen + kStagingBytes);
    const uint32_t bars = staging_u32 + kStagingBytes + kScaleBytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };                       // used in the leader only
    auto empty_bar = [&](int s) { return bars + 8u * (kPairStages + s); };      // per CTA
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * kPairStages + a); };  // per CTA
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * kPairStages + 2 + a); };   // used in the leader only
    uint8_t* tail_gen = staging_gen + kStagingBytes + kScaleBytes + 8 * (2 * kPairStages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail_gen);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail_gen + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();                 // 0 = leader
    const bool leader = cta == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 2 * kEpilogueWarps); }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b_half);
    }
    __syncthreads();
    cluster_sync_all();                                     // both CTAs' barriers exist before anyone arrives remotely
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_slot), 512);          // the same warp in both CTAs
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_pairs = p.status[0] != 0 ? 0 : p.plan[2];   // no tile after a failed bounded wait earlier in the call
    const int num_tiles = num_pairs * p.n_blocks;
    const int k_blocks = p.kdim / kBlockK;
    const int first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one thread in each CTA)
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool alive = true;
            PairWalker w;
            for (int tile = first_tile; tile < num_tiles && alive; tile += tile_step) {
                const int pair = tile / p.n_blocks, nb = tile - pair * p.n_blocks;
                if (!w.seek(p, pair)) break;
                int mb = w.mblock(p, pair, (int)cta);
                if (mb < 0) mb = w.mblock(p, pair, 0);      // no rows of its own: feed the pipeline with the first m-block
                const int a_row = mb * kBlockM;
                const int b_tile0 = (w.e * p.n_blocks + nb) * k_blocks;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.timeout_ns)) { alive = false; break; }
                    const uint32_t a_dst = smem_base + stage * kPairStageBytes;
                    const uint32_t b_dst = a_dst + kABytes;
                    const uint32_t lead_full = mapa_shared(full_bar(stage), 0);
                    // Only the leader arrives (with the bytes of both CTAs); the peer's copies count their bytes on the
                    // leader's barrier as they land.  The peer cannot run a phase ahead: it refills a stage only after the
                    // commit that follows the leader's wait on this barrier.
                    if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * kPairStageBytes);
                    tma_load_2d_pair(a_dst, &tm_a, kb * kBlockK, a_row, lead_full);
                    tma_load_2d_pair(b_dst, &tm_b_half, 0, (b_tile0 + kb) * kBlockN + (int)cta * (kBlockN / 2), lead_full);
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one thread of the leader)
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc_f8(2 * kBlockM, kBlockN);
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool alive = true;
            for (int tile = first_tile; tile < num_tiles && alive; tile += tile_step) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.timeout_ns)) { alive = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBlockN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.timeout_ns)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t a_src = smem_base + stage * kPairStageBytes;
                    const uint64_t da = umma_desc_k_sw128(a_src);
                    const uint64_t db = umma_desc_k_sw128(a_src + kABytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / 32; ++k) umma_f8_pair(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit_pair(empty_bar(stage));                       // both CTAs' producers may refill the stage
                    if (kb == k_blocks - 1) umma_commit_pair(tfull_bar(acc)); // both CTAs' epilogues may read
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..9 of each CTA, own 128 rows)
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const int et = q * 32 + lane;
        uint8_t* my_staging = staging_gen + (warp - 2) * kStagingWarpBytes;
        const bool do_clamp = p.clamp < 3.0e38f;
        int acc = 0; uint32_t acc_phase = 0;
        bool alive = true;
        PairWalker w;
        for (int tile = first_tile; tile < num_tiles && alive; tile += tile_step) {
            if (*abort_flag != 0) break;
            const int pair = tile / p.n_blocks, nb = tile - pair * p.n_blocks;
            if (!w.seek(p, pair)) break;
            const int mb_own = w.mblock(p, pair, (int)cta);
            const int mb = mb_own < 0 ? 0 : mb_own;
            const int e = w.e;
            const int valid = mb_own < 0 ? 0 : p.mblock_valid[mb];
            const int row = mb * kBlockM + et;
            const bool row_ok = et < valid;
            float* sc = scales_gen + acc * kBlockN;
            {
                const int t = (warp - 2) * 32 + lane;
                const float* ws = p.w_scale + static_cast<int64_t>(e) * p.w_rows_per_expert;
                if (kKind == 0) {
                    sc[t] = t < 128 ? ws[nb * 128 + t] : ws[p.w_rows_per_expert / 2 + nb * 128 + (t - 128)];
                } else {
                    const int c0 = nb * kBlockN + t;
                    sc[t] = c0 < p.n_out ? ws[c0] : 0.0f;
                }
            }
            named_bar_sync(1, kEpilogueThreads);
            float row_scale = 0.0f, route_w = 0.0f;
            uint8_t* out_ptr = nullptr;
            if (row_ok) {
                const MmPoolMeta m = p.meta[row];
                if (kKind == 0) {
                    row_scale = m.x_scale;
                    route_w = m.route_weight;
                } else {
                    row_scale = p.act_scale[row];
                    out_ptr = combine_row_ptr(p, m.src_info, m.src_token);
                }
            }
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.timeout_ns)) { alive = false; break; }
            tc_fence_after();
            if (valid > 0)
                epilogue_math<kKind>(p, tmem_base, sc, my_staging, lane, q, half, acc, mb, nb, valid, row, row_ok, row_scale, route_w,
                                     out_ptr, do_clamp);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(tempty_bar(acc));
                else mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0));
            }
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag != 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 1000000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, MM_ERR_PIPE_TIMEOUT) == 0) {
            p.status[1] = 10 + kKind; p.status[2] = blockIdx.x; p.status[3] = num_tiles; p.status[4] = 0;
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer may still arrive on, or read, this CTA's shared memory until it gets here
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

}  // namespace mm
