// Grouped FP8 GEMMs of the layer on the 5th-generation tensor cores (tcgen05, accumulators in TMEM, operands by TMA).
//
//   kind 0 (GEMM1): act[row, j] = bf16( silu(g) * u * w_route ),  g = acc_gate * (sx[row] * s1[j]),  u likewise with
//                   weight row I + j; also the per-row amax of the bf16 values.  Replaces
//                   deep_gemm/include/deep_gemm/impls/mega_moe_dcu_tiles.cuh:380-670 (compute_route_mmac_mtile16_l1_chunk).
//   kind 2 (GEMM1, UE8M0 recipe): the same SwiGLU value in fp32, quantised in the epilogue with one power-of-two scale
//                   per (row, 32 columns): codes e4m3(a * 2^-e), scale byte e + 127 (gemm_ue8m0.cuh consumes them).
//   kind 1 (GEMM2): out[row, h] = bf16( acc * (s2[row] * sw2[h]) ) stored straight into combine[token][slot][:] of the
//                   SOURCE rank over NVLink.  Replaces impls/mega_moe_dcu_tiles.cuh:735-1163.
//
// One persistent CTA per SM, 320 threads: warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM), warps 2-9 = epilogue.
// Tile = 128 pool rows (UMMA M, TMEM lanes) x 256 weight rows (UMMA N, TMEM columns) x 128 bytes of K per stage;
// two accumulator buffers (2 x 256 TMEM columns) so the epilogue of tile i overlaps the MMAs of tile i+1.
// For kind 0 the 256 weight rows are 128 gate rows and the 128 matching up rows, so one tile yields 128 SwiGLU outputs.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include "layout.h"
#include "ptx.cuh"

namespace mm {

constexpr int kBlockM = MM_BLOCK_M;   // 128
constexpr int kBlockN = 256;
constexpr int kBlockK = 128;          // bytes == fp8 elements; one 128-byte swizzle atom
constexpr int kStages = 4;
constexpr int kEpilogueWarps = 8;
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kGemmThreads = 64 + kEpilogueThreads;     // TMA warp + MMA warp + epilogue warps
constexpr int kABytes = kBlockM * kBlockK;              // 16 KiB
constexpr int kBBytes = kBlockN * kBlockK;              // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kStagingWarpBytes = 32 * 128;              // one 128-byte output segment for each of a warp's 32 rows
constexpr int kStagingBytes = kEpilogueWarps * kStagingWarpBytes;
constexpr int kScaleBytes = 2 * kBlockN * 4;
constexpr int kGemmSmemBytes = kStages * kStageBytes + kStagingBytes + kScaleBytes + 256 /*barriers*/;
static_assert(kGemmSmemBytes <= 232448, "exceeds the 227 KiB of shared memory a CTA can have");

struct GemmParams {
    int kdim;                  // reduction length (H for kind 0, I for kind 1)
    int n_blocks;              // tiles along the weight rows (I/128 for kind 0, ceil(H/256) for kind 1)
    int n_out;                 // I (kind 0) or H (kind 1): valid output columns
    int w_rows_per_expert;     // 2I (kind 0) or H (kind 1)
    const int* plan;           // [0] = number of m-blocks in use, [2] = number of m-block pairs (gemm_pair.cuh)
    const int* expert_total;   // [E_loc] rows received per local expert
    const int* expert_off;     // [E_loc] first pool row of each local expert
    int E_loc;
    const int* mblock_expert;
    const int* mblock_valid;
    const MmPoolMeta* meta;    // per pool row
    const float* w_scale;      // [E_loc][w_rows_per_expert]
    // kind 0
    __nv_bfloat16* act_bf16;   // [pool_rows][I]
    unsigned int* row_amax;
    float clamp;               // +inf = none
    // kind 2 (GEMM1 with per-(row, 32 columns) UE8M0 activation scales): FP8 codes and scale bytes, no bf16 round trip
    uint8_t* act_q_out;        // [pool_rows][I] e4m3
    uint8_t* act_sf;           // [m-blocks][I / 128][512]: scale bytes of 128 rows x 4 column blocks, byte (r % 32) * 16 + (r / 32) * 4 + block
    // kind 1
    const float* act_scale;    // [pool_rows]
    __nv_bfloat16* out_rows;   // null: store into the source ranks' combine buffers; else out_rows[row][n_out] (plain grouped GEMM)
    uint64_t peers[MM_MAX_RANKS];
    int64_t combine_off;
    int T, H;
    int R, K;                  // ranks and top-k slots: bounds of the (source rank, slot) a pool row may name
    // error reporting
    int* status;               // MmStatus*
    uint64_t timeout_ns;
};

// Destination of one GEMM2 output row: combine[token][slot][:] on the SOURCE rank.  The row's metadata was written by
// that rank; a pool row nobody wrote in this call (error path, stale or uninitialised memory) may name anything, so the
// three indices are range-checked and a row that fails the check is not stored at all.
__device__ __forceinline__ uint8_t* combine_row_ptr(const GemmParams& p, int src_info, int src_token) {
    const int src_rank = src_info >> 8, slot = src_info & 0xff;
    if (src_rank < 0 || src_rank >= p.R || slot >= p.K || src_token < 0 || src_token >= p.T) return nullptr;
    return reinterpret_cast<uint8_t*>(p.peers[src_rank]) + p.combine_off +
           (static_cast<int64_t>(src_token) * p.K + slot) * p.H * 2;
}

// x * sigmoid(x) with the fast exponential and reciprocal units, as the reference does
// (deep_gemm/include/deep_gemm/common/mega_moe_dcu.cuh:90-99: exp2 and rcp intrinsics)
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Epilogue arithmetic of one output tile for one epilogue warp: read this warp's share of the accumulator from TMEM,
// apply the scales (kind 0: SwiGLU x route weight and the row amax), and write 128-byte row segments.
//   q = TMEM lane quarter of the warp, half = which half of the tile's columns it handles, acc = accumulator buffer.
template <int kKind>
__device__ __forceinline__ void epilogue_math(const GemmParams& p, uint32_t tmem_base, const float* sc, uint8_t* my_staging,
                                              int lane, int q, int half, int acc, int mb, int nb, int valid, int row, bool row_ok,
                                              float row_scale, float route_w, uint8_t* out_ptr, bool do_clamp) {
    const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kBlockN;
    // Each pass handles one 128-byte output segment (64 bf16) per row: two 32-column chunks, staged in shared
    // memory (16-byte pieces XOR-swizzled by row so neither phase has bank conflicts), then written so that
    // 8 lanes cover one row's segment.
    constexpr int kPasses = (kKind == 1) ? 2 : 1;
    float amax = 0.0f;
#pragma unroll 1
    for (int pass = 0; pass < kPasses; ++pass) {
        const int seg_idx = half * kPasses + pass;      // 128-byte segment of this row within the tile
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
            const int c = seg_idx * 2 + sub;             // 32-column chunk of outputs
            uint32_t packed[16];
            if (kKind == 2) {
                // UE8M0 recipe: this thread holds the 32 columns of one scale block of its row
                uint32_t g[32], u[32];
                tmem_ld_32x32(t_addr + c * 32, g);
                tmem_ld_32x32(t_addr + 128 + c * 32, u);
                tmem_ld_wait();
                float o[32];
                float bmax = 0.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float gv = __uint_as_float(g[j]) * (row_scale * sc[c * 32 + j]);
                    float uv = __uint_as_float(u[j]) * (row_scale * sc[128 + c * 32 + j]);
                    if (do_clamp) {
                        gv = fminf(fmaxf(gv, -p.clamp), p.clamp);
                        uv = fminf(fmaxf(uv, -p.clamp), p.clamp);
                    }
                    o[j] = silu_f(gv) * uv * route_w;
                    bmax = fmaxf(bmax, fabsf(o[j]));
                }
                // smallest power of two 2^e with bmax <= 448 * 2^e, on the float bits: 448 = 1.75 * 2^8
                const uint32_t bits = __float_as_uint(bmax);
                int byte = static_cast<int>((bits >> 23) & 0xffu) - 8 + ((bits & 0x7fffffu) > 0x600000u ? 1 : 0);
                byte = min(max(byte, 1), 253);
                const float inv = __uint_as_float(static_cast<uint32_t>(254 - byte) << 23);
                uint32_t q8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(o[4 * j] * inv, o[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
                    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(o[4 * j + 2] * inv, o[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
                    q8[j] = lo | (hi << 16);
                }
                if (row_ok) {
                    uint4* dst = reinterpret_cast<uint4*>(p.act_q_out + static_cast<int64_t>(row) * p.n_out + nb * 128 + c * 32);
                    dst[0] = make_uint4(q8[0], q8[1], q8[2], q8[3]);
                    dst[1] = make_uint4(q8[4], q8[5], q8[6], q8[7]);
                }
                // scale byte of (row, block c): rows past the valid count get 1.0 so that nothing undefined reaches the MMA
                p.act_sf[(static_cast<int64_t>(mb) * p.n_blocks + nb) * 512 + lane * 16 + q * 4 + c] =
                    static_cast<uint8_t>(row_ok ? byte : 127);
                continue;
            }
            if (kKind == 0) {
                uint32_t g[32], u[32];
                tmem_ld_32x32(t_addr + c * 32, g);
                tmem_ld_32x32(t_addr + 128 + c * 32, u);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float o[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float gv = __uint_as_float(g[j + h]) * (row_scale * sc[c * 32 + j + h]);
                        float uv = __uint_as_float(u[j + h]) * (row_scale * sc[128 + c * 32 + j + h]);
                        if (do_clamp) {
                            gv = fminf(fmaxf(gv, -p.clamp), p.clamp);
                            uv = fminf(fmaxf(uv, -p.clamp), p.clamp);
                        }
                        o[h] = silu_f(gv) * uv * route_w;
                    }
                    const uint32_t pk = pack_bf16x2(o[0], o[1]);
                    packed[j / 2] = pk;
                    amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(pk << 16)), fabsf(__uint_as_float(pk & 0xffff0000u))));
                }
            } else {
                uint32_t a[32];
                tmem_ld_32x32(t_addr + c * 32, a);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const float o0 = __uint_as_float(a[j]) * (row_scale * sc[c * 32 + j]);
                    const float o1 = __uint_as_float(a[j + 1]) * (row_scale * sc[c * 32 + j + 1]);
                    packed[j / 2] = pack_bf16x2(o0, o1);
                }
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const int piece = (sub * 4 + v) ^ (lane & 7);
                *reinterpret_cast<uint4*>(my_staging + lane * 128 + piece * 16) =
                    make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
            }
        }
        if (kKind == 2) continue;                        // codes and scale bytes were written directly
        __syncwarp();
        const int col0 = (kKind == 0 ? nb * 128 : nb * kBlockN) + seg_idx * 64;   // first output column of the segment
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + (lane >> 3), piece = lane & 7;
            const uint4 v = *reinterpret_cast<const uint4*>(my_staging + r * 128 + ((piece ^ (r & 7)) * 16));
            if (kKind == 0) {
                if (q * 32 + r < valid) {
                    uint8_t* o = reinterpret_cast<uint8_t*>(p.act_bf16) +
                                 (static_cast<int64_t>(mb * kBlockM + q * 32 + r) * p.n_out + col0) * 2 + piece * 16;
                    *reinterpret_cast<uint4*>(o) = v;
                }
            } else {
                const uint64_t rp = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(out_ptr), r);
                if (rp != 0 && col0 < p.n_out)
                    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(rp) + static_cast<int64_t>(col0) * 2 + piece * 16) = v;
            }
        }
        __syncwarp();
    }
    if (kKind == 0 && row_ok) atomicMax(p.row_amax + row, __float_as_uint(amax));
}

template <int kKind>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];   // the swizzled operand tiles need 1024-byte alignment
    const uint32_t smem_base = smem_u32(smem_raw);
    uint8_t* smem_gen = smem_raw;
    if ((smem_base & 1023u) != 0u) {                         // never expected; refuse to run rather than compute garbage
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, MM_ERR_PIPE_TIMEOUT) == 0) { p.status[1] = 100 + kKind; p.status[2] = blockIdx.x; }
        return;
    }
    // layout: [stages x (A | B)] [staging] [scales] [barriers]
    const uint32_t staging_u32 = smem_base + kStages * kStageBytes;
    uint8_t* staging_gen = smem_gen + kStages * kStageBytes;
    float* scales_gen = reinterpret_cast<float*>(staging_gen + kStagingBytes);
    const uint32_t bars = staging_u32 + kStagingBytes + kScaleBytes;
    // barrier slots (8 bytes each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kStages + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * kStages + 2 + a); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kStages * kStageBytes + kStagingBytes + kScaleBytes + 8 * (2 * kStages + 4));
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + kStages * kStageBytes + kStagingBytes + kScaleBytes + 8 * (2 * kStages + 4) + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), kEpilogueWarps); }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // after a failed bounded wait earlier in the call (status code set) the plan is not trustworthy: run no tile
    const int num_mblocks = p.status[0] != 0 ? 0 : p.plan[0];
    const int num_tiles = num_mblocks * p.n_blocks;
    const int k_blocks = p.kdim / kBlockK;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one thread)
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
                const int mb = tile / p.n_blocks, nb = tile - mb * p.n_blocks;
                if (p.mblock_valid[mb] == 0) continue;       // an m-block of padding rows only (plain grouped GEMM); all roles skip it
                const int e = p.mblock_expert[mb];
                const int a_row = mb * kBlockM;
                // weights are stored tile by tile in the order this kernel consumes them:
                // [expert][n block][k block][256 rows][128 B] -- one TMA box = one contiguous 32 KiB block, and the k blocks
                // of one output tile follow each other, so each CTA streams one sequential run of HBM per tile
                const int b_tile0 = (e * p.n_blocks + nb) * k_blocks;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.timeout_ns)) { alive = false; break; }
                    const uint32_t a_dst = smem_base + stage * kStageBytes;
                    const uint32_t b_dst = a_dst + kABytes;
                    mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
                    tma_load_2d(a_dst, &tm_a, kb * kBlockK, a_row, full_bar(stage));
                    tma_load_2d(b_dst, &tm_b, 0, (b_tile0 + kb) * kBlockN, full_bar(stage));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f8(kBlockM, kBlockN);
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
                if (p.mblock_valid[tile / p.n_blocks] == 0) continue;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.timeout_ns)) { alive = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBlockN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.timeout_ns)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t a_src = smem_base + stage * kStageBytes;
                    const uint64_t da = umma_desc_k_sw128(a_src);
                    const uint64_t db = umma_desc_k_sw128(a_src + kABytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / 32; ++k) {
                        // advance 32 bytes of K inside the swizzle atom: +2 in the (address >> 4) field
                        umma_f8(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));            // smem stage is free once these MMAs retire
                    if (kb == k_blocks - 1) umma_commit(tfull_bar(acc));   // accumulator complete
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..9)
        // Two warps per TMEM lane quarter: warp 2+q (half 0) and warp 6+q (half 1) split the tile's columns, so every
        // scheduler has two epilogue warps to interleave (one warp alone cannot hide its own ALU/MUFU latencies).
        const int q = warp & 3;                       // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;             // which half of the tile's output columns
        const int et = q * 32 + lane;                 // row of the tile == TMEM lane
        uint8_t* my_staging = staging_gen + (warp - 2) * kStagingWarpBytes;
        const bool do_clamp = p.clamp < 3.0e38f;
        int acc = 0; uint32_t acc_phase = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
            if (*abort_flag != 0) break;
            const int mb = tile / p.n_blocks, nb = tile - mb * p.n_blocks;
            const int e = p.mblock_expert[mb];
            const int valid = p.mblock_valid[mb];
            if (valid == 0) continue;
            const int row = mb * kBlockM + et;
            const bool row_ok = et < valid;
            float* sc = scales_gen + acc * kBlockN;
            // stage the 256 per-column weight scales of this tile (one per epilogue thread)
            {
                const int t = (warp - 2) * 32 + lane;
                const float* ws = p.w_scale + static_cast<int64_t>(e) * p.w_rows_per_expert;
                if (kKind != 1) {
                    sc[t] = t < 128 ? ws[nb * 128 + t] : ws[p.w_rows_per_expert / 2 + nb * 128 + (t - 128)];
                } else {
                    const int c0 = nb * kBlockN + t;
                    sc[t] = c0 < p.n_out ? ws[c0] : 0.0f;
                }
            }
            named_bar_sync(1, kEpilogueThreads);
            float row_scale = 0.0f, route_w = 0.0f;
            uint8_t* out_ptr = nullptr;                // kind 1: destination row in the source rank's combine buffer
            if (row_ok) {
                if (kKind != 1) {
                    const MmPoolMeta m = p.meta[row];
                    row_scale = m.x_scale;
                    route_w = m.route_weight;
                } else if (p.out_rows != nullptr) {     // plain grouped GEMM: row scale and a local output row
                    row_scale = p.act_scale[row];
                    out_ptr = reinterpret_cast<uint8_t*>(p.out_rows) + static_cast<int64_t>(row) * p.n_out * 2;
                } else {
                    const MmPoolMeta m = p.meta[row];
                    row_scale = p.act_scale[row];
                    out_ptr = combine_row_ptr(p, m.src_info, m.src_token);
                }
            }
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.timeout_ns)) { alive = false; break; }
            tc_fence_after();
            epilogue_math<kKind>(p, tmem_base, sc, my_staging, lane, q, half, acc, mb, nb, valid, row, row_ok, row_scale, route_w,
                                 out_ptr, do_clamp);
            // accumulator buffer may be overwritten by the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag != 0) {
        // a bounded wait expired: give copies that may still be in flight time to land, then report
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 1000000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, MM_ERR_PIPE_TIMEOUT) == 0) {
            p.status[1] = kKind; p.status[2] = blockIdx.x; p.status[3] = num_tiles; p.status[4] = 0;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace mm
