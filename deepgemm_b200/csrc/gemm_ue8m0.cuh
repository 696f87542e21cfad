// GEMM2 of the UE8M0 recipe: activations are e4m3 codes with one power-of-two scale per (row, 32 columns), the weights keep
// their fp32 per-output-channel scales.  The block scales are applied by the tensor core itself
// (tcgen05.mma kind::mxf8f6f4.block_scale, scale factors in TMEM), so there is no bf16 round trip and no requantisation
// pass between the two GEMMs -- the recipe of the reference's Blackwell kernel
// (deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:839-870 copies scale factors to TMEM and issues the
// block-scaled MMA; :1023-1057 produces the per-32 scales), here with FP8 weights and channelwise weight scales.
//
//   out[row, h] = bf16( (sum_kb 2^e[row, kb] * sum_{k in kb} aq[row, k] * w2q[h, k]) * sw2[h] )
//
// Tile = 128 pool rows x 128 weight rows x 128 bytes of K per stage (four K=32 MMAs, each with its own scale byte); two
// 128-column accumulators; the scale factors of a stage (512 bytes: 128 rows x 4 blocks) travel with the operands through
// the ring and are copied to TMEM with tcgen05.cp right before the stage's MMAs.  The weights' scale factors are a
// constant 1.0 (byte 127).  Same warp roles and bounded waits as grouped_gemm_kernel.
#pragma once
#include "gemm.cuh"

namespace mm {

constexpr int kU8BlockN = 128;
constexpr int kU8Stages = 5;
constexpr int kU8ABytes = kBlockM * kBlockK;          // 16 KiB
constexpr int kU8BBytes = kU8BlockN * kBlockK;        // 16 KiB
constexpr int kU8SfBytes = 512;                       // scale bytes of 128 rows x 4 K blocks
constexpr int kU8StageBytes = kU8ABytes + kU8BBytes;
constexpr int kU8SmemBytes = kU8Stages * (kU8StageBytes + kU8SfBytes) + kU8SfBytes /*weights' 1.0*/ + kStagingBytes +
                             2 * kU8BlockN * 4 /*scales*/ + 256 /*barriers*/;
static_assert(kU8SmemBytes <= 232448, "exceeds the 227 KiB of shared memory a CTA can have");
// TMEM columns: accumulators [0, 256), activation scale factors of stage s at 256 + 4 s, weight scale factors at 288
constexpr uint32_t kU8TmemSfa = 256, kU8TmemSfb = 288;

// Instruction descriptor, kind::mxf8f6f4.block_scale: A = B = e4m3 K-major, scale format E8M0, shape M x N.
//   [4,6) B scale-factor byte | [7,10) A format (0 = e4m3) | [10,13) B format | [17,23) N >> 3 | [23] scale format (1 = E8M0) |
//   [24,29) M >> 4 | [29,31) A scale-factor byte
__host__ __device__ constexpr uint32_t umma_idesc_f8_block_scaled(uint32_t m, uint32_t n, uint32_t a_sf_id, uint32_t b_sf_id) {
    return (b_sf_id << 4) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (a_sf_id << 29);
}
// Shared-memory descriptor of a scale-factor block for tcgen05.cp: no swizzle, 8-row groups of 16 bytes 128 B apart.
__device__ __forceinline__ uint64_t umma_desc_sf(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(128u >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    return d;
}
// 32 lanes x 128 bits from shared memory into TMEM, replicated to the four lane quarters (scale factors of 128 rows).
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_f8_block_scaled(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate,
                                                     uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}
// untiled bulk copy global -> shared (16-byte aligned, size a multiple of 16) counted on an mbarrier
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// tm_a: activations e4m3 [pool_rows][I], box 128 rows; tm_b: tiled W2 [E][H/256][I/128][256][128 B] as a 128-byte-wide matrix,
// box 128 rows (one half of a 256-row block).  p.kdim = I, p.n_blocks = H / 128, p.n_out = H, p.act_sf as written by
// grouped_gemm_kernel<2>, p.w_scale = sw2.
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_ue8m0_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    uint8_t* smem_gen = smem_raw;
    if ((smem_base & 1023u) != 0u) {
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, MM_ERR_PIPE_TIMEOUT) == 0) { p.status[1] = 103; p.status[2] = blockIdx.x; }
        return;
    }
    // layout: [stages x (A | B)] [stages x SF] [SF of the weights] [staging] [scales] [barriers]
    constexpr int kSfOff = kU8Stages * kU8StageBytes;
    constexpr int kSfbOff = kSfOff + kU8Stages * kU8SfBytes;
    constexpr int kStagingOff = kSfbOff + kU8SfBytes;
    constexpr int kScaleOff = kStagingOff + kStagingBytes;
    constexpr int kBarOff = kScaleOff + 2 * kU8BlockN * 4;
    uint8_t* staging_gen = smem_gen + kStagingOff;
    float* scales_gen = reinterpret_cast<float*>(smem_gen + kScaleOff);
    const uint32_t bars = smem_base + kBarOff;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kU8Stages + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * kU8Stages + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * kU8Stages + 2 + a); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kBarOff + 8 * (2 * kU8Stages + 4));
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + kBarOff + 8 * (2 * kU8Stages + 4) + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kU8Stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), kEpilogueWarps); }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
    }
    // the weights' scale factors: 1.0 everywhere (written by ordinary stores, read by the tensor core's copy unit)
    for (int i = threadIdx.x; i < kU8SfBytes / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem_gen + kSfbOff)[i] = 0x7f7f7f7fu;
    fence_proxy_async_smem();
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_mblocks = p.status[0] != 0 ? 0 : p.plan[0];
    const int num_tiles = num_mblocks * p.n_blocks;
    const int k_blocks = p.kdim / kBlockK;
    const int nb256 = (p.n_out + 255) / 256;           // 256-row blocks of the tiled weight layout per expert

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one thread)
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
                const int mb = tile / p.n_blocks, nb = tile - mb * p.n_blocks;
                if (p.mblock_valid[mb] == 0) continue;
                const int e = p.mblock_expert[mb];
                const int b_row0 = ((e * nb256 + (nb >> 1)) * k_blocks) * 256 + (nb & 1) * 128;   // + kb * 256
                const uint8_t* sf_src = p.act_sf + static_cast<int64_t>(mb) * k_blocks * kU8SfBytes;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.timeout_ns)) { alive = false; break; }
                    const uint32_t a_dst = smem_base + stage * kU8StageBytes;
                    mbar_arrive_expect_tx(full_bar(stage), kU8StageBytes + kU8SfBytes);
                    tma_load_2d(a_dst, &tm_a, kb * kBlockK, mb * kBlockM, full_bar(stage));
                    tma_load_2d(a_dst + kU8ABytes, &tm_b, 0, b_row0 + kb * 256, full_bar(stage));
                    bulk_load(smem_base + kSfOff + stage * kU8SfBytes, sf_src + static_cast<int64_t>(kb) * kU8SfBytes, kU8SfBytes, full_bar(stage));
                    if (++stage == kU8Stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one thread)
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool alive = true;
            tmem_cp_sf(tmem_base + kU8TmemSfb, umma_desc_sf(smem_base + kSfbOff));      // once: the weights' 1.0
            for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
                if (p.mblock_valid[tile / p.n_blocks] == 0) continue;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.timeout_ns)) { alive = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kU8BlockN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, p.timeout_ns)) { alive = false; break; }
                    tc_fence_after();
                    const uint32_t a_src = smem_base + stage * kU8StageBytes;
                    const uint64_t da = umma_desc_k_sw128(a_src);
                    const uint64_t db = umma_desc_k_sw128(a_src + kU8ABytes);
                    const uint32_t t_sfa = tmem_base + kU8TmemSfa + 4u * stage;
                    tmem_cp_sf(t_sfa, umma_desc_sf(smem_base + kSfOff + stage * kU8SfBytes));
#pragma unroll
                    for (int k = 0; k < kBlockK / 32; ++k) {
                        umma_f8_block_scaled(d_tmem, da + 2u * k, db + 2u * k, umma_idesc_f8_block_scaled(kBlockM, kU8BlockN, k, 0),
                                             (kb | k) != 0 ? 1u : 0u, t_sfa, tmem_base + kU8TmemSfb);
                    }
                    umma_commit(empty_bar(stage));
                    if (kb == k_blocks - 1) umma_commit(tfull_bar(acc));
                    if (++stage == kU8Stages) { stage = 0; phase ^= 1u; }
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..9)
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;             // columns [64 half, 64 half + 64) of the tile
        const int et = q * 32 + lane;
        uint8_t* my_staging = staging_gen + (warp - 2) * kStagingWarpBytes;
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
            float* sc = scales_gen + acc * kU8BlockN;
            {
                const int t = (warp - 2) * 32 + lane;
                if (t < kU8BlockN) {
                    const int c0 = nb * kU8BlockN + t;
                    sc[t] = c0 < p.n_out ? p.w_scale[static_cast<int64_t>(e) * p.w_rows_per_expert + c0] : 0.0f;
                }
            }
            named_bar_sync(1, kEpilogueThreads);
            uint8_t* out_ptr = nullptr;
            if (row_ok) {
                const MmPoolMeta m = p.meta[row];
                out_ptr = combine_row_ptr(p, m.src_info, m.src_token);
            }
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.timeout_ns)) { alive = false; break; }
            tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kU8BlockN + half * 64;
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                uint32_t a[32];
                tmem_ld_32x32(t_addr + sub * 32, a);
                tmem_ld_wait();
                uint32_t packed[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2)
                    packed[j / 2] = pack_bf16x2(__uint_as_float(a[j]) * sc[half * 64 + sub * 32 + j],
                                                __uint_as_float(a[j + 1]) * sc[half * 64 + sub * 32 + j + 1]);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const int piece = (sub * 4 + v) ^ (lane & 7);
                    *reinterpret_cast<uint4*>(my_staging + lane * 128 + piece * 16) =
                        make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                }
            }
            __syncwarp();
            const int col0 = nb * kU8BlockN + half * 64;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int r = it * 4 + (lane >> 3), piece = lane & 7;
                const uint4 v = *reinterpret_cast<const uint4*>(my_staging + r * 128 + ((piece ^ (r & 7)) * 16));
                const uint64_t rp = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(out_ptr), r);
                if (rp != 0 && col0 < p.n_out)
                    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(rp) + static_cast<int64_t>(col0) * 2 + piece * 16) = v;
            }
            __syncwarp();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }

    if (*abort_flag != 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 1000000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, MM_ERR_PIPE_TIMEOUT) == 0) {
            p.status[1] = 3; p.status[2] = blockIdx.x; p.status[3] = num_tiles; p.status[4] = 0;
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
