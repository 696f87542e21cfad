// The two compute pieces of the reference's SPLIT baseline (DeepEP dispatch -> grouped GEMM -> SwiGLU + quantise ->
// grouped GEMM -> gather, tests/test_mega_moe_dcu.py:188-300), so that baseline can be run on B200 next to the fused
// layer:
//   * the plan of an m-grouped contiguous GEMM (rows grouped by expert, every group padded to 128 rows, m_indices[row] =
//     expert or -1): per 128-row block its expert and its number of valid rows, for grouped_gemm_kernel<1> with local output
//     rows.  Stands in for the external deepgemm.m_grouped_fp8_gemm_nt_contiguous the reference's test calls
//     (tests/test_mega_moe_dcu.py:245-250, 274-279) with per-row / per-output-channel fp32 scales.
//   * swiglu_quant_channelwise_kernel: the reference's K2 kernel
//     (megamoe/dcu_megamoe_large_opt/K2_fused/k2_fused_ext.cu:254-377): bf16 [rows][2I] (gate | up) -> e4m3 [rows][I] with
//     one scale per row, optional bf16 copy.  Same arithmetic and order of operations as the reference kernel.
#pragma once
#include <cuda_bf16.h>
#include "layout.h"
#include "misc.cuh"

namespace mm {

constexpr int MM_ERR_BAD_GROUP_LAYOUT = 5;     // a 128-row block of an m-grouped GEMM mixes experts or has a hole

// One warp per 128-row block.  work: [0..15] status words (MmStatus), [16..31] plan ([16] = number of blocks),
// [32 .. 32+blocks) expert of the block, [32+blocks .. 32+2*blocks) valid rows of the block.
__global__ void __launch_bounds__(256) mgroup_plan_kernel(const int* __restrict__ m_indices, int rows, int num_experts, int* __restrict__ work) {
    const int blocks = rows / MM_BLOCK_M;
    const int lane = threadIdx.x & 31;
    const int mb = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (blockIdx.x == 0 && threadIdx.x == 0) work[16] = blocks;
    if (mb >= blocks) return;
    const int first = m_indices[mb * MM_BLOCK_M];
    int valid = 0;
    bool bad = first >= num_experts;
    bool seen_pad = false;
    for (int r0 = 0; r0 < MM_BLOCK_M; r0 += 32) {
        const int e = m_indices[mb * MM_BLOCK_M + r0 + lane];
        const unsigned ok = __ballot_sync(0xffffffffu, e >= 0);
        const unsigned same = __ballot_sync(0xffffffffu, e < 0 || e == first);
        // valid rows must form a prefix of the block and share one expert
        if (same != 0xffffffffu) bad = true;
        if (ok != 0u && (seen_pad || (ok & (ok + 1u)) != 0u)) bad = true;
        if (ok != 0xffffffffu) seen_pad = true;
        valid += __popc(ok);
    }
    if (lane == 0) {
        work[32 + mb] = first >= 0 && first < num_experts ? first : 0;
        work[32 + blocks + mb] = bad ? 0 : valid;
        if (bad && atomicCAS(work, 0, MM_ERR_BAD_GROUP_LAYOUT) == 0) { work[1] = 0; work[2] = mb; work[3] = first; work[4] = valid; }
    }
}

// grid-stride over rows, one block per row at a time.  y = gate * (1 / (1 + exp(-gate))) * up * weight in fp32 with the
// reference's clamp (up two-sided, gate from above only); scale = max(amax, 1e-4) / 448; codes = e4m3(y * (448 / max(amax,
// 1e-4))), saturating.  A row whose weight is 0 gets zero codes and scale 1e-4 / 448.  Rows whose row_combine_ptrs entry
// is 0 are left untouched (only when no bf16 copy is asked for), as in the reference.
__global__ void __launch_bounds__(256) swiglu_quant_channelwise_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ weights,
                                                                      const int64_t* __restrict__ row_combine_ptrs,
                                                                      uint8_t* __restrict__ out_fp8, float* __restrict__ out_scale,
                                                                      __nv_bfloat16* __restrict__ out_bf16, int rows, int inter,
                                                                      int has_clamp, float clamp_value) {
    __shared__ float red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int quads = inter / 4;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        if (out_bf16 == nullptr && row_combine_ptrs != nullptr && row_combine_ptrs[row] == 0) continue;
        const float w = weights ? weights[row] : 1.0f;
        uint32_t* o8 = reinterpret_cast<uint32_t*>(out_fp8 + static_cast<int64_t>(row) * inter);
        uint2* o16 = out_bf16 ? reinterpret_cast<uint2*>(out_bf16 + static_cast<int64_t>(row) * inter) : nullptr;
        if (weights && w == 0.0f) {
            if (tid == 0) out_scale[row] = 1.0e-4f / 448.0f;
            for (int v = tid; v < quads; v += blockDim.x) {
                o8[v] = 0u;
                if (o16) o16[v] = make_uint2(0u, 0u);
            }
            continue;
        }
        const uint2* g2 = reinterpret_cast<const uint2*>(x + static_cast<int64_t>(row) * inter * 2);
        const uint2* u2 = g2 + quads;
        auto value = [&](uint32_t gbits, uint32_t ubits, bool hi) {
            float g = hi ? bf16_hi(gbits) : bf16_lo(gbits);
            float u = hi ? bf16_hi(ubits) : bf16_lo(ubits);
            if (has_clamp) {
                u = fminf(clamp_value, fmaxf(-clamp_value, u));
                g = fminf(clamp_value, g);
            }
            const float sig = __fdiv_rn(1.0f, 1.0f + __expf(-g));
            return __fmul_rn(__fmul_rn(__fmul_rn(g, sig), u), w);
        };
        float amax = 0.0f;
        for (int v = tid; v < quads; v += blockDim.x) {
            const uint2 g = g2[v], u = u2[v];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(value(g.x, u.x, false)), fabsf(value(g.x, u.x, true))),
                                     fmaxf(fabsf(value(g.y, u.y, false)), fabsf(value(g.y, u.y, true)))));
        }
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        __syncthreads();                    // the previous row's readers of red[] are done
        if (lane == 0) red[warp] = amax;
        __syncthreads();
        amax = red[0];
        for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
        const float clamped = fmaxf(amax, 1.0e-4f);
        const float inv = __fdiv_rn(448.0f, clamped);
        if (tid == 0) out_scale[row] = __fdiv_rn(clamped, 448.0f);
        for (int v = tid; v < quads; v += blockDim.x) {
            const uint2 g = g2[v], u = u2[v];
            const float y0 = value(g.x, u.x, false), y1 = value(g.x, u.x, true), y2 = value(g.y, u.y, false), y3 = value(g.y, u.y, true);
            o8[v] = pack4_e4m3(y0 * inv, y1 * inv, y2 * inv, y3 * inv);
            if (o16) {
                __nv_bfloat162 a = __floats2bfloat162_rn(y0, y1), b = __floats2bfloat162_rn(y2, y3);
                o16[v] = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
            }
        }
    }
}

}  // namespace mm
