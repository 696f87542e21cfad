// HBM-bound elementwise stages: per-token FP8 quantisation, activation requantisation, top-k combine reduce.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include "layout.h"
#include "ptx.cuh"
#include "route.cuh"

namespace mm {

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Per-row FP8 quantisation, bit-exact with megamoe/__init__.py:51-56 (cast_to_fp8_channelwise):
//   scale = max(amax|x|, 1e-4) / 448 ; q = e4m3_rne(float(x) / scale)   (true IEEE divisions, as torch does).
// One warp per row; k % 8 == 0.  The second pass re-reads the row (L1/L2 hit).
__global__ void __launch_bounds__(256) quant_per_token_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int k,
                                                             uint8_t* __restrict__ q, float* __restrict__ scale) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const int vecs = k / 8;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const uint4* src = reinterpret_cast<const uint4*>(x + r * k);
        float amax = 0.0f;
        for (int v = lane; v < vecs; v += 32) {
            const uint4 d = src[v];
            const uint32_t w[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(w[i])), fabsf(bf16_hi(w[i]))));
        }
        amax = warp_max(amax);
        const float s = __fdiv_rn(fmaxf(amax, 1.0e-4f), 448.0f);
        if (lane == 0) scale[r] = s;
        uint2* dst = reinterpret_cast<uint2*>(q + r * k);
        for (int v = lane; v < vecs; v += 32) {
            const uint4 d = src[v];
            uint2 o;
            o.x = pack4_e4m3(__fdiv_rn(bf16_lo(d.x), s), __fdiv_rn(bf16_hi(d.x), s), __fdiv_rn(bf16_lo(d.y), s), __fdiv_rn(bf16_hi(d.y), s));
            o.y = pack4_e4m3(__fdiv_rn(bf16_lo(d.z), s), __fdiv_rn(bf16_hi(d.z), s), __fdiv_rn(bf16_lo(d.w), s), __fdiv_rn(bf16_hi(d.w), s));
            dst[v] = o;
        }
    }
}

// Activation requantisation after GEMM1 (deep_gemm/include/deep_gemm/impls/mega_moe_dcu_tiles.cuh:672-733):
//   s2 = max(amax / 448, 1e-4) ; aq = e4m3(a * (1 / s2)).  The row amax was accumulated by the GEMM1 epilogue
// (atomicMax on the bit pattern); it is reset here so the next call starts from zero.
// One block per 128-row m-block (grid-stride): the block reads the m-block's valid-row count and its 128 row amax
// values with one coalesced load, then each warp streams two rows at a time (16 independent 16-byte loads per lane).
__global__ void __launch_bounds__(256) requant_kernel(const __nv_bfloat16* __restrict__ act, int inter,
                                                     const int* __restrict__ plan, const int* __restrict__ mblock_valid,
                                                     unsigned int* __restrict__ row_amax, float* __restrict__ act_scale,
                                                     uint8_t* __restrict__ act_q, const int* __restrict__ status) {
    __shared__ float s_inv[MM_BLOCK_M];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int num_mblocks = status[0] != 0 ? 0 : plan[0];     // nothing to do after a failed bounded wait
    const int vecs = inter / 8;
    for (int mb = blockIdx.x; mb < num_mblocks; mb += gridDim.x) {
        const int valid = mblock_valid[mb];
        __syncthreads();
        if (threadIdx.x < MM_BLOCK_M && static_cast<int>(threadIdx.x) < valid) {
            const int64_t r = static_cast<int64_t>(mb) * MM_BLOCK_M + threadIdx.x;
            const float amax = __uint_as_float(row_amax[r]);
            row_amax[r] = 0u;
            const float s = fmaxf(__fdiv_rn(amax, 448.0f), 1.0e-4f);
            act_scale[r] = s;
            s_inv[threadIdx.x] = __fdiv_rn(1.0f, s);
        }
        __syncthreads();
        for (int r0 = warp * 2; r0 < valid; r0 += 16) {
            uint4 buf[2][8];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int64_t r = static_cast<int64_t>(mb) * MM_BLOCK_M + r0 + k;
                const uint4* src = reinterpret_cast<const uint4*>(act + r * inter);
                if (r0 + k < valid) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int v = i * 32 + lane;
                        if (v < vecs) buf[k][i] = src[v];
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                if (r0 + k >= valid) continue;
                const int64_t r = static_cast<int64_t>(mb) * MM_BLOCK_M + r0 + k;
                const float inv = s_inv[r0 + k];
                const uint4* src = reinterpret_cast<const uint4*>(act + r * inter);
                uint2* dst = reinterpret_cast<uint2*>(act_q + r * inter);
                for (int v0 = 0; v0 < vecs; v0 += 256) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int v = v0 + i * 32 + lane;
                        if (v < vecs) {
                            const uint4 d = (v0 == 0) ? buf[k][i] : src[v];   // rows longer than 2048 read the rest directly
                            uint2 o;
                            o.x = pack4_e4m3(bf16_lo(d.x) * inv, bf16_hi(d.x) * inv, bf16_lo(d.y) * inv, bf16_hi(d.y) * inv);
                            o.y = pack4_e4m3(bf16_lo(d.z) * inv, bf16_hi(d.z) * inv, bf16_lo(d.w) * inv, bf16_hi(d.w) * inv);
                            dst[v] = o;
                        }
                    }
                }
            }
        }
    }
}

// Top-k combine (deep_gemm/include/deep_gemm/impls/mega_moe_dcu.cuh:706-760):
//   y[t, :] = bf16( sum_{s=0..K-1} f32(combine[t][s][:]) ) in slot order; slots of invalid routes contribute zero.
// The reference zeroes those slots during its route scan; here they are skipped using the same validity rule.
// With several ranks the kernel first does the cross-rank "combine stores done" barrier itself (wait_peers != 0): block 0
// publishes this rank's call epoch to every rank -- the GEMM2 tiles ran in earlier launches of this stream, so their
// remote stores are complete -- and every block waits (bounded) until all ranks have published theirs.  A block only ever
// waits for OTHER ranks' first blocks, never for a block of its own grid.
__global__ void __launch_bounds__(256, 4) combine_reduce_kernel(RouteParams p, __nv_bfloat16* __restrict__ y, int wait_peers,
                                                            int* __restrict__ reset_a, int reset_a_words,
                                                            int* __restrict__ reset_b, int reset_b_words) {
    // Leave the layer kernel's dependency counters zero for the next call (null pointers: nothing to reset).  reset_b are
    // the arrival counters in the symmetric buffer: peers bump them again only after this rank has entered its next call
    // (they wait for its route counts first), which on the stream comes after this kernel.
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < reset_a_words; i += gridDim.x * blockDim.x) reset_a[i] = 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < reset_b_words; i += gridDim.x * blockDim.x) reset_b[i] = 0;
    if (call_failed(p.scratch, p.cl)) return;       // a bounded wait expired earlier in the call: y stays untouched, peers time out
    if (wait_peers && p.R > 1) {
        const int epoch = reinterpret_cast<const int*>(p.scratch + p.cl.epoch)[0];
        if (blockIdx.x == 0 && threadIdx.x < p.R) {
            __threadfence_system();
            int* sig = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(p.peers[threadIdx.x]) + p.sl.signals);
            st_release_sys(sig + MM_BAR_COMBINE * MM_MAX_RANKS + p.rank, epoch);
        }
        const bool ok = wait_rank_signals(p, MM_BAR_COMBINE, epoch);
        if (!__syncthreads_and(ok)) return;
    }
    const uint8_t* sym = p.sym;
    const int E = p.E, K = p.K, H = p.H;
    const int n = route_num_tokens(p);              // a device-side count (graph mode) never exceeds the launch-time count = rows of y
    const int vecs = H / 8;
    const int64_t total = static_cast<int64_t>(n) * vecs;
    const int64_t* topk_idx = reinterpret_cast<const int64_t*>(sym + p.sl.topk_idx);
    const float* topk_w = reinterpret_cast<const float*>(sym + p.sl.topk_weights);
    const uint4* comb = reinterpret_cast<const uint4*>(sym + p.sl.combine);
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(i / vecs), v = static_cast<int>(i - static_cast<int64_t>(t) * vecs);
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int s0 = 0; s0 < K; s0 += 6) {             // up to six slots' loads in flight, summed in slot order
            uint4 buf[6];
            bool ok[6];
            // The slot rows are fetched without waiting for the validity of their routes (a slot nobody wrote holds stale
            // bytes, which are then simply not added): index, weight and row loads are all in flight together.
#pragma unroll
            for (int j = 0; j < 6; ++j) {
                const int s = s0 + j;
                ok[j] = false;
                if (s < K) {
                    buf[j] = __ldcg(comb + (static_cast<int64_t>(t) * K + s) * vecs + v);
                    const int64_t e = topk_idx[static_cast<int64_t>(t) * K + s];
                    const float w = topk_w[static_cast<int64_t>(t) * K + s];
                    ok[j] = e >= 0 && e < E && w != 0.0f;
                }
            }
#pragma unroll
            for (int j = 0; j < 6; ++j) {
                if (!ok[j]) continue;
                const uint4 d = buf[j];
                acc[0] += bf16_lo(d.x); acc[1] += bf16_hi(d.x); acc[2] += bf16_lo(d.y); acc[3] += bf16_hi(d.y);
                acc[4] += bf16_lo(d.z); acc[5] += bf16_hi(d.z); acc[6] += bf16_lo(d.w); acc[7] += bf16_hi(d.w);
            }
        }
        uint4 o;
        __nv_bfloat162 b;
        b = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&b);
        b = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&b);
        b = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&b);
        b = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&b);
        reinterpret_cast<uint4*>(y)[i] = o;
    }
}

}  // namespace mm

namespace mm {

// Upstream of the layer, in one kernel: router top-k + weight normalisation + per-token FP8 quantisation, written
// straight into the symmetric buffer views (x, x_sf, topk_idx, topk_weights).  The reference leaves these steps to the
// caller (torch.topk, softmax over the selected scores, cast_to_fp8_channelwise, four copy_ calls:
// tests/test_mega_moe_dcu.py:491-508).  One warp per token.
//   topk: the K largest logits, ties broken towards the lower expert index, listed in descending order;
//   weights: softmax over the K selected logits (== full softmax renormalised to sum 1).
__global__ void __launch_bounds__(256) router_topk_quant_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ logits,
                                                               int num_tokens, int E, int K, int H, uint8_t* __restrict__ x_q,
                                                               float* __restrict__ x_sf, int64_t* __restrict__ topk_idx,
                                                               float* __restrict__ topk_w) {
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    constexpr int kPer = MM_MAX_EXPERTS / 32;
    for (int t = warp; t < num_tokens; t += nwarps) {
        // ---- router: expert (lane + 32 * i) lives in v[i]
        float v[kPer];
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int e = lane + 32 * i;
            v[i] = e < E ? logits[static_cast<int64_t>(t) * E + e] : -INFINITY;
        }
        float sel_val = 0.0f, denom = 0.0f, top = 0.0f;
        int sel_idx = 0;
        for (int k = 0; k < K; ++k) {
            float best = -INFINITY;
            int best_e = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const int e = lane + 32 * i;
                if (v[i] > best) { best = v[i]; best_e = e; }      // within a lane experts ascend, so '>' keeps the lowest index
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
                if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
            }
            if (k == 0) top = best;
            const float p = expf(best - top);
            denom += p;
            if (lane == k) { sel_val = p; sel_idx = best_e; }
            if ((best_e & 31) == lane) {
#pragma unroll
                for (int i = 0; i < kPer; ++i) if (i == (best_e >> 5)) v[i] = -INFINITY;   // remove the winner
            }
        }
        if (lane < K) {
            topk_idx[static_cast<int64_t>(t) * K + lane] = sel_idx;
            topk_w[static_cast<int64_t>(t) * K + lane] = __fdiv_rn(sel_val, denom);
        }
        // ---- per-token FP8 quantisation (same arithmetic as quant_per_token_kernel)
        const int vecs = H / 8;
        const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(t) * H);
        float amax = 0.0f;
        for (int j = lane; j < vecs; j += 32) {
            const uint4 d = src[j];
            const uint32_t w[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(w[i])), fabsf(bf16_hi(w[i]))));
        }
        amax = warp_max(amax);
        const float s = __fdiv_rn(fmaxf(amax, 1.0e-4f), 448.0f);
        if (lane == 0) x_sf[t] = s;
        uint2* dst = reinterpret_cast<uint2*>(x_q + static_cast<int64_t>(t) * H);
        for (int j = lane; j < vecs; j += 32) {
            const uint4 d = src[j];
            uint2 o;
            o.x = pack4_e4m3(__fdiv_rn(bf16_lo(d.x), s), __fdiv_rn(bf16_hi(d.x), s), __fdiv_rn(bf16_lo(d.y), s), __fdiv_rn(bf16_hi(d.y), s));
            o.y = pack4_e4m3(__fdiv_rn(bf16_lo(d.z), s), __fdiv_rn(bf16_hi(d.z), s), __fdiv_rn(bf16_lo(d.w), s), __fdiv_rn(bf16_hi(d.w), s));
            dst[j] = o;
        }
    }
}

}  // namespace mm
