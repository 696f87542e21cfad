// DeepEP-layout helpers: scatter received tokens into expert-grouped rows before a grouped GEMM, and gather / sum the
// per-route outputs back per token.  They reproduce csrc/kernels/mega_moe_baseline_hip.cu:37-127 of the reference (the
// pre/post-processing of its split DeepEP + grouped-GEMM baseline) so that baseline can be rebuilt on B200.
// One refinement: rows inside an expert are in route order (token-major), where the reference takes whatever order
// atomicAdd produces (mega_moe_baseline_hip.cu:75).
#pragma once
#include <cuda_bf16.h>
#include "misc.cuh"

namespace mm {

template <typename TopkT>
__device__ __forceinline__ int deepep_expert_of(const void* ids, int64_t route) {
    return static_cast<int>(reinterpret_cast<const TopkT*>(ids)[route]);
}

// grid = 1, block = 1024: exclusive prefix of num_recv_tokens_per_expert (mega_moe_baseline_hip.cu:37-48).
__global__ void __launch_bounds__(1024) deepep_prefix_kernel(const int* __restrict__ counts, int* __restrict__ start, int num_experts) {
    __shared__ int buf[1024];
    int run = 0;
    for (int base = 0; base < num_experts; base += 1024) {
        const int e = base + threadIdx.x;
        const int c = e < num_experts ? counts[e] : 0;
        buf[threadIdx.x] = c;
        __syncthreads();
        for (int o = 1; o < 1024; o <<= 1) {
            const int v = threadIdx.x >= o ? buf[threadIdx.x - o] : 0;
            __syncthreads();
            buf[threadIdx.x] += v;
            __syncthreads();
        }
        if (e < num_experts) start[e] = run + buf[threadIdx.x] - c;
        run += buf[1023];
        __syncthreads();
    }
}

// One warp per expert: walk all routes in order and hand out the expert's rows in that order.
// output_index must be pre-filled with -1 (routes with an expert id outside [0, num_experts) keep it).
template <typename TopkT>
__global__ void __launch_bounds__(256) deepep_assign_kernel(const void* __restrict__ ids, const int* __restrict__ start,
                                                           int* __restrict__ output_index, int* __restrict__ m_indices,
                                                           int64_t num_routes, int num_experts, int total_rows) {
    const int lane = threadIdx.x & 31;
    const int e = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (e >= num_experts) return;
    int next = start[e];
    for (int64_t r0 = 0; r0 < num_routes; r0 += 32) {
        const int64_t r = r0 + lane;
        const bool mine = r < num_routes && deepep_expert_of<TopkT>(ids, r) == e;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (mine) {
            const int row = next + __popc(m & ((1u << lane) - 1u));
            const int dst = row < total_rows ? row : -1;
            output_index[r] = dst;
            if (dst >= 0) m_indices[dst] = e;
        }
        next += __popc(m);
    }
}

// One warp per route: copy the FP8 row and its scale / weight to the assigned grouped row.
__global__ void __launch_bounds__(256) deepep_scatter_rows_kernel(const uint8_t* __restrict__ recv_x, const float* __restrict__ recv_x_scale,
                                                                 const float* __restrict__ recv_topk_weights, const int* __restrict__ output_index,
                                                                 uint8_t* __restrict__ grouped_x, float* __restrict__ grouped_x_scale,
                                                                 float* __restrict__ route_weights, int64_t num_routes, int topk, int hidden) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t r = warp; r < num_routes; r += nwarps) {
        const int dst = output_index[r];
        if (dst < 0) continue;
        const int64_t token = r / topk;
        const uint4* src = reinterpret_cast<const uint4*>(recv_x + token * hidden);
        uint4* out = reinterpret_cast<uint4*>(grouped_x + static_cast<int64_t>(dst) * hidden);
        for (int v = lane; v < hidden / 16; v += 32) out[v] = src[v];
        if (lane == 0) {
            grouped_x_scale[dst] = recv_x_scale[token];
            route_weights[dst] = recv_topk_weights[r];
        }
    }
}

// recv_y[token] = bf16( sum over slots of l2_out[output_index[token, slot]] (* weight) ), fp32 sum in slot order
// (mega_moe_baseline_hip.cu:100-127).  Grid-stride over (token, 8-element vector).
template <typename TopkT>
__global__ void __launch_bounds__(256) deepep_gather_kernel(__nv_bfloat16* __restrict__ recv_y, const __nv_bfloat16* __restrict__ l2_out,
                                                           const void* __restrict__ ids, const float* __restrict__ recv_topk_weights,
                                                           const int* __restrict__ output_index, int recv_rows, int topk, int hidden,
                                                           int apply_topk_weights) {
    const int vecs = hidden / 8;
    const int64_t total = static_cast<int64_t>(recv_rows) * vecs;
    const uint4* src = reinterpret_cast<const uint4*>(l2_out);
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t token = i / vecs;
        const int v = static_cast<int>(i - token * vecs);
        float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int s = 0; s < topk; ++s) {
            const int64_t route = token * topk + s;
            const int row = output_index[route];
            if (deepep_expert_of<TopkT>(ids, route) < 0 || row < 0) continue;
            const float w = apply_topk_weights ? recv_topk_weights[route] : 1.0f;
            const uint4 d = src[static_cast<int64_t>(row) * vecs + v];
            // multiply, round, then add (no fused multiply-add), as the reference's `value *= w; sum += value`
            const float t[8] = {bf16_lo(d.x), bf16_hi(d.x), bf16_lo(d.y), bf16_hi(d.y), bf16_lo(d.z), bf16_hi(d.z), bf16_lo(d.w), bf16_hi(d.w)};
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] = __fadd_rn(a[j], __fmul_rn(t[j], w));
        }
        uint4 o;
        __nv_bfloat162 b;
        b = __floats2bfloat162_rn(a[0], a[1]); o.x = *reinterpret_cast<uint32_t*>(&b);
        b = __floats2bfloat162_rn(a[2], a[3]); o.y = *reinterpret_cast<uint32_t*>(&b);
        b = __floats2bfloat162_rn(a[4], a[5]); o.z = *reinterpret_cast<uint32_t*>(&b);
        b = __floats2bfloat162_rn(a[6], a[7]); o.w = *reinterpret_cast<uint32_t*>(&b);
        reinterpret_cast<uint4*>(recv_y)[i] = o;
    }
}

}  // namespace mm
