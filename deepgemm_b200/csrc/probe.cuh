// Measurement aid: the dense FP8 tensor-core rate this GPU sustains for the MMA shape the GEMM kernels use
// (tcgen05.mma.cta_group::1.kind::f8f6f4, M128 x N256 x K32), with operands resident in shared memory and no loads.
// It is the denominator for tensor-bound roofline fractions (the machine-readable peak file only has a bf16 figure).
#pragma once
#include "gemm.cuh"

namespace mm {

// One CTA per SM; lane 0 of warp 0 issues `iters` groups of 8 MMAs (4 per accumulator buffer), committing every group to
// an mbarrier and keeping at most two groups in flight.  flops per CTA = iters * 8 * 2 * 128 * 256 * 32.
// pattern 0: every operand byte 1.0 (few bits toggle: the burst rate); 1: pseudo-random finite e4m3 values of both signs,
// magnitude below 2; 2: e4m3 codes with exponent fields 9..14, random sign and mantissa -- what per-row quantisation of
// N(0,1) data produces.  An MMA takes 128 cycles with all three; the data-dependent power draw differs, and under the
// board's power cap so does the clock (measured: about 4450 / 4100 / 3400 TFLOP/s in a short burst).
__device__ __forceinline__ uint4 probe_fill(int pattern, uint32_t i) {
    if (pattern == 0) return make_uint4(0x38383838u, 0x38383838u, 0x38383838u, 0x38383838u);
    uint32_t v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t h = (i * 4u + j + 1u) * 2654435761u;
        h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
        v[j] = h & 0xBEBEBEBEu;      // bit 0 and bit 6 of every byte clear: finite, magnitude below 2
        if (pattern == 2) {
            uint32_t w = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t byte = (h >> (8 * b)) & 0xFFu;
                const uint32_t e = 9u + (byte >> 3) % 6u;
                w |= ((byte & 0x80u) | (e << 3) | (byte & 7u)) << (8 * b);
            }
            v[j] = w;
        }
    }
    return make_uint4(v[0], v[1], v[2], v[3]);
}

__global__ void __launch_bounds__(128, 1) fp8_mma_peak_kernel(int iters, int* status, int pattern) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    __shared__ __align__(8) uint64_t bar_store[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if ((smem_base & 1023u) != 0u) return;
    // operands: any finite bit pattern will do (0x38 = 1.0 in e4m3)
    for (int i = threadIdx.x; i < (kABytes + kBBytes) / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(smem_raw)[i] = probe_fill(pattern, i);
    const uint32_t bar0 = smem_u32(&bar_store[0]), bar1 = smem_u32(&bar_store[1]);
    if (threadIdx.x == 0) {
        mbar_init(bar0, 1); mbar_init(bar1, 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    fence_proxy_async_smem();            // the generic-proxy stores above are read by the tensor core (async proxy)
    if (warp == 0) { tmem_alloc(smem_u32(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (warp == 0) {
        constexpr uint32_t idesc = umma_idesc_f8(kBlockM, kBlockN);
        const uint64_t da = umma_desc_k_sw128(smem_base);
        const uint64_t db = umma_desc_k_sw128(smem_base + kABytes);
        uint32_t phase[2] = {0, 0};
        bool ok = true;
        for (int it = 0; it < iters && ok; ++it) {
            const int b = it & 1;
            if (it >= 2) {                                   // wait for the group issued two iterations ago
                ok = mbar_wait(b ? bar1 : bar0, phase[b], &abort_flag, 2000000000ull);
                phase[b] ^= 1u;
            }
            if (lane == 0 && ok) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    umma_f8(tmem_base + (j >> 2) * kBlockN, da + 2u * (j & 3), db + 2u * (j & 3), idesc, 1u);
                umma_commit(b ? bar1 : bar0);
            }
            __syncwarp();
        }
        for (int b = 0; b < 2 && ok; ++b) {                  // drain
            if (iters > b) ok = mbar_wait(((iters - 1 - b) & 1) ? bar1 : bar0, phase[(iters - 1 - b) & 1], &abort_flag, 2000000000ull);
        }
        if (!ok && lane == 0) atomicCAS(status, 0, MM_ERR_PIPE_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// The same measurement for the CTA-pair form (tcgen05.mma.cta_group::2, M256 x N256 x K32 across two SMs): one thread
// of each pair's leader issues the MMAs; the commit arrives on the barriers of both CTAs.  Operands per CTA: 128 rows of
// A and 128 of the 256 rows of B.  flops per CTA are the same as above.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) fp8_mma_peak_pair_kernel(int iters, int* status, int pattern) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    __shared__ __align__(8) uint64_t bar_store[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool leader = cluster_ctarank() == 0;
    if ((smem_base & 1023u) != 0u) return;
    for (int i = threadIdx.x; i < (kABytes + kBBytes / 2) / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(smem_raw)[i] = probe_fill(pattern, i);
    const uint32_t bar0 = smem_u32(&bar_store[0]), bar1 = smem_u32(&bar_store[1]);
    if (threadIdx.x == 0) {
        mbar_init(bar0, 1); mbar_init(bar1, 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    fence_proxy_async_smem();
    __syncthreads();
    cluster_sync_all();
    if (warp == 0) { tmem_alloc_pair(smem_u32(&tmem_slot), 512); tmem_relinquish_pair(); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (warp == 0 && leader) {
        constexpr uint32_t idesc = umma_idesc_f8(2 * kBlockM, kBlockN);
        const uint64_t da = umma_desc_k_sw128(smem_base);
        const uint64_t db = umma_desc_k_sw128(smem_base + kABytes);
        uint32_t phase[2] = {0, 0};
        bool ok = true;
        for (int it = 0; it < iters && ok; ++it) {
            const int b = it & 1;
            if (it >= 2) {
                ok = mbar_wait(b ? bar1 : bar0, phase[b], &abort_flag, 2000000000ull);
                phase[b] ^= 1u;
            }
            if (lane == 0 && ok) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    umma_f8_pair(tmem_base + (j >> 2) * kBlockN, da + 2u * (j & 3), db + 2u * (j & 3), idesc, 1u);
                umma_commit_pair(b ? bar1 : bar0);
            }
            __syncwarp();
        }
        for (int b = 0; b < 2 && ok; ++b) {
            if (iters > b) ok = mbar_wait(((iters - 1 - b) & 1) ? bar1 : bar0, phase[(iters - 1 - b) & 1], &abort_flag, 2000000000ull);
        }
        if (!ok && lane == 0) atomicCAS(status, 0, MM_ERR_PIPE_TIMEOUT);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 0) { tc_fence_after(); tmem_dealloc_pair(tmem_base, 512); }
}


// Measurement aid: store `vecs` 16-byte vectors into each of `n_dst` destinations (device addresses; with peer-mapped
// addresses this is the plain-store NVLink write rate the dispatch push and the GEMM2 combine stores can at best reach).
// Every warp writes runs of 512 contiguous bytes, round-robin over the destinations, grid-stride.
struct PeerStoreDsts { uint64_t ptr[MM_MAX_RANKS]; };
__global__ void __launch_bounds__(256) peer_store_probe_kernel(PeerStoreDsts d, int n_dst, int64_t vecs) {
    const uint4 v = make_uint4(threadIdx.x, blockIdx.x, 0x5a5a5a5au, 0xa5a5a5a5u);
    const int64_t total = vecs * n_dst;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t run = i >> 5;                    // one 512-byte run per warp iteration
        const int dst = static_cast<int>(run % n_dst);
        const int64_t pos = (run / n_dst) * 32 + (i & 31);
        if (pos < vecs) reinterpret_cast<uint4*>(d.ptr[dst])[pos] = v;
    }
}

}  // namespace mm
