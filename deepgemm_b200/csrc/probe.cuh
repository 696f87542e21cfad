// Measurement aid: the dense FP8 tensor-core rate this GPU sustains for the MMA shape the GEMM kernels use
// (tcgen05.mma.cta_group::1.kind::f8f6f4, M128 x N256 x K32), with operands resident in shared memory and no loads.
// It is the denominator for tensor-bound roofline fractions (the machine-readable peak file only has a bf16 figure).
#pragma once
#include "gemm.cuh"

namespace mm {

// One CTA per SM; lane 0 of warp 0 issues `iters` groups of 8 MMAs (4 per accumulator buffer), committing every group to
// an mbarrier and keeping at most two groups in flight.  flops per CTA = iters * 8 * 2 * 128 * 256 * 32.
__global__ void __launch_bounds__(128, 1) fp8_mma_peak_kernel(int iters, int* status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    __shared__ __align__(8) uint64_t bar_store[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if ((smem_base & 1023u) != 0u) return;
    // operands: any finite bit pattern will do (0x38 = 1.0 in e4m3)
    for (int i = threadIdx.x; i < (kABytes + kBBytes) / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(smem_raw)[i] = make_uint4(0x38383838u, 0x38383838u, 0x38383838u, 0x38383838u);
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

}  // namespace mm
