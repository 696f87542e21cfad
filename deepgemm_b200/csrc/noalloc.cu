// mm_fp8_w8a8_mega_moe_static: the single-rank layer for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at all: an inference server that hands its whole HBM budget to its
// own arena at start-up, a plugin running under a framework that forbids allocation on the serving path because
// cudaMalloc synchronises the device, or a tool that only owns the tensors it was given.  The regular entry point
// needs two caller-allocated work buffers (the "symmetric" buffer and the scratch buffer, a few MiB to several GiB).
// This variant keeps both in one file-scope device array of fixed size instead, so the caller passes nothing but the
// inputs and the output.  The price: the array (MM_STATIC_WORK_BYTES) is part of the library image, every GPU that
// loads the library holds it until the process exits, and only shapes whose work buffers fit are accepted.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/megamoe_b200.h"
#include "layout.h"

namespace {

// Work area shared by every call on a device.  It keeps whatever the previous call left in it.
__device__ __align__(256) unsigned char g_static_work[MM_STATIC_WORK_BYTES];

// g_static_work is, in host code, only a handle for the runtime -- not a device address.  The address a kernel can
// use has to be asked for once per device, with that device current.
std::mutex g_mu;
void* g_work_ptr[64] = {nullptr};
int64_t g_scratch_base[64] = {0};      // where the last call on each device put its scratch region (status words first)

}  // namespace

void mm_detail_set_error(const char* msg);   // defined next to mm_last_error: stores the message that function returns

namespace {

char g_static_err[384];   // formatting buffer, guarded by g_mu only where it is shared; messages are copied out at once

int static_fail(const char* msg) {
    mm_detail_set_error(msg);
    return 1;
}

}  // namespace

extern "C" {

int mm_fp8_w8a8_mega_moe_static(void* y, const void* x_fp8, const float* x_sf, const int64_t* topk_idx,
                                const float* topk_weights, const void* w1, const float* s1, const void* w2, const float* s2,
                                int* stats, int num_tokens, int num_experts, int K, int H, int I, float activation_clamp,
                                void* stream_) {
    if (num_tokens < 0 || num_experts <= 0 || K <= 0 || H <= 0 || I <= 0) return static_fail("mm_fp8_w8a8_mega_moe_static: bad shape");
    if (num_tokens > 0 && (!y || !x_fp8 || !x_sf || !topk_idx || !topk_weights))
        return static_fail("mm_fp8_w8a8_mega_moe_static: null input or output pointer");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int T = ((num_tokens > 0 ? num_tokens : 1) + MM_TOKEN_ALIGNMENT - 1) / MM_TOKEN_ALIGNMENT * MM_TOKEN_ALIGNMENT;
    int64_t sym_off[MM_SYM_NUM_OFFSETS], scr_off[MM_SCR_NUM_OFFSETS], sym_bytes = 0, scr_bytes = 0;
    if (int rc = mm_symm_buffer_layout(1, num_experts, T, K, H, I, sym_off, &sym_bytes)) return rc;   // also validates the shape
    if (int rc = mm_scratch_layout(1, num_experts, T, K, H, I, scr_off, &scr_bytes)) return rc;
    const int64_t scr_base = (sym_bytes + 1023) / 1024 * 1024;
    if (scr_base + scr_bytes > (int64_t)MM_STATIC_WORK_BYTES) {
        char msg[384];
        snprintf(msg, sizeof(msg),
                 "mm_fp8_w8a8_mega_moe_static: this shape needs %lld bytes of work memory, the built-in area holds %lld; "
                 "use mm_fp8_w8a8_mega_moe with caller-allocated buffers",
                 (long long)(scr_base + scr_bytes), (long long)MM_STATIC_WORK_BYTES);
        return static_fail(msg);
    }

    // one-time set-up per device: resolve the device address of the built-in work area
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess || dev < 0 || dev >= 64) return static_fail("mm_fp8_w8a8_mega_moe_static: cudaGetDevice failed");
    unsigned char* work = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_work_ptr[dev]) {
            void* p = nullptr;
            err = cudaGetSymbolAddress(&p, g_static_work);
            if (err != cudaSuccess || !p) {
                snprintf(g_static_err, sizeof(g_static_err), "cudaGetSymbolAddress(g_static_work) failed: %s", cudaGetErrorString(err));
                return static_fail(g_static_err);
            }
            g_work_ptr[dev] = p;
        }
        work = static_cast<unsigned char*>(g_work_ptr[dev]);
        g_scratch_base[dev] = scr_base;
    }
    unsigned char* sym = work;
    unsigned char* scr = work + scr_base;

    // The area still holds the previous call's data (possibly laid out for another shape): clear everything the
    // kernels expect to start from zero -- signal words and count matrix, status / epoch / plan / histograms / m-block
    // tables, and the per-row amax accumulators.
#define MM_ST(expr) do { err = (expr); if (err != cudaSuccess) { char m_[384]; snprintf(m_, sizeof(m_), "%s failed: %s", #expr, cudaGetErrorString(err)); return static_fail(m_); } } while (0)
    MM_ST(cudaMemsetAsync(sym, 0, (size_t)sym_off[MM_SYM_X], stream));
    MM_ST(cudaMemsetAsync(scr, 0, (size_t)scr_off[MM_SCR_DEST_ROW], stream));
    MM_ST(cudaMemsetAsync(scr + scr_off[MM_SCR_ROW_AMAX], 0, (size_t)(scr_off[MM_SCR_ACT_BF16] - scr_off[MM_SCR_ROW_AMAX]), stream));
    if (num_tokens > 0) {
        MM_ST(cudaMemcpyAsync(sym + sym_off[MM_SYM_X], x_fp8, (size_t)num_tokens * H, cudaMemcpyDeviceToDevice, stream));
        MM_ST(cudaMemcpyAsync(sym + sym_off[MM_SYM_X_SF], x_sf, (size_t)num_tokens * 4, cudaMemcpyDeviceToDevice, stream));
        MM_ST(cudaMemcpyAsync(sym + sym_off[MM_SYM_TOPK_IDX], topk_idx, (size_t)num_tokens * K * 8, cudaMemcpyDeviceToDevice, stream));
        MM_ST(cudaMemcpyAsync(sym + sym_off[MM_SYM_TOPK_WEIGHTS], topk_weights, (size_t)num_tokens * K * 4, cudaMemcpyDeviceToDevice, stream));
    }
#undef MM_ST
    uint64_t peers[MM_ABI_MAX_RANKS] = {0};
    peers[0] = reinterpret_cast<uint64_t>(sym);
    return mm_fp8_w8a8_mega_moe(y, w1, s1, w2, s2, stats, sym, scr, peers, 0, 1, T, num_experts, num_tokens, K, H, I,
                                activation_clamp, MM_MODE_STAGED, nullptr, stream_);
}

int mm_fp8_w8a8_mega_moe_static_status(void* stream_, int32_t* out5) {
    if (!out5) return static_fail("mm_fp8_w8a8_mega_moe_static_status: null pointer");
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess || dev < 0 || dev >= 64) return static_fail("mm_fp8_w8a8_mega_moe_static_status: cudaGetDevice failed");
    const unsigned char* status = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_work_ptr[dev]) return static_fail("mm_fp8_w8a8_mega_moe_static_status: no static call has been made on this device");
        status = static_cast<const unsigned char*>(g_work_ptr[dev]) + g_scratch_base[dev];
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    err = cudaMemcpyAsync(out5, status, 5 * sizeof(int32_t), cudaMemcpyDeviceToHost, stream);
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    if (err != cudaSuccess) return static_fail(cudaGetErrorString(err));
    return 0;
}

}  // extern "C"
