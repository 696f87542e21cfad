// extern "C" entry points of libmegamoe_b200.so (declared in include/megamoe_b200.h) and the host-side launch logic.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/megamoe_b200.h"
#include "deepep_layout.cuh"
#include "fused.cuh"
#include "gemm.cuh"
#include "gemm_pair.cuh"
#include "gemm_ue8m0.cuh"
#include "layout.h"
#include "misc.cuh"
#include "probe.cuh"
#include "route.cuh"
#include "split_baseline.cuh"

static_assert(MM_ABI_MAX_RANKS == MM_MAX_RANKS, "header and layout disagree");

namespace {

thread_local char g_err[512] = "";
std::atomic<int64_t> g_launches{0};
std::atomic<int> g_barrier_ms{30000};
std::atomic<int> g_pipe_ms{4000};
// tuning switches of the layer kernel (FusedParams::policy, waves of its tile order): environment at load, or mm_set_tuning
std::atomic<int> g_policy{[] { const char* v = getenv("MEGAMOE_HELPER_POLICY"); return v ? atoi(v) : 2; }()};
std::atomic<int> g_wave_mblocks{[] { const char* v = getenv("MEGAMOE_WAVE_MBLOCKS"); return v ? atoi(v) : 0; }()};
// per-tile cycle stamps of one CTA of the layer kernel (mm_set_tile_trace); null = off
std::atomic<long long*> g_trace{nullptr};
std::atomic<int> g_trace_cta{0};
std::atomic<int> g_trace_tiles{0};

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

#define MM_CUDA(expr)                                                                          \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess) return fail(100 + (int)_e, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

#define MM_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) return fail(1, __VA_ARGS__); \
    } while (0)

int check_shape(int R, int E, int T, int K, int H, int I) {
    MM_REQUIRE(R > 0 && R <= MM_MAX_RANKS, "num_ranks must be in 1..%d", MM_MAX_RANKS);
    MM_REQUIRE(E > 0 && E % R == 0, "num_experts must be divisible by num_ranks");
    MM_REQUIRE(E <= MM_MAX_EXPERTS, "num_experts must be <= %d", MM_MAX_EXPERTS);
    MM_REQUIRE(T >= 0, "num_max_tokens_per_rank must be non-negative");
    MM_REQUIRE(K > 0 && K <= MM_MAX_TOPK, "num_topk must be in 1..%d", MM_MAX_TOPK);
    MM_REQUIRE(H > 0 && I > 0, "hidden sizes must be positive");
    MM_REQUIRE(H % 128 == 0 && I % 128 == 0, "hidden and intermediate_hidden must be multiples of 128");
    MM_REQUIRE((int64_t)R * T * K < (1ll << 30), "capacity too large");
    return 0;
}

// ------------------------------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn* out) {
    static EncodeTiledFn fn = nullptr;
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        MM_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
        MM_REQUIRE(p != nullptr && qres == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available in this driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    *out = fn;
    return 0;
}

struct MapKey { const void* ptr; uint64_t inner, rows; uint32_t box_rows; };
struct MapEntry { MapKey key; CUtensorMap map; };
std::mutex g_map_mu;
std::vector<MapEntry> g_maps;

// 2-D row-major byte matrix [rows][inner], box = box_rows rows x 128 bytes, 128-byte swizzle.
int tensor_map_2d(const void* ptr, uint64_t inner, uint64_t rows, uint32_t box_rows, CUtensorMap* out) {
    {
        std::lock_guard<std::mutex> lk(g_map_mu);
        for (auto& m : g_maps)
            if (m.key.ptr == ptr && m.key.inner == inner && m.key.rows == rows && m.key.box_rows == box_rows) { *out = m.map; return 0; }
    }
    EncodeTiledFn enc;
    if (int rc = get_encode_fn(&enc)) return rc;
    MM_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, "tensor base must be 16-byte aligned");
    MM_REQUIRE(inner % 16 == 0, "row pitch must be a multiple of 16 bytes");
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {inner};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap map;
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MM_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    std::lock_guard<std::mutex> lk(g_map_mu);
    if (g_maps.size() > 256) g_maps.clear();
    g_maps.push_back({{ptr, inner, rows, box_rows}, map});
    *out = map;
    return 0;
}

int sm_count(int* out) {
    int dev = 0;
    MM_CUDA(cudaGetDevice(&dev));
    static int cached[64] = {0};
    if (dev < 64 && cached[dev]) { *out = cached[dev]; return 0; }
    int n = 0;
    MM_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    if (dev < 64) cached[dev] = n;
    *out = n;
    return 0;
}

// Launch of the layer kernel: one CTA per SM, and its CTAs wait on one another, so all of them have to be resident.  The
// default is a cooperative launch, which guarantees that (or fails).  MEGAMOE_COOPERATIVE_LAUNCH=0 selects an ordinary
// launch of exactly one CTA per SM after an occupancy check (226 KiB of shared memory: a second CTA cannot share an SM);
// it is resident as soon as the SMs are free of other kernels, and until then its waits spin -- bounded, so the worst case
// is an error status, not a hang.
int fused_resident_ctas(int sms, int* out);

int ensure_gemm_attrs() {
    static std::mutex mu;
    static bool done[64] = {false};
    int dev = 0;
    MM_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 64 && done[dev]) return 0;
    MM_CUDA(cudaFuncSetAttribute(mm::grouped_gemm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, mm::kGemmSmemBytes));
    MM_CUDA(cudaFuncSetAttribute(mm::grouped_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, mm::kGemmSmemBytes));
    MM_CUDA(cudaFuncSetAttribute(mm::grouped_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, mm::kGemmSmemBytes));
    MM_CUDA(cudaFuncSetAttribute(mm::grouped_gemm_ue8m0_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mm::kU8SmemBytes));
    MM_CUDA(cudaFuncSetAttribute(mm::mega_moe_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mm::kGemmSmemBytes));
    MM_CUDA(cudaFuncSetAttribute(mm::grouped_gemm_pair_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, mm::kPairSmemBytes));
    MM_CUDA(cudaFuncSetAttribute(mm::grouped_gemm_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, mm::kPairSmemBytes));
    if (dev < 64) done[dev] = true;
    return 0;
}

int fused_resident_ctas(int sms, int* out) {
    static std::mutex mu;
    static int cached[64] = {0};
    int dev = 0;
    MM_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 64 && cached[dev]) { *out = cached[dev]; return 0; }
    int per_sm = 0;
    MM_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mm::mega_moe_fused_kernel, mm::kFusedThreads, mm::kGemmSmemBytes));
    const int n = per_sm * sms;
    if (dev < 64) cached[dev] = n;
    *out = n;
    return 0;
}

// CTA pairs that can be resident at once (the pair kernels stride their tiles over the grid, so a pair that only
// starts after another has finished would double the run time).  Not every SM need have a free partner in its GPC.
int pair_cluster_count(int sms, int* out) {
    static std::mutex mu;
    static int cached[64] = {0};
    int dev = 0;
    MM_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    if (dev < 64 && cached[dev]) { *out = cached[dev] > 0 ? cached[dev] : 0; return 0; }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(sms / 2 * 2);
    cfg.blockDim = dim3(mm::kGemmThreads);
    cfg.dynamicSmemBytes = mm::kPairSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n0 = 0, n1 = 0;
    MM_CUDA(cudaOccupancyMaxActiveClusters(&n0, mm::grouped_gemm_pair_kernel<0>, &cfg));
    MM_CUDA(cudaOccupancyMaxActiveClusters(&n1, mm::grouped_gemm_pair_kernel<1>, &cfg));
    int n = n0 < n1 ? n0 : n1;
    if (n > sms / 2) n = sms / 2;
    if (dev < 64) cached[dev] = n > 0 ? n : -1;
    if (getenv("MEGAMOE_VERBOSE")) fprintf(stderr, "megamoe: %d resident CTA pairs on %d SMs (device %d)\n", n, sms, dev);
    *out = n;
    return 0;
}

int launch_layer_kernel(int sms, void** args, const CUtensorMap& tm_pool, const CUtensorMap& tm_w1, const CUtensorMap& tm_act,
                        const CUtensorMap& tm_w2, const mm::FusedParams& fp, cudaStream_t stream) {
    static const bool cooperative = [] { const char* v = getenv("MEGAMOE_COOPERATIVE_LAUNCH"); return !(v && v[0] == '0'); }();
    if (cooperative) {
        MM_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(mm::mega_moe_fused_kernel), dim3(sms), dim3(mm::kFusedThreads),
                                            args, mm::kGemmSmemBytes, stream));
        return 0;
    }
    int resident = 0;
    if (int rc = fused_resident_ctas(sms, &resident)) return rc;
    MM_REQUIRE(resident >= sms, "the layer kernel needs one resident CTA per SM (%d), the device offers %d", sms, resident);
    mm::mega_moe_fused_kernel<<<sms, mm::kFusedThreads, mm::kGemmSmemBytes, stream>>>(tm_pool, tm_w1, tm_act, tm_w2, fp);
    return 0;
}

#define MM_LAUNCHED()                 \
    do {                              \
        g_launches.fetch_add(1);      \
        MM_CUDA(cudaGetLastError());  \
    } while (0)

// Optional per-stage timing of the staged layer call: CUDA events recorded on the caller's stream around every launch.
std::atomic<int> g_stage_timing{0};
std::mutex g_stage_mu;
cudaEvent_t g_stage_ev[MM_NUM_STAGES + 1];
bool g_stage_ev_made = false;
bool g_stage_recorded[MM_NUM_STAGES];
int g_stage_order[MM_NUM_STAGES];      // stage ids in the order they were recorded by the last call
int g_stage_count = 0;

int stage_begin(cudaStream_t stream) {
    if (!g_stage_timing.load()) return 0;
    std::lock_guard<std::mutex> lk(g_stage_mu);
    if (!g_stage_ev_made) {
        for (auto& e : g_stage_ev) MM_CUDA(cudaEventCreate(&e));
        g_stage_ev_made = true;
    }
    for (auto& r : g_stage_recorded) r = false;
    g_stage_count = 0;
    MM_CUDA(cudaEventRecord(g_stage_ev[0], stream));
    return 0;
}
// called after the launch of stage `id` (each stage at most once per call, in any order)
int stage_end(int id, cudaStream_t stream) {
    if (!g_stage_timing.load()) return 0;
    std::lock_guard<std::mutex> lk(g_stage_mu);
    MM_CUDA(cudaEventRecord(g_stage_ev[id + 1], stream));
    if (!g_stage_recorded[id] && g_stage_count < MM_NUM_STAGES) g_stage_order[g_stage_count++] = id;
    g_stage_recorded[id] = true;
    return 0;
}

}  // namespace

// lets the other translation units of the library report through mm_last_error
void mm_detail_set_error(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }

extern "C" {

const char* mm_last_error(void) { return g_err; }

int mm_token_alignment(void) { return MM_TOKEN_ALIGNMENT; }

int mm_symm_buffer_layout(int R, int E, int T, int K, int H, int I, int64_t* offsets, int64_t* total_bytes) {
    if (int rc = check_shape(R, E, T, K, H, I)) return rc;
    const MmSymLayout L = mm_sym_layout(R, E, T, K, H, I);
    if (offsets) {
        offsets[MM_SYM_PEER_PTRS] = L.peer_ptrs; offsets[MM_SYM_SIGNALS] = L.signals;
        offsets[MM_SYM_RUNTIME_NUM_TOKENS] = L.runtime_num_tokens; offsets[MM_SYM_COUNT_MATRIX] = L.count_matrix;
        offsets[MM_SYM_X] = L.x; offsets[MM_SYM_X_SF] = L.x_sf; offsets[MM_SYM_TOPK_IDX] = L.topk_idx;
        offsets[MM_SYM_TOPK_WEIGHTS] = L.topk_weights; offsets[MM_SYM_POOL_X] = L.pool_x; offsets[MM_SYM_POOL_META] = L.pool_meta;
        offsets[MM_SYM_COMBINE] = L.combine; offsets[MM_SYM_POOL_ROWS] = L.pool_rows;
    }
    if (total_bytes) *total_bytes = L.total;
    return 0;
}

int mm_scratch_layout(int R, int E, int T, int K, int H, int I, int64_t* offsets, int64_t* total_bytes) {
    if (int rc = check_shape(R, E, T, K, H, I)) return rc;
    const MmScratchLayout L = mm_scratch_layout_of(R, E, T, K, H, I);
    if (offsets) {
        offsets[MM_SCR_STATUS] = L.status; offsets[MM_SCR_EPOCH] = L.epoch; offsets[MM_SCR_PLAN] = L.plan;
        offsets[MM_SCR_BLOCK_COUNTS] = L.block_counts; offsets[MM_SCR_DEST_BASE] = L.dest_base;
        offsets[MM_SCR_EXPERT_TOTAL] = L.expert_total; offsets[MM_SCR_EXPERT_OFF] = L.expert_off;
        offsets[MM_SCR_MBLOCK_EXPERT] = L.mblock_expert; offsets[MM_SCR_MBLOCK_VALID] = L.mblock_valid;
        offsets[MM_SCR_DEST_ROW] = L.dest_row; offsets[MM_SCR_ROW_AMAX] = L.row_amax; offsets[MM_SCR_ACT_SCALE] = L.act_scale;
        offsets[MM_SCR_ACT_BF16] = L.act_bf16; offsets[MM_SCR_ACT_FP8] = L.act_fp8; offsets[MM_SCR_ROUTE_BLOCKS] = L.route_blocks;
        offsets[MM_SCR_SEND_BASE] = L.send_base; offsets[MM_SCR_SEND_LIST] = L.send_list;
        offsets[MM_SCR_L1_DONE] = L.l1_done; offsets[MM_SCR_L2_READY] = L.l2_ready; offsets[MM_SCR_GRID_SYNC] = L.grid_sync;
        offsets[MM_SCR_ACT_SF] = L.act_sf;
    }
    if (total_bytes) *total_bytes = L.total;
    return 0;
}

int mm_ipc_alloc(int64_t bytes, void** dev_ptr, void* handle64) {
    MM_REQUIRE(bytes > 0 && dev_ptr != nullptr, "mm_ipc_alloc: bad arguments");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    void* p = nullptr;
    MM_CUDA(cudaMalloc(&p, (size_t)bytes));
    if (handle64) {
        cudaIpcMemHandle_t h;
        cudaError_t e = cudaIpcGetMemHandle(&h, p);
        if (e != cudaSuccess) {
            cudaFree(p);
            return fail(100 + (int)e, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
        }
        memcpy(handle64, &h, 64);
    }
    *dev_ptr = p;
    return 0;
}

int mm_ipc_open(const void* handle64, void** dev_ptr) {
    MM_REQUIRE(handle64 != nullptr && dev_ptr != nullptr, "mm_ipc_open: bad arguments");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    MM_CUDA(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}

int mm_ipc_close(void* dev_ptr) {
    if (dev_ptr) MM_CUDA(cudaIpcCloseMemHandle(dev_ptr));
    return 0;
}

int mm_ipc_free(void* dev_ptr) {
    if (dev_ptr) MM_CUDA(cudaFree(dev_ptr));
    return 0;
}

int mm_init_buffers(void* sym_base, void* scratch, const uint64_t* peer_ptrs, int rank, int R, int E, int T, int K, int H,
                    int I, void* stream_) {
    if (int rc = check_shape(R, E, T, K, H, I)) return rc;
    MM_REQUIRE(sym_base && scratch && peer_ptrs, "mm_init_buffers: null pointer");
    MM_REQUIRE(rank >= 0 && rank < R, "rank out of range");
    MM_REQUIRE(peer_ptrs[rank] == reinterpret_cast<uint64_t>(sym_base), "peer_ptrs[rank] must be the local buffer");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const MmSymLayout sl = mm_sym_layout(R, E, T, K, H, I);
    const MmScratchLayout cl = mm_scratch_layout_of(R, E, T, K, H, I);
    uint8_t* s = static_cast<uint8_t*>(sym_base);
    uint8_t* c = static_cast<uint8_t*>(scratch);
    MM_CUDA(cudaMemsetAsync(s, 0, (size_t)sl.x, stream));                                 // header .. count matrix
    MM_CUDA(cudaMemsetAsync(c, 0, (size_t)cl.dest_row, stream));                          // status .. m-block tables
    MM_CUDA(cudaMemsetAsync(c + cl.row_amax, 0, (size_t)(cl.act_bf16 - cl.row_amax), stream));
    uint64_t table[MM_MAX_RANKS] = {0};
    for (int r = 0; r < R; ++r) table[r] = peer_ptrs[r];
    MM_CUDA(cudaMemcpyAsync(s + sl.peer_ptrs, table, sizeof(table), cudaMemcpyHostToDevice, stream));
    MM_CUDA(cudaStreamSynchronize(stream));   // `table` lives on this stack frame
    return 0;
}

int mm_quant_per_token(const void* x_bf16, int64_t rows, int k, void* out_fp8, float* out_scale, void* stream_) {
    MM_REQUIRE(rows >= 0 && k > 0 && k % 8 == 0, "mm_quant_per_token: k must be a positive multiple of 8");
    if (rows == 0) return 0;
    MM_REQUIRE(x_bf16 && out_fp8 && out_scale, "mm_quant_per_token: null pointer");
    MM_REQUIRE((reinterpret_cast<uintptr_t>(x_bf16) & 15) == 0 && (reinterpret_cast<uintptr_t>(out_fp8) & 7) == 0,
               "mm_quant_per_token: pointers must be 16-byte (input) and 8-byte (output) aligned");
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    int64_t blocks = (rows + 7) / 8;
    if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
    mm::quant_per_token_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
        static_cast<const __nv_bfloat16*>(x_bf16), rows, k, static_cast<uint8_t*>(out_fp8), out_scale);
    MM_LAUNCHED();
    return 0;
}

int mm_deepep_scatter_channelwise(void* grouped_x, float* grouped_x_scale, float* route_weights, int* m_indices, int* output_index,
                                  int* expert_start_loc, const void* recv_x, const float* recv_x_scale, const void* recv_topk_ids,
                                  const float* recv_topk_weights, const int* num_recv_tokens_per_expert, int total_rows,
                                  int recv_rows, int topk, int hidden, int num_experts, int topk_ids_i64, void* stream_) {
    MM_REQUIRE(total_rows >= 0 && recv_rows >= 0 && topk > 0 && hidden > 0 && hidden % 16 == 0 && num_experts > 0,
               "mm_deepep_scatter_channelwise: bad shape (hidden must be a multiple of 16)");
    MM_REQUIRE(expert_start_loc && num_recv_tokens_per_expert, "mm_deepep_scatter_channelwise: null pointer");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    mm::deepep_prefix_kernel<<<1, 1024, 0, stream>>>(num_recv_tokens_per_expert, expert_start_loc, num_experts);
    MM_LAUNCHED();
    const int64_t routes = (int64_t)recv_rows * topk;
    if (routes == 0) return 0;
    MM_REQUIRE(grouped_x && grouped_x_scale && route_weights && m_indices && output_index && recv_x && recv_x_scale && recv_topk_ids &&
               recv_topk_weights, "mm_deepep_scatter_channelwise: null pointer");
    const int blocks = (num_experts + 7) / 8;
    if (topk_ids_i64)
        mm::deepep_assign_kernel<int64_t><<<blocks, 256, 0, stream>>>(recv_topk_ids, expert_start_loc, output_index, m_indices, routes, num_experts, total_rows);
    else
        mm::deepep_assign_kernel<int32_t><<<blocks, 256, 0, stream>>>(recv_topk_ids, expert_start_loc, output_index, m_indices, routes, num_experts, total_rows);
    MM_LAUNCHED();
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    int64_t cblocks = (routes + 7) / 8;
    if (cblocks > (int64_t)sms * 8) cblocks = (int64_t)sms * 8;
    mm::deepep_scatter_rows_kernel<<<(unsigned)cblocks, 256, 0, stream>>>(static_cast<const uint8_t*>(recv_x), recv_x_scale, recv_topk_weights,
                                                                         output_index, static_cast<uint8_t*>(grouped_x), grouped_x_scale,
                                                                         route_weights, routes, topk, hidden);
    MM_LAUNCHED();
    return 0;
}

int mm_deepep_gather_channelwise(void* recv_y, const void* l2_out, const void* recv_topk_ids, const float* recv_topk_weights,
                                 const int* output_index, int recv_rows, int topk, int hidden, int topk_ids_i64,
                                 int apply_topk_weights, void* stream_) {
    MM_REQUIRE(recv_rows >= 0 && topk > 0 && hidden > 0 && hidden % 8 == 0, "mm_deepep_gather_channelwise: bad shape (hidden must be a multiple of 8)");
    if (recv_rows == 0) return 0;
    MM_REQUIRE(recv_y && l2_out && recv_topk_ids && recv_topk_weights && output_index, "mm_deepep_gather_channelwise: null pointer");
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (topk_ids_i64)
        mm::deepep_gather_kernel<int64_t><<<sms * 8, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(recv_y), static_cast<const __nv_bfloat16*>(l2_out),
                                                                      recv_topk_ids, recv_topk_weights, output_index, recv_rows, topk, hidden, apply_topk_weights);
    else
        mm::deepep_gather_kernel<int32_t><<<sms * 8, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(recv_y), static_cast<const __nv_bfloat16*>(l2_out),
                                                                      recv_topk_ids, recv_topk_weights, output_index, recv_rows, topk, hidden, apply_topk_weights);
    MM_LAUNCHED();
    return 0;
}

int mm_m_grouped_fp8_gemm_nt_contiguous(const void* a_fp8, const float* a_scale, const void* w_tiled, const float* w_scale,
                                        void* out_bf16, const int* m_indices, int rows, int N, int K, int E, int* work,
                                        void* stream_) {
    MM_REQUIRE(rows >= 0 && rows % MM_BLOCK_M == 0, "m-grouped GEMM: rows must be a multiple of %d (groups padded to it)", MM_BLOCK_M);
    MM_REQUIRE(N > 0 && N % 64 == 0 && K > 0 && K % mm::kBlockK == 0 && E > 0, "m-grouped GEMM: need N %% 64 == 0, K %% 128 == 0, E > 0");
    if (rows == 0) return 0;
    MM_REQUIRE(a_fp8 && a_scale && w_tiled && w_scale && out_bf16 && m_indices && work, "m-grouped GEMM: null pointer");
    MM_REQUIRE((reinterpret_cast<uintptr_t>(out_bf16) & 15) == 0, "m-grouped GEMM: output must be 16-byte aligned");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    if (int rc = ensure_gemm_attrs()) return rc;
    const int blocks = rows / MM_BLOCK_M;
    const int n_blocks = (N + mm::kBlockN - 1) / mm::kBlockN;
    CUtensorMap tm_a, tm_b;
    if (int rc = tensor_map_2d(a_fp8, (uint64_t)K, (uint64_t)rows, 128, &tm_a)) return rc;
    if (int rc = tensor_map_2d(w_tiled, 128, (uint64_t)E * n_blocks * (K / 128) * 256, 256, &tm_b)) return rc;
    MM_CUDA(cudaMemsetAsync(work, 0, 32 * sizeof(int), stream));
    mm::mgroup_plan_kernel<<<(blocks * 32 + 255) / 256, 256, 0, stream>>>(m_indices, rows, E, work);
    MM_LAUNCHED();
    mm::GemmParams g;
    memset(&g, 0, sizeof(g));
    g.kdim = K; g.n_blocks = n_blocks; g.n_out = N; g.w_rows_per_expert = N;
    g.plan = work + 16;
    g.mblock_expert = work + 32;
    g.mblock_valid = work + 32 + blocks;
    g.w_scale = w_scale;
    g.act_scale = a_scale;
    g.out_rows = static_cast<__nv_bfloat16*>(out_bf16);
    g.status = work;
    g.timeout_ns = (uint64_t)g_pipe_ms.load() * 1000000ull;
    g.E_loc = E;
    mm::grouped_gemm_kernel<1><<<sms, mm::kGemmThreads, mm::kGemmSmemBytes, stream>>>(tm_a, tm_b, g);
    MM_LAUNCHED();
    return 0;
}

int mm_swiglu_quant_channelwise(const void* x_bf16, const float* weights, const int64_t* row_combine_ptrs, void* out_fp8,
                                float* out_scale, void* out_bf16, int rows, int inter, int has_clamp, float clamp_value,
                                void* stream_) {
    MM_REQUIRE(rows >= 0 && inter > 0 && inter % 4 == 0, "swiglu_quant: need rows >= 0 and inter %% 4 == 0");
    if (rows == 0) return 0;
    MM_REQUIRE(x_bf16 && out_fp8 && out_scale, "swiglu_quant: null pointer");
    MM_REQUIRE((reinterpret_cast<uintptr_t>(x_bf16) & 7) == 0 && (reinterpret_cast<uintptr_t>(out_fp8) & 3) == 0 &&
               (reinterpret_cast<uintptr_t>(out_bf16) & 7) == 0, "swiglu_quant: x / out_bf16 must be 8-byte, out_fp8 4-byte aligned");
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    int blocks = rows < sms * 8 ? rows : sms * 8;
    mm::swiglu_quant_channelwise_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
        static_cast<const __nv_bfloat16*>(x_bf16), weights, row_combine_ptrs, static_cast<uint8_t*>(out_fp8), out_scale,
        static_cast<__nv_bfloat16*>(out_bf16), rows, inter, has_clamp, clamp_value);
    MM_LAUNCHED();
    return 0;
}

int mm_fp8_mma_peak_probe(int iters, int operands, int cta_pair, int* status_dev, void* stream_, double* flops_out) {
    MM_REQUIRE(iters > 0 && status_dev && operands >= 0 && operands <= 2 && (cta_pair == 0 || cta_pair == 1),
               "mm_fp8_mma_peak_probe: bad arguments");
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    // the attribute is per device; setting it on every call keeps multi-device processes correct (the call is cheap)
    MM_CUDA(cudaFuncSetAttribute(mm::fp8_mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mm::kABytes + mm::kBBytes));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (cta_pair) {
        sms = sms / 2 * 2;
        MM_CUDA(cudaFuncSetAttribute(mm::fp8_mma_peak_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mm::kABytes + mm::kBBytes));
        mm::fp8_mma_peak_pair_kernel<<<sms, 128, mm::kABytes + mm::kBBytes, stream>>>(iters, status_dev, operands);
    } else {
        mm::fp8_mma_peak_kernel<<<sms, 128, mm::kABytes + mm::kBBytes, stream>>>(iters, status_dev, operands);
    }
    MM_LAUNCHED();
    if (flops_out) *flops_out = (double)sms * iters * 8.0 * 2.0 * mm::kBlockM * mm::kBlockN * 32.0;
    return 0;
}

int mm_peer_store_probe(const uint64_t* dst_ptrs, int n_dst, int64_t bytes_per_dst, void* stream_) {
    MM_REQUIRE(dst_ptrs && n_dst > 0 && n_dst <= MM_MAX_RANKS && bytes_per_dst > 0 && bytes_per_dst % 512 == 0,
               "mm_peer_store_probe: need 1..%d destinations and a positive multiple of 512 bytes", MM_MAX_RANKS);
    mm::PeerStoreDsts d;
    memset(&d, 0, sizeof(d));
    for (int i = 0; i < n_dst; ++i) {
        MM_REQUIRE(dst_ptrs[i] != 0 && (dst_ptrs[i] & 15) == 0, "mm_peer_store_probe: destinations must be 16-byte aligned");
        d.ptr[i] = dst_ptrs[i];
    }
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    mm::peer_store_probe_kernel<<<sms * 8, 256, 0, static_cast<cudaStream_t>(stream_)>>>(d, n_dst, bytes_per_dst / 16);
    MM_LAUNCHED();
    return 0;
}

int mm_router_topk_quant(const void* x_bf16, const float* router_logits, int num_tokens, int E, int K, int H, void* x_fp8,
                         float* x_sf, int64_t* topk_idx, float* topk_weights, void* stream_) {
    MM_REQUIRE(num_tokens >= 0 && E > 0 && E <= MM_MAX_EXPERTS && K > 0 && K <= MM_MAX_TOPK && K <= E && H > 0 && H % 8 == 0,
               "mm_router_topk_quant: need 0 < K <= min(E, %d), E <= %d, H %% 8 == 0", MM_MAX_TOPK, MM_MAX_EXPERTS);
    if (num_tokens == 0) return 0;
    MM_REQUIRE(x_bf16 && router_logits && x_fp8 && x_sf && topk_idx && topk_weights, "mm_router_topk_quant: null pointer");
    MM_REQUIRE((reinterpret_cast<uintptr_t>(x_bf16) & 15) == 0 && (reinterpret_cast<uintptr_t>(x_fp8) & 7) == 0,
               "mm_router_topk_quant: x must be 16-byte aligned, x_fp8 8-byte aligned");
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    int blocks = (num_tokens + 7) / 8;
    if (blocks > sms * 8) blocks = sms * 8;
    mm::router_topk_quant_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
        static_cast<const __nv_bfloat16*>(x_bf16), router_logits, num_tokens, E, K, H, static_cast<uint8_t*>(x_fp8), x_sf, topk_idx,
        topk_weights);
    MM_LAUNCHED();
    return 0;
}

int mm_fp8_w8a8_mega_moe(void* y, const void* w1, const float* s1, const void* w2, const float* s2, int* stats, void* sym_base,
                         void* scratch, const uint64_t* peer_ptrs, int rank, int R, int T_max, int E_loc, int num_tokens,
                         int K, int H, int I, float activation_clamp, int mode, const int* runtime_num_tokens, void* stream_) {
    MM_REQUIRE(E_loc > 0, "num_experts_per_rank must be positive");
    const int E = E_loc * R;
    if (int rc = check_shape(R, E, T_max, K, H, I)) return rc;
    MM_REQUIRE((y || num_tokens == 0) && w1 && s1 && w2 && s2 && sym_base && scratch && peer_ptrs,
               "mm_fp8_w8a8_mega_moe: null pointer");
    MM_REQUIRE(rank >= 0 && rank < R, "rank out of range");
    MM_REQUIRE(num_tokens >= 0 && num_tokens <= T_max, "too many tokens");
    MM_REQUIRE(peer_ptrs[rank] == reinterpret_cast<uint64_t>(sym_base), "peer_ptrs[rank] must be the local buffer");
    MM_REQUIRE(!isnan(activation_clamp) && activation_clamp > 0.0f, "activation_clamp must be positive (+inf for none)");
    MM_REQUIRE(mode == MM_MODE_STAGED || mode == MM_MODE_FUSED || mode == MM_MODE_STAGED_SPLIT || mode == MM_MODE_STAGED_UE8M0, "unknown mode");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    mm::RouteParams rp;
    memset(&rp, 0, sizeof(rp));
    rp.sym = static_cast<uint8_t*>(sym_base);
    rp.scratch = static_cast<uint8_t*>(scratch);
    for (int r = 0; r < R; ++r) rp.peers[r] = peer_ptrs[r];
    rp.sl = mm_sym_layout(R, E, T_max, K, H, I);
    rp.cl = mm_scratch_layout_of(R, E, T_max, K, H, I);
    rp.rank = rank; rp.R = R; rp.E = E; rp.E_loc = E_loc; rp.T = T_max; rp.K = K; rp.H = H;
    rp.num_tokens = num_tokens;
    rp.runtime_num_tokens = runtime_num_tokens;
    rp.stats = stats;
    rp.barrier_timeout_ns = (uint64_t)g_barrier_ms.load() * 1000000ull;
    // a device-side token count is clamped to num_tokens (the rows of y), so num_tokens bounds the routes in both modes
    const int64_t tokens_bound = num_tokens;
    int route_blocks = (int)((tokens_bound * K + MM_ROUTE_CHUNK - 1) / MM_ROUTE_CHUNK);
    if (route_blocks < 1) route_blocks = 1;
    rp.cl.route_blocks = route_blocks;   // blocks whose histogram rows are live in this call

    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    if (int rc = ensure_gemm_attrs()) return rc;

    uint8_t* sc = rp.scratch;
    CUtensorMap tm_pool, tm_w1, tm_act, tm_w2;
    if (int rc = tensor_map_2d(rp.sym + rp.sl.pool_x, (uint64_t)H, (uint64_t)rp.sl.pool_rows, 128, &tm_pool)) return rc;
    if (int rc = tensor_map_2d(w1, 128, (uint64_t)E_loc * (I / 128) * (H / 128) * 256, 256, &tm_w1)) return rc;
    if (int rc = tensor_map_2d(sc + rp.cl.act_fp8, (uint64_t)I, (uint64_t)rp.sl.pool_rows, 128, &tm_act)) return rc;
    if (int rc = tensor_map_2d(w2, 128, (uint64_t)E_loc * ((H + 255) / 256) * (I / 128) * 256, 256, &tm_w2)) return rc;

    mm::GemmParams g1;
    memset(&g1, 0, sizeof(g1));
    g1.plan = reinterpret_cast<const int*>(sc + rp.cl.plan);
    g1.mblock_expert = reinterpret_cast<const int*>(sc + rp.cl.mblock_expert);
    g1.mblock_valid = reinterpret_cast<const int*>(sc + rp.cl.mblock_valid);
    g1.expert_total = reinterpret_cast<const int*>(sc + rp.cl.expert_total);
    g1.expert_off = reinterpret_cast<const int*>(sc + rp.cl.expert_off);
    g1.E_loc = E_loc;
    g1.meta = reinterpret_cast<const MmPoolMeta*>(rp.sym + rp.sl.pool_meta);
    g1.status = reinterpret_cast<int*>(sc + rp.cl.status);
    g1.timeout_ns = (uint64_t)g_pipe_ms.load() * 1000000ull;
    for (int r = 0; r < R; ++r) g1.peers[r] = peer_ptrs[r];
    g1.combine_off = rp.sl.combine;
    g1.T = T_max; g1.H = H; g1.R = R; g1.K = K;
    g1.act_bf16 = reinterpret_cast<__nv_bfloat16*>(sc + rp.cl.act_bf16);
    g1.row_amax = reinterpret_cast<unsigned int*>(sc + rp.cl.row_amax);
    g1.act_scale = reinterpret_cast<const float*>(sc + rp.cl.act_scale);
    g1.clamp = activation_clamp;
    mm::GemmParams g2 = g1;
    g1.kdim = H; g1.n_blocks = I / 128; g1.n_out = I; g1.w_rows_per_expert = 2 * I; g1.w_scale = s1;
    g2.kdim = I; g2.n_blocks = (H + mm::kBlockN - 1) / mm::kBlockN; g2.n_out = H; g2.w_rows_per_expert = H; g2.w_scale = s2;

    mm::FusedParams fp;
    memset(&fp, 0, sizeof(fp));
    fp.rp = rp;
    fp.g1 = g1;
    fp.g2 = g2;
    fp.y = static_cast<__nv_bfloat16*>(y);
    fp.plan = reinterpret_cast<int*>(sc + rp.cl.plan);
    fp.l1_done = reinterpret_cast<int*>(sc + rp.cl.l1_done);
    fp.l2_ready = reinterpret_cast<int*>(sc + rp.cl.l2_ready);
    fp.grid_sync = reinterpret_cast<int*>(sc + rp.cl.grid_sync);
    fp.send_list = reinterpret_cast<const int4*>(sc + rp.cl.send_list);
    fp.act_fp8 = sc + rp.cl.act_fp8;
    fp.act_scale_w = reinterpret_cast<float*>(sc + rp.cl.act_scale);
    fp.w1_tiled = static_cast<const uint8_t*>(w1);
    // a wave holds enough GEMM1 tiles for about two rounds over the SMs; its GEMM2 tiles come up kWaveLookahead waves later,
    // by when its requantisation is done
    fp.wave_mblocks = (2 * sms + g1.n_blocks - 1) / g1.n_blocks;
    const int wave_override = g_wave_mblocks.load();                      // tuning aid (MEGAMOE_WAVE_MBLOCKS / mm_set_tuning)
    if (wave_override != 0) fp.wave_mblocks = wave_override > 0 ? wave_override : (1 << 28);
    fp.policy = g_policy.load();                                          // tuning aid (MEGAMOE_HELPER_POLICY / mm_set_tuning)
    fp.trace = g_trace.load();
    fp.trace_cta = g_trace_cta.load();
    fp.trace_tiles = g_trace_tiles.load();
    void* fused_args[] = {&tm_pool, &tm_w1, &tm_act, &tm_w2, &fp};

    if (mode == MM_MODE_FUSED) {
        if (int rc = stage_begin(stream)) return rc;
        // cooperative launch: all CTAs must be resident because they wait on one another
        if (int rc = launch_layer_kernel(sms, fused_args, tm_pool, tm_w1, tm_act, tm_w2, fp, stream)) return rc;
        MM_LAUNCHED();
        if (int rc = stage_end(MM_STAGE_FUSED, stream)) return rc;
        return 0;
    }

    // Staged variants: routing as small kernels, then
    //   MM_MODE_STAGED        the layer kernel in gemm_only mode: NVLink push, GEMM1, requantisation and GEMM2 tiles in one
    //                         launch, so that the transfers overlap the tensor work expert by expert;
    //   MM_MODE_STAGED_SPLIT  dispatch, a cross-rank barrier, GEMM1, requantisation and GEMM2 as separate launches.
    if (int rc = stage_begin(stream)) return rc;
    int* reset_a = nullptr; int* reset_b = nullptr;
    int reset_a_words = 0, reset_b_words = 0;
#define MM_STAGE(id) do { MM_LAUNCHED(); if (int rc_ = stage_end(id, stream)) return rc_; } while (0)
    mm::route_count_kernel<<<route_blocks, 1024, 0, stream>>>(rp);     // its last block also exchanges the counts
    MM_STAGE(MM_STAGE_ROUTE_COUNT);
    mm::route_plan_kernel<<<1, 1024, 0, stream>>>(rp);
    MM_STAGE(MM_STAGE_ROUTE_PLAN);
    if (mode == MM_MODE_STAGED) {
        mm::send_plan_kernel<<<route_blocks, MM_ROUTE_CHUNK, 0, stream>>>(rp);
        MM_STAGE(MM_STAGE_DISPATCH);
        fp.gemm_only = 1;
        if (int rc = launch_layer_kernel(sms, fused_args, tm_pool, tm_w1, tm_act, tm_w2, fp, stream)) return rc;
        MM_STAGE(MM_STAGE_FUSED);
        // the reduce kernel below leaves the per-m-block dependency counters zero for the next call: l1_done, l2_ready and
        // grid_sync are adjacent in the scratch buffer, the arrival counters live in the symmetric buffer
        const int64_t n_mb = rp.sl.pool_rows / MM_BLOCK_M;
        reset_a = reinterpret_cast<int*>(sc + rp.cl.l1_done);
        reset_a_words = (int)((rp.cl.grid_sync + 32 - rp.cl.l1_done) / 4);
        reset_b = reinterpret_cast<int*>(rp.sym + rp.sl.pool_arrive);
        reset_b_words = (int)(n_mb + 1);
    } else {
    mm::dispatch_kernel<<<route_blocks, mm::MM_DISPATCH_THREADS, 0, stream>>>(rp);
    MM_STAGE(MM_STAGE_DISPATCH);
    if (R > 1) {
        mm::rank_barrier_kernel<<<1, 32, 0, stream>>>(rp, MM_BAR_DISPATCH);
        MM_STAGE(MM_STAGE_BARRIER_DISPATCH);
    }
    // CTA-pair GEMMs (two m-blocks of one expert share each weight tile).  Measured on B200 (hidden 4096, intermediate
    // 2048): with 192 rows per expert -- two m-blocks, the regime between HBM-bound and tensor-bound, where the one-CTA
    // kernel streams every weight tile once from HBM and once more from L2 -- they take 10 % off both GEMMs; with 384 rows
    // (three m-blocks: the second pair is half empty) they lose 7 % on GEMM1, with 768 rows 9 %, with 1536 rows they tie.
    // So they are used when an expert is expected to hold two m-blocks; MEGAMOE_GEMM_PAIR=0/1 overrides.
    const int64_t expected_routes = (int64_t)tokens_bound * K;        // per local expert: expected_routes / E_loc
    bool pair_gemms = expected_routes > (int64_t)144 * E_loc && expected_routes <= (int64_t)256 * E_loc && sms >= 2;
    if (const char* v = getenv("MEGAMOE_GEMM_PAIR")) pair_gemms = v[0] == '1' && sms >= 2;   // read per call: tests switch it
    CUtensorMap tm_w1h, tm_w2h;
    if (pair_gemms) {
        if (int rc = tensor_map_2d(w1, 128, (uint64_t)E_loc * (I / 128) * (H / 128) * 256, 128, &tm_w1h)) return rc;
        if (int rc = tensor_map_2d(w2, 128, (uint64_t)E_loc * ((H + 255) / 256) * (I / 128) * 256, 128, &tm_w2h)) return rc;
    }
    int pair_grid = 0;
    if (pair_gemms) {
        int clusters = 0;
        if (int rc = pair_cluster_count(sms, &clusters)) return rc;
        if (clusters < sms / 4) pair_gemms = false;      // too few resident pairs to be worth it
        pair_grid = 2 * clusters;
    }
    if (mode == MM_MODE_STAGED_UE8M0) {
        // UE8M0 recipe: GEMM1 quantises in its epilogue (codes into the FP8 activation region, scale bytes beside them),
        // GEMM2 applies the block scales in the tensor core: no bf16 activations, no requantisation launch
        MM_REQUIRE(H % 128 == 0 && I % 128 == 0, "the UE8M0 recipe needs hidden sizes that are multiples of 128");
        CUtensorMap tm_w2q;
        if (int rc = tensor_map_2d(w2, 128, (uint64_t)E_loc * ((H + 255) / 256) * (I / 128) * 256, 128, &tm_w2q)) return rc;
        mm::GemmParams u1 = g1, u2 = g2;
        u1.act_q_out = sc + rp.cl.act_fp8;
        u1.act_sf = sc + rp.cl.act_sf;
        u2.act_sf = sc + rp.cl.act_sf;
        u2.n_blocks = H / 128;
        mm::grouped_gemm_kernel<2><<<sms, mm::kGemmThreads, mm::kGemmSmemBytes, stream>>>(tm_pool, tm_w1, u1);
        MM_STAGE(MM_STAGE_GEMM1);
        mm::grouped_gemm_ue8m0_kernel<<<sms, mm::kGemmThreads, mm::kU8SmemBytes, stream>>>(tm_act, tm_w2q, u2);
        MM_STAGE(MM_STAGE_GEMM2);
    } else {
    if (pair_gemms) mm::grouped_gemm_pair_kernel<0><<<pair_grid, mm::kGemmThreads, mm::kPairSmemBytes, stream>>>(tm_pool, tm_w1h, g1);
    else mm::grouped_gemm_kernel<0><<<sms, mm::kGemmThreads, mm::kGemmSmemBytes, stream>>>(tm_pool, tm_w1, g1);
    MM_STAGE(MM_STAGE_GEMM1);
    mm::requant_kernel<<<sms * 4, 256, 0, stream>>>(g1.act_bf16, I, g1.plan, g1.mblock_valid, g1.row_amax,
                                                   reinterpret_cast<float*>(sc + rp.cl.act_scale), sc + rp.cl.act_fp8, g1.status);
    MM_STAGE(MM_STAGE_REQUANT);
    if (pair_gemms) mm::grouped_gemm_pair_kernel<1><<<pair_grid, mm::kGemmThreads, mm::kPairSmemBytes, stream>>>(tm_act, tm_w2h, g2);
    else mm::grouped_gemm_kernel<1><<<sms, mm::kGemmThreads, mm::kGemmSmemBytes, stream>>>(tm_act, tm_w2, g2);
    MM_STAGE(MM_STAGE_GEMM2);
    }   // channelwise recipe
    }   // split launches
    // the reduce kernel does the cross-rank "combine stores done" barrier itself before it reads the combine buffer
    mm::combine_reduce_kernel<<<sms * 8, 256, 0, stream>>>(rp, static_cast<__nv_bfloat16*>(y), R > 1 ? 1 : 0, reset_a, reset_a_words,
                                                          reset_b, reset_b_words);
    MM_STAGE(MM_STAGE_REDUCE);
#undef MM_STAGE
    return 0;
}

int mm_read_status(const void* scratch, void* stream_, int32_t* out5) {
    MM_REQUIRE(scratch && out5, "mm_read_status: null pointer");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MM_CUDA(cudaMemcpyAsync(out5, scratch, 5 * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    MM_CUDA(cudaStreamSynchronize(stream));
    return 0;
}

int mm_set_timeouts(int rank_barrier_ms, int pipeline_ms) {
    MM_REQUIRE(rank_barrier_ms > 0 && pipeline_ms > 0, "timeouts must be positive");
    g_barrier_ms.store(rank_barrier_ms);
    g_pipe_ms.store(pipeline_ms);
    return 0;
}

int mm_set_tuning(int policy, int wave_mblocks) {
    MM_REQUIRE(policy >= 0, "mm_set_tuning: policy must be non-negative");
    g_policy.store(policy);
    g_wave_mblocks.store(wave_mblocks);
    return 0;
}

int mm_tile_order(int num_mblocks, int wave_mblocks, int gemm1_blocks, int gemm2_blocks, int tile_interleave, int32_t* out3) {
    MM_REQUIRE(num_mblocks >= 0 && wave_mblocks > 0 && gemm1_blocks > 0 && gemm2_blocks > 0 && out3, "mm_tile_order: bad arguments");
    mm::WaveOrder order(num_mblocks, wave_mblocks, gemm1_blocks, gemm2_blocks, tile_interleave != 0);
    const int64_t tiles = (int64_t)num_mblocks * (gemm1_blocks + gemm2_blocks);
    for (int64_t t = 0; t < tiles; ++t) {
        int kind, mb, nb;
        order.seek((int)t, kind, mb, nb);
        out3[3 * t] = kind; out3[3 * t + 1] = mb; out3[3 * t + 2] = nb;
    }
    return 0;
}

int mm_set_tile_trace(void* device_words, int max_tiles, int cta) {
    MM_REQUIRE(max_tiles >= 0 && cta >= 0, "mm_set_tile_trace: bad arguments");
    g_trace.store(max_tiles > 0 ? static_cast<long long*>(device_words) : nullptr);
    g_trace_cta.store(cta);
    g_trace_tiles.store(max_tiles);
    return 0;
}

int mm_build_config(char* json, int capacity) {
    MM_REQUIRE(json && capacity > 0, "mm_build_config: bad arguments");
    const int n = snprintf(json, (size_t)capacity,
                           "{\"operator\": \"fp8_w8a8_mega_moe\", \"package\": \"megamoe\", \"arch\": \"sm_100a\", "
                           "\"weight_scale_mode\": \"channelwise_fp32\", \"input_scale_mode\": \"channelwise_fp32\", "
                           "\"l2_act_scale_mode\": \"channelwise_fp32\", \"has_fp8_api\": true, \"has_fp4_api\": false, "
                           "\"fusion_boundary\": \"dispatch_pool_l1_swiglu_quant_l2_combine\", "
                           "\"block_m\": %d, \"block_n\": %d, \"block_k\": %d, \"stages\": %d, \"token_alignment\": %d, "
                           "\"max_ranks\": %d}",
                           mm::kBlockM, mm::kBlockN, mm::kBlockK, mm::kStages, MM_TOKEN_ALIGNMENT, MM_MAX_RANKS);
    MM_REQUIRE(n > 0 && n < capacity, "mm_build_config: buffer too small");
    return 0;
}

int64_t mm_launch_count(void) { return g_launches.load(); }

int mm_set_stage_timing(int enable) {
    g_stage_timing.store(enable ? 1 : 0);
    return 0;
}

int mm_get_stage_times(float* ms, int n) {
    MM_REQUIRE(ms && n >= MM_NUM_STAGES, "mm_get_stage_times: need room for %d floats", MM_NUM_STAGES);
    std::lock_guard<std::mutex> lk(g_stage_mu);
    MM_REQUIRE(g_stage_ev_made, "no timed call has been made");
    for (int i = 0; i < MM_NUM_STAGES; ++i) ms[i] = -1.0f;
    if (g_stage_count == 0) return 0;
    MM_CUDA(cudaEventSynchronize(g_stage_ev[g_stage_order[g_stage_count - 1] + 1]));
    int prev = 0;                          // event index: 0 = start of the call, id + 1 = end of stage id
    for (int k = 0; k < g_stage_count; ++k) {
        const int id = g_stage_order[k];
        MM_CUDA(cudaEventElapsedTime(&ms[id], g_stage_ev[prev], g_stage_ev[id + 1]));
        prev = id + 1;
    }
    return 0;
}

}  // extern "C"
