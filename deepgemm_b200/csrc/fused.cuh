// The whole layer as ONE persistent, warp-specialised kernel (small and medium token counts).
//
// Replaces mega_moe_multirank_persistent_w8a8_channelwise_kernel
// (deep_gemm/include/deep_gemm/impls/mega_moe_dcu.cuh:259-765).  One CTA per SM, launched cooperatively so that all
// CTAs are resident (they wait on one another).  Timeline of a CTA:
//   1. every CTA histograms this rank's routes in shared memory; CTA 0 publishes the count vector to all ranks;
//   2. wait (bounded) for all ranks' count vectors, derive the plan (totals, pool offsets, m-block table) locally;
//   3. push this CTA's share of the routed rows to the owners' pools over NVLink; every row bumps the owner's per-m-block
//      arrival counter (red.release.sys);
//   4. tile loop, round-robin over CTAs, with the same TMA / MMA / epilogue warp roles as grouped_gemm_kernel.  The
//      m-blocks are grouped in waves; GEMM1 tiles of wave k+2, requantisation tiles of wave k and GEMM2 tiles of wave k
//      alternate (see WaveOrder), so the tensor-bound GEMM1 work overlaps the NVLink-bound combine stores of GEMM2.
//      Dependencies are per m-block, not global barriers:
//        - GEMM1 tile: weights start streaming at once; the token operand waits for the m-block's arrival counter; each
//          epilogue warp counts its stored share in l1_done[m-block];
//        - requantisation tile (epilogue warps only, the MMA pipeline runs on): waits for all GEMM1 tiles of the m-block,
//          turns its bf16 rows into e4m3 (the channelwise scale needs the whole row) and sets l2_ready[m-block];
//        - GEMM2 tile: the activation operand waits for l2_ready[m-block] == 4; its epilogue stores to the source rank;
//   5. grid barrier -> CTA 0 tells every rank "my combine stores are done"; wait for all ranks; top-k reduce; clean up.
// Every wait is for tiles earlier in the tile order (or for dispatch), and every role of a CTA walks its tiles in order,
// so the waits cannot form a cycle.  Every wait is bounded and ends in a status code, never in a hang.
// gemm_only = 1 runs step 4 alone, between the staged routing / dispatch launches and the staged combine barrier and
// reduce launches (any token count); the host resets the dependency counters afterwards.
#pragma once
#include "gemm.cuh"
#include "misc.cuh"
#include "route.cuh"

namespace mm {

constexpr int kFusedMaxRoutes = 4096;      // routes of this rank held in shared memory (tokens * top-k)
constexpr int kFusedThreads = kGemmThreads;

struct FusedParams {
    RouteParams rp;
    GemmParams g1, g2;
    __nv_bfloat16* y;
    int* l1_done;          // [4 * m-blocks]
    int* l2_ready;         // [m-blocks]
    int* grid_sync;        // [0] CTA arrivals (monotonic), [1] fused calls completed
    uint8_t* act_fp8;      // [pool_rows][I]
    float* act_scale_w;    // writable alias of g2.act_scale
    int wave_mblocks;      // m-blocks per wave of the tile order (see decode_tile)
    int gemm_only;         // 1: routing and dispatch were done by the staged kernels (and a dispatch barrier); start at the tile loop
};

// shared-memory scratch of the routing phases, aliased onto the (not yet used) operand ring
struct FusedRouteSmem {
    int hist[MM_MAX_EXPERTS];        // this rank's routes per expert
    int tot[MM_MAX_EXPERTS];         // rows received by each expert (all ranks)
    int dest[MM_MAX_EXPERTS];        // first pool row on the owner for this rank's routes to the expert
    int off[MM_MAX_EXPERTS];         // pool offset of the expert on its owner
    short expert[kFusedMaxRoutes];   // expert of each local route, -1 = invalid
};
static_assert(sizeof(FusedRouteSmem) <= kStages * kStageBytes, "routing scratch must fit in the operand ring");

// Spin (bounded) until *flag - target >= 0.  `sys` selects system scope (flag written by another GPU).
// Gives up when the time budget is spent or another wait of the grid already failed (status code set).
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int target, bool sys, const int* status_code, uint64_t timeout_ns,
                                             int* observed) {
    int v = sys ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    if (v - target >= 0) { *observed = v; return true; }
    const uint64_t t0 = global_timer_ns();
    uint32_t it = 0;
    while (true) {
        v = sys ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
        if (v - target >= 0) { *observed = v; return true; }
        if ((++it & 15u) == 0u) {
            if (ld_acquire_gpu(status_code) != 0 || global_timer_ns() - t0 > timeout_ns) { *observed = v; return false; }
        }
        __nanosleep(40);
    }
}

// Position of a tile index in the wave order of the kernel below.  A CTA's tile indices grow, so seek() only moves forward.
struct WaveOrder {
    enum { kG1 = 0, kRequant = 1, kG2 = 2 };
    int n_waves, wave_m, num_mblocks, nb1, nb2;
    int g, base, size, kind, wave;
    __device__ WaveOrder(int num_mblocks_, int wave_m_, int nb1_, int nb2_)
        : n_waves((num_mblocks_ + wave_m_ - 1) / wave_m_), wave_m(wave_m_), num_mblocks(num_mblocks_), nb1(nb1_), nb2(nb2_),
          g(0), base(0) { set(); }
    __device__ __forceinline__ int wave_mblocks(int w) const { return w < n_waves ? min(wave_m, num_mblocks - w * wave_m) : 0; }
    __device__ __forceinline__ void set() {      // groups: G1(0), G1(1), then triples R(k), G1(k+2), G2(k)
        if (g < 2) { kind = kG1; wave = g; }
        else {
            const int k = (g - 2) / 3, j = (g - 2) - 3 * k;
            kind = j == 0 ? kRequant : (j == 1 ? kG1 : kG2);
            wave = j == 1 ? k + 2 : k;
        }
        size = wave_mblocks(wave) * (kind == kG1 ? nb1 : (kind == kRequant ? 1 : nb2));
    }
    // tile -> (kind, m-block, n-block); the caller guarantees tile < num_mblocks * (nb1 + 1 + nb2)
    __device__ __forceinline__ void seek(int tile, int& kind_out, int& mb, int& nb) {
        while (tile >= base + size) { base += size; ++g; set(); }
        const int r = tile - base;
        const int per = kind == kG1 ? nb1 : (kind == kRequant ? 1 : nb2);
        mb = wave * wave_m + r / per;
        nb = r - (r / per) * per;
        kind_out = kind;
    }
};

__global__ void __launch_bounds__(kFusedThreads, 1)
mega_moe_fused_kernel(const __grid_constant__ CUtensorMap tm_pool, const __grid_constant__ CUtensorMap tm_w1,
                      const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_w2, FusedParams fp) {
    const RouteParams& rp = fp.rp;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    uint8_t* smem_gen = smem_raw;
    int* status = fp.g1.status;
    if ((smem_base & 1023u) != 0u) {
        if (threadIdx.x == 0 && atomicCAS(status, 0, MM_ERR_PIPE_TIMEOUT) == 0) { status[1] = 102; status[2] = blockIdx.x; }
        return;
    }
    const uint32_t staging_u32 = smem_base + kStages * kStageBytes;
    uint8_t* staging_gen = smem_gen + kStages * kStageBytes;
    float* scales_gen = reinterpret_cast<float*>(staging_gen + kStagingBytes);
    const uint32_t bars = staging_u32 + kStagingBytes + kScaleBytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kStages + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * kStages + 2 + a); };
    uint8_t* tail = smem_gen + kStages * kStageBytes + kStagingBytes + kScaleBytes + 8 * (2 * kStages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8);
    int* s_misc = reinterpret_cast<int*>(tail + 16);       // [0] number of m-blocks, [1] ok flag of block-wide waits, [2] rows to receive, [3] requant-owner flag
    FusedRouteSmem& rs = *reinterpret_cast<FusedRouteSmem*>(smem_gen);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tid = threadIdx.x, nthr = blockDim.x;
    // timeline of CTA 0 (tenths of a microsecond since kernel entry) in the spare status words, for tuning:
    // [5] plan ready, [6] rows pushed, [7] producer done, [8] MMA done, [9] epilogue done, [10] all ranks done, [11] reduced
    const uint64_t t_entry = global_timer_ns();
    auto stamp = [&](int slot) { if (blockIdx.x == 0) status[slot] = static_cast<int>((global_timer_ns() - t_entry) / 100); };

    // ------------------------------------------------------------------ phase 0: barriers, TMEM, call identity
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), kEpilogueWarps); }
        *abort_flag = 0;
        s_misc[0] = 0; s_misc[1] = 1; s_misc[2] = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_pool); prefetch_tensormap(&tm_w1); prefetch_tensormap(&tm_act); prefetch_tensormap(&tm_w2);
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    // the epoch words are only rewritten at the very end of the kernel, after every CTA has passed the grid barrier
    const int epoch = reinterpret_cast<const int*>(rp.scratch + rp.cl.epoch)[0] + (fp.gemm_only ? 0 : 1);
    const int fused_calls = fp.grid_sync[1];
    const int n_tokens = route_num_tokens(rp);
    const int n_routes = n_tokens * rp.K;
    for (int e = tid; e < rp.E; e += nthr) rs.hist[e] = 0;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (!fp.gemm_only) {
    // ------------------------------------------------------------------ phase 1: local histogram, publish counts
    {
        const int64_t* idx = reinterpret_cast<const int64_t*>(rp.sym + rp.sl.topk_idx);
        const float* tw = reinterpret_cast<const float*>(rp.sym + rp.sl.topk_weights);
        for (int i = tid; i < n_routes; i += nthr) {
            const int64_t e64 = idx[i];
            const bool ok = e64 >= 0 && e64 < rp.E && tw[i] != 0.0f;
            rs.expert[i] = ok ? static_cast<short>(e64) : static_cast<short>(-1);
            if (ok) atomicAdd(&rs.hist[static_cast<int>(e64)], 1);
        }
    }
    __syncthreads();
    if (blockIdx.x == 0) {
        for (int i = tid; i < rp.R * rp.E; i += nthr) {
            const int r = i / rp.E, e = i - r * rp.E;
            int* cm = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(rp.peers[r]) + rp.sl.count_matrix);
            cm[static_cast<int64_t>(rp.rank) * rp.E + e] = rs.hist[e];
        }
        __threadfence_system();
        __syncthreads();
        if (tid < rp.R) {
            int* sig = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(rp.peers[tid]) + rp.sl.signals);
            st_release_sys(sig + MM_BAR_COUNTS * MM_MAX_RANKS + rp.rank, epoch);
        }
    }

    // ------------------------------------------------------------------ phase 2: all ranks' counts, plan
    if (tid < rp.R) {
        int seen = 0;
        const int* sig = reinterpret_cast<const int*>(rp.sym + rp.sl.signals) + MM_BAR_COUNTS * MM_MAX_RANKS + tid;
        if (!wait_flag_ge(sig, epoch, true, status, rp.barrier_timeout_ns, &seen)) {
            report_status(rp.scratch, rp.cl, MM_ERR_RANK_BARRIER_TIMEOUT, MM_BAR_COUNTS, tid, epoch, seen);
            s_misc[1] = 0;
        }
    }
    __syncthreads();
    {
        const int* cm = reinterpret_cast<const int*>(rp.sym + rp.sl.count_matrix);
        for (int e = tid; e < rp.E; e += nthr) {
            int t = 0, b = 0;
            for (int r = 0; r < rp.R; ++r) {
                const int c = __ldcg(cm + static_cast<int64_t>(r) * rp.E + e);
                if (r < rp.rank) b += c;
                t += c;
            }
            rs.tot[e] = t;
            rs.dest[e] = b;      // rows of lower ranks for now; the pool offset is added below
        }
    }
    __syncthreads();
    if (tid < rp.R) {            // one thread per owner: exclusive prefix of padded totals over its experts
        int run = 0, rows = 0;
        for (int le = 0; le < rp.E_loc; ++le) {
            const int e = tid * rp.E_loc + le;
            rs.off[e] = run;
            rows += rs.tot[e];
            run += (rs.tot[e] + MM_BLOCK_M - 1) / MM_BLOCK_M * MM_BLOCK_M;
        }
        if (tid == rp.rank) {
            s_misc[2] = rows;             // rows this rank receives in total
            if (run > rp.sl.pool_rows) {
                report_status(rp.scratch, rp.cl, MM_ERR_POOL_OVERFLOW, 0, rp.rank, static_cast<int>(rp.sl.pool_rows), run);
                s_misc[1] = 0;
                run = 0;
            }
            s_misc[0] = run / MM_BLOCK_M;
            int* plan = reinterpret_cast<int*>(rp.scratch + rp.cl.plan);
            plan[0] = run / MM_BLOCK_M;   // every CTA writes the same values
            plan[1] = run;
        }
    }
    __syncthreads();
    {
        // m-block table of the local experts: identical in every CTA, written to global memory by all of them
        int* e_tot = reinterpret_cast<int*>(rp.scratch + rp.cl.expert_total);
        int* e_off = reinterpret_cast<int*>(rp.scratch + rp.cl.expert_off);
        int* mb_e = const_cast<int*>(fp.g1.mblock_expert);
        int* mb_v = const_cast<int*>(fp.g1.mblock_valid);
        int* dest_base = reinterpret_cast<int*>(rp.scratch + rp.cl.dest_base);
        for (int e = tid; e < rp.E; e += nthr) {
            rs.dest[e] += rs.off[e];
            dest_base[e] = rs.dest[e];
        }
        if (s_misc[1]) {
            for (int le = tid; le < rp.E_loc; le += nthr) {
                const int e = rp.rank * rp.E_loc + le;
                const int t = rs.tot[e], o = rs.off[e];
                e_tot[le] = t;
                e_off[le] = o;
                if (rp.stats && blockIdx.x == 0) rp.stats[le] += t;
                for (int m = 0; m * MM_BLOCK_M < t; ++m) {
                    mb_e[o / MM_BLOCK_M + m] = le;
                    mb_v[o / MM_BLOCK_M + m] = min(MM_BLOCK_M, t - m * MM_BLOCK_M);
                }
            }
        }
    }
    } else if (tid == 0) {
        s_misc[0] = fp.g1.plan[0];      // the plan was made by route_plan_kernel
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) stamp(5);
    const int num_mblocks = s_misc[0];
    const bool healthy = s_misc[1] != 0;
    const int rows_expected = s_misc[2];
    const int arrive_total_slot = static_cast<int>(rp.sl.pool_rows / MM_BLOCK_M);   // last word of the arrival array

    // ------------------------------------------------------------------ phase 3: push this CTA's share of the rows
    if (healthy && !fp.gemm_only) {
        const uint8_t* x = rp.sym + rp.sl.x;
        const float* x_sf = reinterpret_cast<const float*>(rp.sym + rp.sl.x_sf);
        const float* tw = reinterpret_cast<const float*>(rp.sym + rp.sl.topk_weights);
        int* dest_row = reinterpret_cast<int*>(rp.scratch + rp.cl.dest_row);
        const int warps_per_cta = nthr >> 5;
        for (int i = blockIdx.x * warps_per_cta + warp; i < n_routes; i += gridDim.x * warps_per_cta) {
            const int e = rs.expert[i];
            if (e < 0) { if (lane == 0) dest_row[i] = -1; continue; }
            // slot inside the expert: routes of this rank are ordered by (token, top-k slot) == route index
            int within = 0;
            for (int j = lane; j < i; j += 32) within += (rs.expert[j] == e);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) within += __shfl_xor_sync(0xffffffffu, within, o);
            const int row = rs.dest[e] + within;
            if (lane == 0) dest_row[i] = row;
            const int token = i / rp.K, slot = i - token * rp.K;
            uint8_t* peer = reinterpret_cast<uint8_t*>(rp.peers[e / rp.E_loc]);
            const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(token) * rp.H);
            uint4* dst = reinterpret_cast<uint4*>(peer + rp.sl.pool_x + static_cast<int64_t>(row) * rp.H);
            const int nvec = rp.H / 16;
            for (int v0 = 0; v0 < nvec; v0 += 32 * 8) {
                uint4 buf[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) { const int v = v0 + k * 32 + lane; if (v < nvec) buf[k] = __ldg(src + v); }
#pragma unroll
                for (int k = 0; k < 8; ++k) { const int v = v0 + k * 32 + lane; if (v < nvec) dst[v] = buf[k]; }
            }
            if (lane == 0) {
                MmPoolMeta m;
                m.x_scale = x_sf[token];
                m.route_weight = tw[i];
                m.src_token = token;
                m.src_info = (rp.rank << 8) | slot;
                *reinterpret_cast<uint4*>(peer + rp.sl.pool_meta + static_cast<int64_t>(row) * sizeof(MmPoolMeta)) =
                    *reinterpret_cast<uint4*>(&m);
            }
        }
        // All rows of this warp are written: one system-scope fence (ordered after the other lanes' stores by the warp
        // barrier), then the arrival counters of all its rows, one row per lane, as relaxed reductions.
        __syncwarp();
        __threadfence_system();
        for (int i0 = blockIdx.x * warps_per_cta + warp; i0 < n_routes; i0 += 32 * gridDim.x * warps_per_cta) {
            const int i = i0 + lane * gridDim.x * warps_per_cta;
            if (i < n_routes) {
                const int e = rs.expert[i];
                if (e >= 0) {
                    const int row = __ldcg(dest_row + i);     // written by lane 0 above, before the fence
                    int* arr = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(rp.peers[e / rp.E_loc]) + rp.sl.pool_arrive);
                    asm volatile("red.relaxed.sys.global.add.s32 [%0], 1;" ::"l"(arr + row / MM_BLOCK_M) : "memory");
                    asm volatile("red.relaxed.sys.global.add.s32 [%0], 1;" ::"l"(arr + arrive_total_slot) : "memory");
                }
            }
        }
    }
    // the routing scratch is dead from here on; the operand ring (same shared memory) is written by TMA next
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) stamp(6);

    // ------------------------------------------------------------------ phase 4: GEMM1 tiles, then GEMM2 tiles
    const GemmParams& g1 = fp.g1;
    const GemmParams& g2 = fp.g2;
    // Tile order: m-blocks are grouped in waves of `wave_mblocks`; with G1(k) / G2(k) = all GEMM1 / GEMM2 tiles of wave k
    // and R(k) = one requantisation tile per m-block of wave k (epilogue warps only), the global order is
    //     G1(0), G1(1), [R(0), G1(2), G2(0)], [R(1), G1(3), G2(1)], ..., [R(n-1), G2(n-1)]
    // Interleaving the two GEMMs spreads the combine stores (NVLink) over the whole compute phase; R(k) comes a full
    // wave after G1(k) and G2(k) a full wave after R(k), so their waits are normally satisfied on arrival.
    // Every wait is for tiles that come earlier in this order and every role of a CTA walks its tiles in order, so the
    // waits cannot form a cycle.
    const int nb1 = g1.n_blocks, nb2 = g2.n_blocks;
    const WaveOrder order_init(num_mblocks, max(1, fp.wave_mblocks), nb1, nb2);
    const int tiles_all = healthy ? num_mblocks * (nb1 + 1 + nb2) : 0;
    const int* arrive = reinterpret_cast<const int*>(rp.sym + rp.sl.pool_arrive);

    // Requantisation tile, run by all eight epilogue warps: wait until every GEMM1 tile of the m-block is stored (each
    // epilogue warp of each of its n_blocks tiles counts once), turn its bf16 rows into e4m3 with one scale per row, two
    // rows per warp at a time, and release the m-block to GEMM2.
    auto requantise_mblock = [&](int mb) -> bool {
        const int valid = g1.mblock_valid[mb];
        if (warp == 2 && lane == 0) {
            int seen = 0;
            const int target = nb1 * kEpilogueWarps;
            const bool ok = wait_flag_ge(fp.l1_done + mb, target, false, status, g1.timeout_ns, &seen);
            if (!ok) {
                report_status(rp.scratch, rp.cl, MM_ERR_GRID_BARRIER_TIMEOUT, 4, mb, target, seen);
                *abort_flag = 1;
            }
            s_misc[3] = ok ? 1 : 0;
        }
        named_bar_sync(2, kEpilogueThreads);
        const bool ok = s_misc[3] != 0;
        if (ok) {
            __threadfence();
            const int inter = g1.n_out, vecs = inter / 8;
            const int ew = warp - 2;
            for (int r = ew; r < valid; r += 2 * kEpilogueWarps) {
                uint4 buf[2][8];
                float inv[2], sc2[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int64_t prow = static_cast<int64_t>(mb) * kBlockM + min(r + u * kEpilogueWarps, valid - 1);
                    const float amax = __uint_as_float(__ldcg(g1.row_amax + prow));
                    sc2[u] = fmaxf(__fdiv_rn(amax, 448.0f), 1.0e-4f);
                    inv[u] = __fdiv_rn(1.0f, sc2[u]);
                    const uint4* src = reinterpret_cast<const uint4*>(g1.act_bf16 + prow * inter);
#pragma unroll
                    for (int k = 0; k < 8; ++k) { const int v = k * 32 + lane; if (v < vecs) buf[u][k] = __ldcg(src + v); }
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (r + u * kEpilogueWarps >= valid) continue;
                    const int64_t prow = static_cast<int64_t>(mb) * kBlockM + r + u * kEpilogueWarps;
                    const uint4* src = reinterpret_cast<const uint4*>(g1.act_bf16 + prow * inter);
                    uint2* dst = reinterpret_cast<uint2*>(fp.act_fp8 + prow * inter);
                    for (int v0 = 0; v0 < vecs; v0 += 32 * 8) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            const int v = v0 + k * 32 + lane;
                            if (v < vecs) {
                                const uint4 d = (v0 == 0) ? buf[u][k] : __ldcg(src + v);
                                uint2 o;
                                o.x = pack4_e4m3(bf16_lo(d.x) * inv[u], bf16_hi(d.x) * inv[u], bf16_lo(d.y) * inv[u], bf16_hi(d.y) * inv[u]);
                                o.y = pack4_e4m3(bf16_lo(d.z) * inv[u], bf16_hi(d.z) * inv[u], bf16_lo(d.w) * inv[u], bf16_hi(d.w) * inv[u]);
                                dst[v] = o;
                            }
                        }
                    }
                    if (lane == 0) { fp.act_scale_w[prow] = sc2[u]; g1.row_amax[prow] = 0u; }
                }
            }
        }
        named_bar_sync(2, kEpilogueThreads);             // all rows of the m-block are requantised
        if (ok && warp == 2 && lane == 0) {
            __threadfence();
            atomicAdd(fp.l2_ready + mb, 4);              // GEMM2 producers wait for 4
            atomicAdd(fp.grid_sync + 2, 1);
        }
        return ok;
    };

    if (warp == 0) {
        // -------------------------------------------------------------- TMA producer
        int stage = 0; uint32_t phase = 0;
        bool alive = true;
        // once every row has arrived (every m-block is requantised) no further per-tile polling is needed
        bool all_arrived = fp.gemm_only != 0, all_ready = false;
        WaveOrder order = order_init;
        for (int tile = blockIdx.x; tile < tiles_all && alive; tile += gridDim.x) {
            int kind, mb, nb;
            order.seek(tile, kind, mb, nb);
            if (kind == WaveOrder::kRequant) continue;          // epilogue warps only
            const bool second = kind == WaveOrder::kG2;
            const GemmParams& g = second ? g2 : g1;
            const int e = g.mblock_expert[mb];
            const int k_blocks = g.kdim / kBlockK;
            const int b_tile0 = (e * g.n_blocks + nb) * k_blocks;
            const CUtensorMap* ta = second ? &tm_act : &tm_pool;
            const CUtensorMap* tb = second ? &tm_w2 : &tm_w1;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, g.timeout_ns)) { alive = false; break; }
                const uint32_t a_dst = smem_base + stage * kStageBytes;
                if (lane == 0) {
                    mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
                    tma_load_2d(a_dst + kABytes, tb, 0, (b_tile0 + kb) * kBlockN, full_bar(stage));   // weights first
                }
                if (kb == 0 && !(second ? all_ready : all_arrived)) {
                    // the token operand of this m-block must be complete before TMA may read it
                    int seen = 0;
                    bool ok = true;
                    if (second) {
                        all_ready = ld_acquire_gpu(fp.grid_sync + 2) - num_mblocks >= 0;
                        if (!all_ready) ok = wait_flag_ge(fp.l2_ready + mb, 4, false, status, g.timeout_ns, &seen);
                    } else {
                        all_arrived = ld_acquire_sys(arrive + arrive_total_slot) - rows_expected >= 0;
                        if (!all_arrived) ok = wait_flag_ge(arrive + mb, g.mblock_valid[mb], true, status, rp.barrier_timeout_ns, &seen);
                    }
                    if (!ok) {
                        if (lane == 0) report_status(rp.scratch, rp.cl, MM_ERR_GRID_BARRIER_TIMEOUT, second ? 2 : 1, mb,
                                                     second ? 4 : g.mblock_valid[mb], seen);
                        *abort_flag = 1;
                        alive = false;
                    }
                    // rows were written with ordinary stores (by other SMs or GPUs); order them before the TMA reads
                    asm volatile("fence.proxy.async;" ::: "memory");
                }
                // issue the token tile even on failure so that the stage's byte count completes and nobody is left waiting
                if (lane == 0) tma_load_2d(a_dst, ta, kb * kBlockK, mb * kBlockM, full_bar(stage));
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
                if (!alive) break;
            }
        }
        if (lane == 0) stamp(7);
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        constexpr uint32_t idesc = umma_idesc_f8(kBlockM, kBlockN);
        int stage = 0; uint32_t phase = 0;
        int acc = 0; uint32_t acc_phase = 0;
        bool alive = true;
        WaveOrder order = order_init;
        for (int tile = blockIdx.x; tile < tiles_all && alive; tile += gridDim.x) {
            int kind, mb, nb;
            order.seek(tile, kind, mb, nb);
            if (kind == WaveOrder::kRequant) continue;
            const GemmParams& g = kind == WaveOrder::kG2 ? g2 : g1;
            const int k_blocks = g.kdim / kBlockK;
            if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, g.timeout_ns)) { alive = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * kBlockN;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag, g.timeout_ns)) { alive = false; break; }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t a_src = smem_base + stage * kStageBytes;
                    const uint64_t da = umma_desc_k_sw128(a_src);
                    const uint64_t db = umma_desc_k_sw128(a_src + kABytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / 32; ++k) umma_f8(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit(empty_bar(stage));
                    if (kb == k_blocks - 1) umma_commit(tfull_bar(acc));
                }
                __syncwarp();
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (lane == 0) stamp(8);
    } else {
        // -------------------------------------------------------------- epilogue (warps 2..9)
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const int et = q * 32 + lane;
        uint8_t* my_staging = staging_gen + (warp - 2) * kStagingWarpBytes;
        const bool do_clamp = g1.clamp < 3.0e38f;
        int acc = 0; uint32_t acc_phase = 0;
        bool alive = true;
        WaveOrder order = order_init;
        for (int tile = blockIdx.x; tile < tiles_all && alive; tile += gridDim.x) {
            if (*abort_flag != 0) break;
            int kind, mb, nb;
            order.seek(tile, kind, mb, nb);
            if (kind == WaveOrder::kRequant) {
                if (!requantise_mblock(mb)) { alive = false; break; }
                continue;
            }
            const bool second = kind == WaveOrder::kG2;
            const GemmParams& g = second ? g2 : g1;
            const int e = g.mblock_expert[mb];
            const int valid = g.mblock_valid[mb];
            const int row = mb * kBlockM + et;
            const bool row_ok = et < valid;
            float* sc = scales_gen + acc * kBlockN;
            {
                const int st = (warp - 2) * 32 + lane;
                const float* ws = g.w_scale + static_cast<int64_t>(e) * g.w_rows_per_expert;
                if (!second) {
                    sc[st] = st < 128 ? ws[nb * 128 + st] : ws[g.w_rows_per_expert / 2 + nb * 128 + (st - 128)];
                } else {
                    const int c0 = nb * kBlockN + st;
                    sc[st] = c0 < g.n_out ? ws[c0] : 0.0f;
                }
            }
            named_bar_sync(1, kEpilogueThreads);
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, g.timeout_ns)) { alive = false; break; }
            tc_fence_after();
            // the accumulator is complete, so the m-block's rows (and, for GEMM2, its activation scales) are in place
            float row_scale = 0.0f, route_w = 0.0f;
            uint8_t* out_ptr = nullptr;
            if (row_ok) {
                const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(g.meta + row));
                if (!second) {
                    row_scale = __uint_as_float(raw.x);
                    route_w = __uint_as_float(raw.y);
                } else {
                    row_scale = __ldcg(g.act_scale + row);
                    const int src_info = static_cast<int>(raw.w);
                    const int src_rank = src_info >> 8, slot = src_info & 0xff;
                    out_ptr = reinterpret_cast<uint8_t*>(g.peers[src_rank]) + g.combine_off +
                              (static_cast<int64_t>(slot) * g.T + static_cast<int>(raw.z)) * g.H * 2;
                }
            }
            if (!second) epilogue_math<0>(g1, tmem_base, sc, my_staging, lane, q, half, acc, mb, nb, valid, row, row_ok, row_scale, route_w, out_ptr, do_clamp);
            else         epilogue_math<1>(g2, tmem_base, sc, my_staging, lane, q, half, acc, mb, nb, valid, row, row_ok, row_scale, route_w, out_ptr, do_clamp);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }

            if (!second) {
                // this warp's share of the tile (bf16 values, row amax) is stored: count it towards the m-block's GEMM1 total
                __syncwarp();
                if (lane == 0) {
                    __threadfence();
                    red_release_gpu_add(fp.l1_done + mb, 1);
                }
            }
        }
    }

    __threadfence_system();
    __syncthreads();
    if (tid == 0) stamp(9);
    // gemm_only: the combine barrier, the reduce and the counter reset are separate launches after this kernel
    if (!fp.gemm_only) {
    // ------------------------------------------------------------------ phase 5: all ranks' combine stores done
    const int grid_target = static_cast<int>(gridDim.x) * (fused_calls + 1);
    if (tid == 0) red_release_gpu_add(fp.grid_sync, 1);
    if (blockIdx.x == 0) {
        if (tid == 0) {
            int seen = 0;
            if (!wait_flag_ge(fp.grid_sync, grid_target, false, status, rp.barrier_timeout_ns, &seen))
                report_status(rp.scratch, rp.cl, MM_ERR_GRID_BARRIER_TIMEOUT, 3, blockIdx.x, grid_target, seen);
            __threadfence_system();
        }
        __syncthreads();
        if (tid < rp.R) {
            int* sig = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(rp.peers[tid]) + rp.sl.signals);
            st_release_sys(sig + MM_BAR_COMBINE * MM_MAX_RANKS + rp.rank, epoch);
        }
    }
    if (tid < rp.R) {      // includes this rank's own signal, which also stands for "all local CTAs are done"
        int seen = 0;
        const int* sig = reinterpret_cast<const int*>(rp.sym + rp.sl.signals) + MM_BAR_COMBINE * MM_MAX_RANKS + tid;
        if (!wait_flag_ge(sig, epoch, true, status, rp.barrier_timeout_ns, &seen))
            report_status(rp.scratch, rp.cl, MM_ERR_RANK_BARRIER_TIMEOUT, MM_BAR_COMBINE, tid, epoch, seen);
    }
    __syncthreads();
    if (tid == 0) stamp(10);

    // ------------------------------------------------------------------ phase 6: top-k reduce in slot order
    {
        const int vecs = rp.H / 8;
        const int64_t total = static_cast<int64_t>(n_tokens) * vecs;
        const int64_t* topk_idx = reinterpret_cast<const int64_t*>(rp.sym + rp.sl.topk_idx);
        const float* topk_w = reinterpret_cast<const float*>(rp.sym + rp.sl.topk_weights);
        const uint4* comb = reinterpret_cast<const uint4*>(rp.sym + rp.sl.combine);
        for (int64_t i = static_cast<int64_t>(blockIdx.x) * nthr + tid; i < total; i += static_cast<int64_t>(gridDim.x) * nthr) {
            const int t = static_cast<int>(i / vecs), v = static_cast<int>(i - static_cast<int64_t>(t) * vecs);
            float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int s0 = 0; s0 < rp.K; s0 += 6) {          // up to six slots' loads in flight, summed in slot order
                uint4 buf[6];
                bool ok[6];
#pragma unroll
                for (int j = 0; j < 6; ++j) {
                    const int s = s0 + j;
                    ok[j] = false;
                    if (s < rp.K) {
                        const int64_t e = topk_idx[static_cast<int64_t>(t) * rp.K + s];
                        const float w = topk_w[static_cast<int64_t>(t) * rp.K + s];
                        ok[j] = e >= 0 && e < rp.E && w != 0.0f;
                        if (ok[j]) buf[j] = __ldcg(comb + (static_cast<int64_t>(s) * rp.T + t) * vecs + v);
                    }
                }
#pragma unroll
                for (int j = 0; j < 6; ++j) {
                    if (!ok[j]) continue;
                    const uint4 d = buf[j];
                    a[0] += bf16_lo(d.x); a[1] += bf16_hi(d.x); a[2] += bf16_lo(d.y); a[3] += bf16_hi(d.y);
                    a[4] += bf16_lo(d.z); a[5] += bf16_hi(d.z); a[6] += bf16_lo(d.w); a[7] += bf16_hi(d.w);
                }
            }
            uint4 o;
            o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]); o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
            reinterpret_cast<uint4*>(fp.y)[i] = o;
        }
    }

    // ------------------------------------------------------------------ phase 7: leave the counters ready for the next call
    if (tid == 0) stamp(11);
    {
        int* arr = reinterpret_cast<int*>(rp.sym + rp.sl.pool_arrive);
        for (int i = blockIdx.x * nthr + tid; i < num_mblocks; i += gridDim.x * nthr) { arr[i] = 0; fp.l2_ready[i] = 0; }
        for (int i = blockIdx.x * nthr + tid; i < num_mblocks * 4; i += gridDim.x * nthr) fp.l1_done[i] = 0;
        if (blockIdx.x == 0 && tid == 0) {
            arr[arrive_total_slot] = 0;
            fp.grid_sync[2] = 0;
            reinterpret_cast<int*>(rp.scratch + rp.cl.epoch)[0] = epoch;
            fp.grid_sync[1] = fused_calls + 1;
        }
    }
    }   // !gemm_only
    if (*abort_flag != 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 1000000ull) __nanosleep(1000);
        if (tid == 0 && atomicCAS(status, 0, MM_ERR_PIPE_TIMEOUT) == 0) { status[1] = 2; status[2] = blockIdx.x; status[3] = tiles_all; status[4] = 0; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace mm
