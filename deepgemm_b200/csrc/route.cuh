// Routing and dispatch: per-expert histogram, count exchange, deterministic slot assignment, NVLink push.
//
// Replaces the reference's route scan + tile build + dispatch pull
// (deep_gemm/include/deep_gemm/impls/mega_moe_dcu.cuh:335-537, impls/mega_moe_dcu_task.cuh:55-150).  Differences:
//   * every rank scans only ITS OWN topk_idx and pushes rows to the owner (the reference scans all ranks' routes on
//     every rank and pulls);
//   * slots are a pure function of the inputs: an expert's rows are ordered by (source rank, token, top-k slot), the
//     reference leaves the order to atomicAdd (impls/mega_moe_dcu.cuh:359).
// Route validity is the reference's rule: 0 <= expert < E and weight != 0 (impls/mega_moe_dcu.cuh:350-354).
#pragma once
#include "layout.h"
#include "ptx.cuh"

namespace mm {

struct RouteParams {
    uint8_t* sym;            // local symmetric buffer
    uint8_t* scratch;        // local scratch
    uint64_t peers[MM_MAX_RANKS];
    MmSymLayout sl;
    MmScratchLayout cl;
    int rank, R, E, E_loc, T, K, H;
    int num_tokens;                  // host-side token count (ignored when runtime_num_tokens != nullptr)
    const int* runtime_num_tokens;   // device-side token count (graph mode) or nullptr
    int* stats;                      // cumulative_local_expert_recv_stats or nullptr
    uint64_t barrier_timeout_ns;
};

// Tokens of this call.  A device-side count (graph mode) is clamped to the launch-time count, which is the number of
// rows of y the caller provided (deep_gemm/include/deep_gemm/impls/mega_moe_dcu.cuh:292 clamps the same way), so a
// stale or oversized device value can never make a kernel write past the end of y.
__device__ __forceinline__ int route_num_tokens(const RouteParams& p) {
    const int bound = min(p.num_tokens, p.T);
    const int n = p.runtime_num_tokens ? *p.runtime_num_tokens : p.num_tokens;
    return min(max(n, 0), bound);
}

// True once a bounded wait of this buffer has expired (or the pool overflowed): every later kernel of the call, and of
// later calls until the buffers are re-initialised, returns at once instead of working on an unvalidated plan.
__device__ __forceinline__ bool call_failed(const uint8_t* scratch, const MmScratchLayout& cl) {
    return ld_acquire_gpu(reinterpret_cast<const int*>(scratch + cl.status)) != 0;
}

__device__ __forceinline__ void report_status(uint8_t* scratch, const MmScratchLayout& cl, int code, int phase, int rank,
                                              int expected, int observed) {
    MmStatus* st = reinterpret_cast<MmStatus*>(scratch + cl.status);
    if (atomicCAS(&st->code, 0, code) == 0) {
        st->phase = phase; st->rank = rank; st->expected = expected; st->observed = observed;
    }
}

// ---- 1. per-block histogram of valid routes; the block that finishes last turns the histograms into prefixes over the
//         blocks and publishes this rank's count vector to every rank -----------------------------------------------
// grid = route_blocks, block = 1024 threads; thread i < MM_ROUTE_CHUNK of block b owns route b*CHUNK + i (token-major).
__device__ __forceinline__ void route_exchange_block(const RouteParams& p, int* part_sum) {
    const int route_blocks = static_cast<int>(p.cl.route_blocks);
    int* bc = reinterpret_cast<int*>(p.scratch + p.cl.block_counts);
    // blockDim / E threads share one expert: each sums a contiguous range of blocks, then turns its range into an
    // exclusive prefix starting from the ranges before it (loads are independent, so they overlap)
    const int parts = max(1, min(static_cast<int>(blockDim.x) / p.E, 32));
    const int per = (route_blocks + parts - 1) / parts;
    for (int e0 = 0; e0 < p.E; e0 += blockDim.x / parts) {
        const int e = e0 + threadIdx.x % (blockDim.x / parts);
        const int part = threadIdx.x / (blockDim.x / parts);
        const bool on = e < p.E && part < parts;
        const int b0 = part * per, b1 = min(route_blocks, b0 + per);
        int sum = 0;
        if (on) {
#pragma unroll 8
            for (int b = b0; b < b1; ++b) sum += __ldcg(bc + static_cast<int64_t>(b) * p.E + e);
        }
        part_sum[threadIdx.x] = sum;
        __syncthreads();
        if (on) {
            int run = 0;
            for (int q = 0; q < part; ++q) run += part_sum[q * (blockDim.x / parts) + threadIdx.x % (blockDim.x / parts)];
            int vals[8];
            for (int b = b0; b < b1; b += 8) {
#pragma unroll
                for (int i = 0; i < 8; ++i) vals[i] = (b + i < b1) ? __ldcg(bc + static_cast<int64_t>(b + i) * p.E + e) : 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (b + i < b1) bc[static_cast<int64_t>(b + i) * p.E + e] = run;   // rows of earlier blocks
                    run += vals[i];
                }
            }
            if (part == parts - 1) {
                for (int r = 0; r < p.R; ++r) {
                    int* cm = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(p.peers[r]) + p.sl.count_matrix);
                    cm[static_cast<int64_t>(p.rank) * p.E + e] = run;
                }
            }
        }
        __syncthreads();
    }
    if (p.R > 1) {
        __threadfence_system();
        __syncthreads();
        const int epoch = reinterpret_cast<const int*>(p.scratch + p.cl.epoch)[0];
        if (threadIdx.x < p.R) {
            int* sig = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(p.peers[threadIdx.x]) + p.sl.signals);
            st_release_sys(sig + MM_BAR_COUNTS * MM_MAX_RANKS + p.rank, epoch);
        }
    }
}

__global__ void __launch_bounds__(1024) route_count_kernel(RouteParams p) {
    __shared__ int hist[MM_MAX_EXPERTS];           // later reused as the partial sums of the exchange step
    __shared__ int s_last;
    const int n_routes = route_num_tokens(p) * p.K;
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const int route = blockIdx.x * MM_ROUTE_CHUNK + threadIdx.x;
    if (threadIdx.x < MM_ROUTE_CHUNK && route < n_routes) {
        const int64_t e = reinterpret_cast<const int64_t*>(p.sym + p.sl.topk_idx)[route];
        const float w = reinterpret_cast<const float*>(p.sym + p.sl.topk_weights)[route];
        if (e >= 0 && e < p.E && w != 0.0f) atomicAdd(&hist[static_cast<int>(e)], 1);
    }
    __syncthreads();
    int* bc = reinterpret_cast<int*>(p.scratch + p.cl.block_counts) + static_cast<int64_t>(blockIdx.x) * p.E;
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) bc[e] = hist[e];
    // the last block to get here has every block's histogram in front of it
    int* epoch = reinterpret_cast<int*>(p.scratch + p.cl.epoch);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int done = atomicAdd(epoch + 1, 1) + 1;
        s_last = done == static_cast<int>(gridDim.x) ? 1 : 0;
        if (s_last) {
            epoch[1] = 0;                          // ready for the next call
            epoch[0] = epoch[0] + 1;               // one epoch per layer call; later kernels of the call read it
            __threadfence();
        }
    }
    __syncthreads();
    if (s_last) route_exchange_block(p, hist);
}

// Bounded wait until every rank has published `epoch` on barrier `bar` of the LOCAL signal block.
// Called by the first R threads of a block; returns false on timeout (status recorded).
__device__ __forceinline__ bool wait_rank_signals(const RouteParams& p, int bar, int epoch) {
    bool ok = true;
    if (threadIdx.x < p.R) {
        const int* sig = reinterpret_cast<const int*>(p.sym + p.sl.signals) + bar * MM_MAX_RANKS + threadIdx.x;
        const uint64_t t0 = global_timer_ns();
        int v;
        while ((v = ld_acquire_sys(sig)) - epoch < 0) {
            if (global_timer_ns() - t0 > p.barrier_timeout_ns) {
                report_status(p.scratch, p.cl, MM_ERR_RANK_BARRIER_TIMEOUT, bar, threadIdx.x, epoch, v);
                ok = false;
                break;
            }
            __nanosleep(100);
        }
    }
    return ok;
}

// ---- 3. plan: totals, pool offsets, m-block table, destination bases ------------------------------------------
// grid = 1, block = 1024.  Waits (bounded) for all ranks' count vectors when R > 1.
__global__ void __launch_bounds__(1024) route_plan_kernel(RouteParams p) {
    __shared__ int tot[MM_MAX_EXPERTS];
    __shared__ int before[MM_MAX_EXPERTS];
    __shared__ int off[MM_MAX_EXPERTS];
    int* plan_w = reinterpret_cast<int*>(p.scratch + p.cl.plan);
    bool ok = !call_failed(p.scratch, p.cl);
    if (ok && p.R > 1) {
        const int epoch = reinterpret_cast<const int*>(p.scratch + p.cl.epoch)[0];
        ok = wait_rank_signals(p, MM_BAR_COUNTS, epoch);
    }
    if (!__syncthreads_and(ok)) {
        // a rank's counts never arrived: leave an empty plan so that nothing downstream touches the pool or y
        if (threadIdx.x == 0) { plan_w[0] = 0; plan_w[1] = 0; plan_w[2] = 0; plan_w[3] = 0; }
        return;
    }
    const int* cm = reinterpret_cast<const int*>(p.sym + p.sl.count_matrix);
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
        int t = 0, b = 0;
        for (int r = 0; r < p.R; ++r) {
            const int c = cm[static_cast<int64_t>(r) * p.E + e];
            if (r < p.rank) b += c;
            t += c;
        }
        tot[e] = t;
        before[e] = b;
    }
    __syncthreads();
    if (threadIdx.x < p.R) {   // one thread per owner: exclusive prefix of padded totals over its experts
        int run = 0, pairs = 0;
        for (int le = 0; le < p.E_loc; ++le) {
            const int e = threadIdx.x * p.E_loc + le;
            off[e] = run;
            const int blocks = (tot[e] + MM_BLOCK_M - 1) / MM_BLOCK_M;
            run += blocks * MM_BLOCK_M;
            pairs += (blocks + 1) / 2;      // two m-blocks of one expert share a weight tile in the CTA-pair GEMMs
        }
        if (threadIdx.x == p.rank) {
            int* plan = reinterpret_cast<int*>(p.scratch + p.cl.plan);
            int rows = 0;
            for (int le = 0; le < p.E_loc; ++le) rows += tot[p.rank * p.E_loc + le];
            plan[0] = run / MM_BLOCK_M;
            plan[1] = run;
            plan[2] = pairs;
            plan[6] = rows;                          // valid rows this rank receives
            if (run > p.sl.pool_rows) report_status(p.scratch, p.cl, MM_ERR_POOL_OVERFLOW, 0, p.rank, (int)p.sl.pool_rows, run);
        }
    }
    __syncthreads();
    int* dest_base = reinterpret_cast<int*>(p.scratch + p.cl.dest_base);
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) dest_base[e] = off[e] + before[e];
    // Send order of this rank's routes: by local expert index first, then by owner starting with the rank after this one
    // (so that at any moment the ranks fill the same expert of every owner, and no two ranks start on the same owner).
    // send_base[e] = exclusive prefix of this rank's own counts in that order.  E <= blockDim.x.
    {
        __shared__ int s_cnt[MM_MAX_EXPERTS];
        __shared__ int s_warp[32];
        auto order_of = [&](int e) { const int owner = e / p.E_loc, le = e - owner * p.E_loc; return le * p.R + (owner - p.rank - 1 + p.R) % p.R; };
        for (int e = threadIdx.x; e < p.E; e += blockDim.x) s_cnt[order_of(e)] = cm[static_cast<int64_t>(p.rank) * p.E + e];
        __syncthreads();
        const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
        const int v = static_cast<int>(threadIdx.x) < p.E ? s_cnt[threadIdx.x] : 0;
        int inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += t; }
        if (lane == 31) s_warp[wid] = inc;
        __syncthreads();
        if (wid == 0) {
            int w = s_warp[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w += t; }
            s_warp[lane] = w;                       // inclusive prefix of the warp totals
        }
        __syncthreads();
        const int excl = inc - v + (wid > 0 ? s_warp[wid - 1] : 0);
        __syncthreads();
        if (static_cast<int>(threadIdx.x) < p.E) s_cnt[threadIdx.x] = excl;
        __syncthreads();
        int* send_base = reinterpret_cast<int*>(p.scratch + p.cl.send_base);
        for (int e = threadIdx.x; e < p.E; e += blockDim.x) send_base[e] = s_cnt[order_of(e)];
        if (threadIdx.x == 0) plan_w[3] = s_warp[31];     // valid routes of this rank == length of the send list
    }
    int* e_tot = reinterpret_cast<int*>(p.scratch + p.cl.expert_total);
    int* e_off = reinterpret_cast<int*>(p.scratch + p.cl.expert_off);
    int* mb_e = reinterpret_cast<int*>(p.scratch + p.cl.mblock_expert);
    int* mb_v = reinterpret_cast<int*>(p.scratch + p.cl.mblock_valid);
    for (int le = threadIdx.x; le < p.E_loc; le += blockDim.x) {
        const int e = p.rank * p.E_loc + le;
        const int t = tot[e], o = off[e];
        e_tot[le] = t;
        e_off[le] = o;
        if (p.stats) p.stats[le] += t;
        for (int m = 0; m * MM_BLOCK_M < t; ++m) {
            mb_e[o / MM_BLOCK_M + m] = le;
            mb_v[o / MM_BLOCK_M + m] = min(MM_BLOCK_M, t - m * MM_BLOCK_M);
        }
    }
}

// ---- 4. slot assignment + push -----------------------------------------------------------------------------------
// grid = route_blocks, block = MM_DISPATCH_THREADS.  Thread i < CHUNK owns route b*CHUNK+i; its pool row on the owner is
//   dest_base[e] + (rows of earlier blocks for e) + (earlier routes of this block with the same e).
// Then all warps of the block copy the chunk's rows (H bytes of fp8 + 16 bytes of metadata) to the owners' pools.
constexpr int MM_DISPATCH_THREADS = 1024;
__global__ void __launch_bounds__(MM_DISPATCH_THREADS) dispatch_kernel(RouteParams p) {
    __shared__ int s_e[MM_ROUTE_CHUNK];
    __shared__ int s_row[MM_ROUTE_CHUNK];
    if (call_failed(p.scratch, p.cl)) return;
    const int n_routes = route_num_tokens(p) * p.K;
    const int route = blockIdx.x * MM_ROUTE_CHUNK + threadIdx.x;
    const bool owner_thread = threadIdx.x < MM_ROUTE_CHUNK;
    int e = -1;
    float w = 0.0f;
    if (owner_thread && route < n_routes) {
        const int64_t e64 = reinterpret_cast<const int64_t*>(p.sym + p.sl.topk_idx)[route];
        w = reinterpret_cast<const float*>(p.sym + p.sl.topk_weights)[route];
        if (e64 >= 0 && e64 < p.E && w != 0.0f) e = static_cast<int>(e64);
    }
    if (owner_thread) s_e[threadIdx.x] = e;
    __syncthreads();
    int row = -1;
    if (owner_thread && e >= 0) {
        int within = 0;
        for (int j = 0; j < static_cast<int>(threadIdx.x); ++j) within += (s_e[j] == e);
        const int* bc = reinterpret_cast<const int*>(p.scratch + p.cl.block_counts) + static_cast<int64_t>(blockIdx.x) * p.E;
        row = reinterpret_cast<const int*>(p.scratch + p.cl.dest_base)[e] + bc[e] + within;
        if (row >= p.sl.pool_rows) row = -1;   // cannot happen with worst-case sizing; never write out of bounds
    }
    if (owner_thread) {
        s_row[threadIdx.x] = row;
        if (route < n_routes) reinterpret_cast<int*>(p.scratch + p.cl.dest_row)[route] = row;
    }
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint8_t* x = p.sym + p.sl.x;
    const float* x_sf = reinterpret_cast<const float*>(p.sym + p.sl.x_sf);
    const float* tw = reinterpret_cast<const float*>(p.sym + p.sl.topk_weights);
    constexpr int kWarps = MM_DISPATCH_THREADS / 32;
    for (int li = warp; li < MM_ROUTE_CHUNK; li += kWarps) {
        const int r_row = s_row[li];
        if (r_row < 0) continue;
        const int r_e = s_e[li];
        const int r_route = blockIdx.x * MM_ROUTE_CHUNK + li;
        const int token = r_route / p.K, slot = r_route - token * p.K;
        uint8_t* peer = reinterpret_cast<uint8_t*>(p.peers[r_e / p.E_loc]);
        const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(token) * p.H);
        uint4* dst = reinterpret_cast<uint4*>(peer + p.sl.pool_x + static_cast<int64_t>(r_row) * p.H);
        const int nvec = p.H / 16;
        for (int v0 = 0; v0 < nvec; v0 += 32 * 8) {     // up to eight independent 16-byte loads in flight per lane
            uint4 buf[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int v = v0 + i * 32 + lane;
                if (v < nvec) buf[i] = __ldg(src + v);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int v = v0 + i * 32 + lane;
                if (v < nvec) dst[v] = buf[i];
            }
        }
        if (lane == 0) {
            MmPoolMeta m;
            m.x_scale = x_sf[token];
            m.route_weight = tw[r_route];
            m.src_token = token;
            m.src_info = (p.rank << 8) | slot;
            *reinterpret_cast<uint4*>(peer + p.sl.pool_meta + static_cast<int64_t>(r_row) * sizeof(MmPoolMeta)) =
                *reinterpret_cast<uint4*>(&m);
        }
    }
}

// ---- 4'. slot assignment + send list, no data movement (the layer kernel's helper warps push the rows) ------------
// grid = route_blocks, block = MM_ROUTE_CHUNK.  Thread i owns route b*CHUNK+i.  Besides the pool row on the owner
// (as in dispatch_kernel) it computes the route's position in this rank's send order and records
// {route, row, owner rank, token} there, so a pushing warp needs one load per row to know what to copy where.
__global__ void __launch_bounds__(MM_ROUTE_CHUNK) send_plan_kernel(RouteParams p) {
    __shared__ int s_e[MM_ROUTE_CHUNK];
    if (call_failed(p.scratch, p.cl)) return;
    const int n_routes = route_num_tokens(p) * p.K;
    const int route = blockIdx.x * MM_ROUTE_CHUNK + threadIdx.x;
    int e = -1;
    if (route < n_routes) {
        const int64_t e64 = reinterpret_cast<const int64_t*>(p.sym + p.sl.topk_idx)[route];
        const float w = reinterpret_cast<const float*>(p.sym + p.sl.topk_weights)[route];
        if (e64 >= 0 && e64 < p.E && w != 0.0f) e = static_cast<int>(e64);
    }
    s_e[threadIdx.x] = e;
    __syncthreads();
    int row = -1;
    if (e >= 0) {
        int within = 0;
        for (int j = 0; j < static_cast<int>(threadIdx.x); ++j) within += (s_e[j] == e);
        const int earlier = reinterpret_cast<const int*>(p.scratch + p.cl.block_counts)[static_cast<int64_t>(blockIdx.x) * p.E + e] + within;
        row = reinterpret_cast<const int*>(p.scratch + p.cl.dest_base)[e] + earlier;
        if (row >= p.sl.pool_rows) row = -1;   // cannot happen with worst-case sizing; never write out of bounds
        const int pos = reinterpret_cast<const int*>(p.scratch + p.cl.send_base)[e] + earlier;
        if (pos >= 0 && pos < p.T * p.K)
            reinterpret_cast<int4*>(p.scratch + p.cl.send_list)[pos] = make_int4(route, row, e / p.E_loc, route / p.K);
    }
    if (route < n_routes) reinterpret_cast<int*>(p.scratch + p.cl.dest_row)[route] = row;
}

// ---- cross-rank barrier as a kernel of its own (staged path) ---------------------------------------------------
// grid = 1, block = 32: publish the call epoch on barrier `bar` of every rank, then wait for all ranks.
__global__ void rank_barrier_kernel(RouteParams p, int bar) {
    // after a failure this rank stays silent: its peers' own bounded waits expire and each of them records a status
    if (call_failed(p.scratch, p.cl)) return;
    const int epoch = reinterpret_cast<const int*>(p.scratch + p.cl.epoch)[0];
    __threadfence_system();
    if (threadIdx.x < p.R) {
        int* sig = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(p.peers[threadIdx.x]) + p.sl.signals);
        st_release_sys(sig + bar * MM_MAX_RANKS + p.rank, epoch);
    }
    wait_rank_signals(p, bar, epoch);
}

}  // namespace mm
