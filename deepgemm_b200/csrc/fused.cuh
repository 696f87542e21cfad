// The layer's compute phase -- and, in MM_MODE_FUSED, the whole layer -- as ONE persistent, warp-specialised kernel.
//
// Replaces mega_moe_multirank_persistent_w8a8_channelwise_kernel
// (deep_gemm/include/deep_gemm/impls/mega_moe_dcu.cuh:259-765).  One CTA per SM; the CTAs wait on one another, so all of
// them have to be resident: the host launches it cooperatively (or, on request, as exactly as many CTAs as SMs after an
// occupancy check: a second CTA cannot share an SM with 226 KiB of shared memory).  Warp roles of a CTA (384 threads):
//   warp 0      TMA producer: streams weight tiles and pool / activation tiles into the operand ring;
//   warp 1      MMA issuer: tcgen05.mma into two TMEM accumulators;
//   warps 2-3   helpers: (a) push routed rows to the owners' receive pools over NVLink, (b) requantise finished m-blocks;
//   warps 4-11  epilogue: TMEM -> scales / SwiGLU -> global memory (GEMM2: straight into the source rank's combine buffer).
//
// Two entry modes.
//   gemm_only = 0 (MM_MODE_FUSED, small token counts, one launch per layer call):
//     1. every CTA histograms ALL of this rank's routes in shared memory and counts those before its own contiguous
//        share; CTA 0 publishes the count vector to all ranks;
//     2. bounded wait for all ranks' count vectors; every CTA derives the plan (totals, pool offsets, m-block table);
//     3. all warps push the CTA's share of the rows (row = base of the expert + routes before the share + rank inside
//        the share) and bump the owner's per-m-block arrival counters;
//     4. the tile loop below;  5. grid barrier, cross-rank "combine stores done" barrier;  6. top-k reduce;  7. clean-up.
//   gemm_only = 1 (MM_MODE_STAGED, any token count): the routing kernels of route.cuh made the plan, the destination row
//     of every route and a SEND LIST (this rank's valid routes ordered by local expert index, then owner); the kernel
//     runs step 4 only, and its helper warps first walk the send list -- so all ranks fill expert 0 of every owner first,
//     then expert 1, ... and an owner's GEMM1 tiles start as soon as their m-block has arrived, while later experts'
//     rows are still crossing NVLink.  The combine barrier, the reduce and the counter reset are launches after it.
//
// Step 4, the tile loop: m-blocks are grouped in waves; with G1(k) / G2(k) = all GEMM1 / GEMM2 tiles of wave k the
// order is  G1(0), G1(1), G1(2), {G1(3), G2(0)}, {G1(4), G2(1)}, ..., G2(n-1), the two lists of a {group} alternating tile
// by tile, and CTAs take tiles from this order dynamically: tensor-bound GEMM1 work overlaps the NVLink-bound combine
// stores of GEMM2 on every SM all the time.  Dependencies are per m-block, never global barriers:
//   - GEMM1 tile: weights start streaming at once; the token operand waits for arrive[m-block] == valid rows; each
//     epilogue warp counts its stored share in l1_done[m-block];
//   - requantisation unit (a quarter of an m-block's rows, claimed in order by the helper warps of ALL CTAs): waits for
//     every GEMM1 tile of the m-block (the channelwise scale needs the whole row), converts bf16 -> e4m3, bumps l2_ready;
//   - GEMM2 tile: the activation operand waits for l2_ready[m-block] == 4.
// A tile only ever waits for work that belongs to tiles earlier in the order (or for pushes, which wait for nothing),
// every role walks its items in order and all CTAs become resident, so the waits cannot form a cycle.  Every wait is
// bounded and ends in a status code, never in a hang.
#pragma once
#include "gemm.cuh"
#include "misc.cuh"
#include "route.cuh"

namespace mm {

constexpr int kHelperWarps = 2;
constexpr int kFusedFirstEpilogueWarp = 2 + kHelperWarps;                    // a multiple of 4: warp & 3 == TMEM lane quarter
constexpr int kFusedThreads = (kFusedFirstEpilogueWarp + kEpilogueWarps) * 32;
constexpr int kPushChunk = 8;             // rows a helper warp claims, pushes and signals at a time
constexpr int kPushChunkStart = 2;        // ... at kernel start, when every warp of the grid pushes at once: small chunks let the
                                          // first m-blocks complete (and the first GEMM1 tiles start) several microseconds earlier
static_assert(kFusedFirstEpilogueWarp % 4 == 0, "epilogue warps must start at a multiple of four");

// words of the `plan` array in the scratch buffer (written by route_plan_kernel or by this kernel's step 2)
enum { MM_PLAN_MBLOCKS = 0, MM_PLAN_ROWS_PADDED = 1, MM_PLAN_PAIRS = 2, MM_PLAN_SEND = 3, MM_PLAN_ROWS_EXPECTED = 6 };
// words of the `grid_sync` array: all zero between calls (this kernel's last step, or a memset after a gemm_only launch)
enum { MM_SYNC_CTAS = 0, MM_SYNC_CALLS = 1, MM_SYNC_UNITS_DONE = 2, MM_SYNC_PUSH_HEAD = 3, MM_SYNC_REQUANT_HEAD = 4, MM_SYNC_TILE_HEAD = 5 };

struct FusedParams {
    RouteParams rp;
    GemmParams g1, g2;
    __nv_bfloat16* y;
    int* plan;             // [8] see MM_PLAN_*
    int* l1_done;          // [m-blocks] epilogue warps that stored their share of a GEMM1 tile of the m-block
    int* l2_ready;         // [m-blocks] requantised quarters of the m-block
    int* grid_sync;        // [8] see MM_SYNC_*
    const int4* send_list; // [valid routes] {route, pool row, owner rank, token} in send order (gemm_only)
    uint8_t* act_fp8;      // [pool_rows][I]
    float* act_scale_w;    // writable alias of g2.act_scale
    const uint8_t* w1_tiled;   // GEMM1 weights as stored (the tensor map's base): L2 prefetch while the routing steps run
    int wave_mblocks;      // m-blocks per wave of the tile order
    int gemm_only;         // 1: routing was done by the staged kernels; start at the tile loop and stop after it
    int policy;            // tuning switches: bit 0 = both helper warps push (default: one pushes, one requantises from the start),
                           //                  bit 1 = epilogue warps help pushing until their first accumulator is complete
    long long* trace;      // tuning aid, normally null: per-tile cycle stamps of one CTA, kTraceWords words per tile (see TraceSlot)
    int trace_cta, trace_tiles;
};

// Per-tile cycle stamps (clock64 of the traced CTA's SM) written by the three roles of that CTA; word 0 = tile | kind << 32.
enum TraceSlot { TR_TILE = 0, TR_PROD_BEGIN, TR_PROD_DEP, TR_PROD_END, TR_MMA_BEGIN, TR_MMA_FIRST, TR_MMA_END, TR_EPI_BEGIN, TR_EPI_FULL,
                 TR_EPI_END, kTraceWords = 12 };

// shared-memory scratch of the routing steps, aliased onto the (not yet used) operand ring
struct FusedRouteSmem {
    int hist[MM_MAX_EXPERTS];        // this rank's valid routes per expert
    int before[MM_MAX_EXPERTS];      // ... of them, routes that come before this CTA's share (then: running count inside it)
    int tot[MM_MAX_EXPERTS];         // rows received by each expert (all ranks)
    int dest[MM_MAX_EXPERTS];        // first pool row on the owner for this rank's routes to the expert
    int off[MM_MAX_EXPERTS];         // pool offset of the expert on its owner
};
static_assert(sizeof(FusedRouteSmem) <= kStages * kStageBytes, "routing scratch must fit in the operand ring");

// Spin (bounded) until *flag - target >= 0.  `sys` selects system scope (flag written by another GPU).
// Gives up when the time budget is spent or another wait of the grid already failed (status code set).
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int target, bool sys, const int* status_code, uint64_t timeout_ns,
                                             int* observed, unsigned sleep_ns = 40) {
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
        __nanosleep(sleep_ns);
    }
}

// Ordering of pushed rows before their arrival signal, and the signal itself.  With one rank nothing leaves the GPU, so GPU
// scope is enough -- and it matters: a system-scope fence also waits for PCIe traffic, so with host<->device copies running
// in other streams (a serving loop that uploads the next batch while this one computes) it takes several times longer.
__device__ __forceinline__ void fence_rows_pushed(bool multi_rank) {
    if (multi_rank) __threadfence_system(); else __threadfence();
}
__device__ __forceinline__ void signal_row_arrived(int* counter, bool multi_rank) {
    if (multi_rank) asm volatile("red.relaxed.sys.global.add.s32 [%0], 1;" ::"l"(counter) : "memory");
    else asm volatile("red.relaxed.gpu.global.add.s32 [%0], 1;" ::"l"(counter) : "memory");
}
__device__ __forceinline__ int load_arrivals(const int* counter, bool multi_rank) {
    return multi_rank ? ld_acquire_sys(counter) : ld_acquire_gpu(counter);
}

// Position of a tile index in the tile order.  A CTA's tile indices grow, so seek() only moves forward.
// Groups: G1(0) .. G1(L-1) alone, then for k = 0, 1, ... the group {G1(k+L), G2(k)} whose tiles ALTERNATE one by one (the
// longer list's surplus follows), L = kWaveLookahead: a wave's requantisation has L waves of GEMM1 tiles to finish before
// its GEMM2 tiles come up, and at any moment the SMs are a steady mix of tensor-bound GEMM1 tiles and GEMM2 tiles whose
// epilogues write over NVLink -- instead of all SMs bursting onto the link at once.
constexpr int kWaveLookahead = 3;
struct WaveOrder {
    enum { kG1 = 0, kG2 = 1 };
    int n_waves, wave_m, num_mblocks, nb1, nb2;
    int g, base, size, n1, n2, w1, w2;          // current group: n1 GEMM1 tiles of wave w1, n2 GEMM2 tiles of wave w2
    bool tile_interleave;                       // false: inside a group all GEMM1 tiles come before the GEMM2 tiles
    __host__ __device__ WaveOrder(int num_mblocks_, int wave_m_, int nb1_, int nb2_, bool tile_interleave_)
        : n_waves((num_mblocks_ + wave_m_ - 1) / wave_m_), wave_m(wave_m_), num_mblocks(num_mblocks_), nb1(nb1_), nb2(nb2_),
          g(0), base(0), tile_interleave(tile_interleave_) { set(); }
    __host__ __device__ __forceinline__ int wave_mblocks(int w) const {
        if (w >= n_waves) return 0;
        const int left = num_mblocks - w * wave_m;
        return left < wave_m ? left : wave_m;
    }
    __host__ __device__ __forceinline__ void set() {
        w1 = g;
        w2 = g - kWaveLookahead;
        n1 = wave_mblocks(w1) * nb1;
        n2 = w2 >= 0 ? wave_mblocks(w2) * nb2 : 0;
        size = n1 + n2;
    }
    // tile -> (kind, m-block, n-block); the caller guarantees tile < num_mblocks * (nb1 + nb2)
    __host__ __device__ __forceinline__ void seek(int tile, int& kind_out, int& mb, int& nb) {
        while (tile >= base + size) { base += size; ++g; set(); }
        const int r = tile - base;
        const int m = tile_interleave ? (n1 < n2 ? n1 : n2) : 0;
        int idx;
        if (r < 2 * m) { kind_out = (r & 1) ? kG2 : kG1; idx = r >> 1; }
        else if (tile_interleave) { kind_out = n1 > n2 ? kG1 : kG2; idx = r - m; }
        else { kind_out = r < n1 ? kG1 : kG2; idx = r < n1 ? r : r - n1; }
        const int per = kind_out == kG1 ? nb1 : nb2;
        mb = (kind_out == kG1 ? w1 : w2) * wave_m + idx / per;
        nb = idx - (idx / per) * per;
    }
};

// Tiles are handed out dynamically: the producer thread of a CTA claims the next tile index from a global counter (one
// claim ahead, so the atomic's latency is hidden), and publishes it to the CTA's other roles through a small ring in shared
// memory: slot j % 8 holds {j, tile} for the CTA's j-th tile, tile < 0 = no more tiles.  The producer is never more than
// three tiles ahead of the epilogue (two accumulators, four operand stages), so eight slots cannot wrap onto a live one.
constexpr int kTileRing = 8;
__device__ __forceinline__ void ring_publish(volatile int* ring, int j, int tile) {
    ring[2 * (j & (kTileRing - 1)) + 1] = tile;
    __threadfence_block();
    ring[2 * (j & (kTileRing - 1))] = j;
}
// the j-th tile of this CTA once the producer has published it; kRingAbort when the CTA gave up or the wait ran out
constexpr int kRingAbort = -2;
__device__ __forceinline__ int ring_wait(const volatile int* ring, int j, volatile int* abort_flag, uint64_t timeout_ns) {
    const volatile int* slot = ring + 2 * (j & (kTileRing - 1));
    if (slot[0] != j) {
        const uint64_t t0 = global_timer_ns();
        uint32_t it = 0;
        while (slot[0] != j) {
            if ((++it & 63u) == 0u) {
                if (*abort_flag != 0) return kRingAbort;
                if (global_timer_ns() - t0 > timeout_ns) { *abort_flag = 1; return kRingAbort; }
            }
        }
    }
    __threadfence_block();
    return slot[1];
}

// Copy up to two FP8 rows of `H` bytes (16-byte vectors, all their loads in flight together) -- the data part of a push.
__device__ __forceinline__ void push_two_rows(const uint8_t* src0, uint8_t* dst0, const uint8_t* src1, uint8_t* dst1, int H, int lane) {
    const int nvec = H / 16;
    for (int v0 = 0; v0 < nvec; v0 += 32 * 8) {
        uint4 a[8], b[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int v = v0 + k * 32 + lane;
            if (v < nvec) {
                a[k] = __ldg(reinterpret_cast<const uint4*>(src0) + v);
                if (src1) b[k] = __ldg(reinterpret_cast<const uint4*>(src1) + v);
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int v = v0 + k * 32 + lane;
            if (v < nvec) {
                reinterpret_cast<uint4*>(dst0)[v] = a[k];
                if (src1) reinterpret_cast<uint4*>(dst1)[v] = b[k];
            }
        }
    }
}

// One chunk of the send list (helper warps, gemm_only): copy up to kPushChunk rows into their owners' receive pools, write
// their metadata, then -- warp barrier, one system-scope fence -- count one arrival per row on the owner (per m-block and
// in total).
__device__ __forceinline__ void push_chunk(const FusedParams& fp, int j0, int chunk, int n_send, int lane) {
    const RouteParams& rp = fp.rp;
    const float* tw = reinterpret_cast<const float*>(rp.sym + rp.sl.topk_weights);
    const float* x_sf = reinterpret_cast<const float*>(rp.sym + rp.sl.x_sf);
    const uint8_t* x = rp.sym + rp.sl.x;
    const int arrive_total_slot = static_cast<int>(rp.sl.pool_rows / MM_BLOCK_M);
    const int n = min(chunk, n_send - j0);
    // lane j < n describes row j of the chunk
    int route = -1, row = -1, owner = 0, token = 0;
    if (lane < n) {
        const int4 rec = __ldcg(fp.send_list + j0 + lane);
        route = rec.x; row = rec.y; owner = rec.z; token = rec.w;
        if (row < 0 || owner < 0 || owner >= rp.R || token < 0 || token >= rp.T) row = -1;
    }
    for (int j = 0; j < n; j += 2) {
        const int row0 = __shfl_sync(0xffffffffu, row, j), tok0 = __shfl_sync(0xffffffffu, token, j);
        const int own0 = __shfl_sync(0xffffffffu, owner, j);
        const int row1 = __shfl_sync(0xffffffffu, row, j + 1), tok1 = __shfl_sync(0xffffffffu, token, j + 1);
        const int own1 = __shfl_sync(0xffffffffu, owner, j + 1);
        const bool has0 = row0 >= 0, has1 = j + 1 < n && row1 >= 0;
        const uint8_t* s0 = x + static_cast<int64_t>(tok0) * rp.H;
        uint8_t* d0 = reinterpret_cast<uint8_t*>(rp.peers[own0]) + rp.sl.pool_x + static_cast<int64_t>(row0) * rp.H;
        const uint8_t* s1 = x + static_cast<int64_t>(tok1) * rp.H;
        uint8_t* d1 = reinterpret_cast<uint8_t*>(rp.peers[own1]) + rp.sl.pool_x + static_cast<int64_t>(row1) * rp.H;
        if (has0) push_two_rows(s0, d0, has1 ? s1 : nullptr, d1, rp.H, lane);
        else if (has1) push_two_rows(s1, d1, nullptr, nullptr, rp.H, lane);
    }
    if (row >= 0) {
        MmPoolMeta m;
        m.x_scale = x_sf[token];
        m.route_weight = tw[route];
        m.src_token = token;
        m.src_info = (rp.rank << 8) | (route - token * rp.K);
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(rp.peers[owner]) + rp.sl.pool_meta +
                                  static_cast<int64_t>(row) * sizeof(MmPoolMeta)) = *reinterpret_cast<uint4*>(&m);
    }
    __syncwarp();
    fence_rows_pushed(rp.R > 1);
    if (row >= 0) {
        int* arr = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(rp.peers[owner]) + rp.sl.pool_arrive);
        signal_row_arrived(arr + row / MM_BLOCK_M, rp.R > 1);
        signal_row_arrived(arr + arrive_total_slot, rp.R > 1);
    }
}

// One requantisation unit (helper warps): a quarter of the row pairs of m-block mb, bf16 -> e4m3 with one scale per row,
// s2 = max(amax / 448, 1e-4) (deep_gemm/include/deep_gemm/impls/mega_moe_dcu_tiles.cuh:672-733), then count the quarter
// towards l2_ready[mb].  The caller has seen, with an acquire load, that every GEMM1 tile of the m-block is stored.
__device__ __forceinline__ void requant_unit(const FusedParams& fp, int u, int lane) {
    const GemmParams& g1 = fp.g1;
    const int inter = g1.n_out, vecs = inter / 8;
    // the four units of an m-block take its row pairs in turn (pairs 0, 4, 8, ... / 1, 5, 9, ... / ...), so a block with few
    // valid rows (decode) is still spread over four warps
    const int mb = u >> 2;
    const int r_hi = g1.mblock_valid[mb];
    for (int r = 2 * (u & 3); r < r_hi; r += 8) {
        uint4 buf[2][8];
        float inv[2], sc2[2];
#pragma unroll
        for (int u2 = 0; u2 < 2; ++u2) {
            const int64_t prow = static_cast<int64_t>(mb) * kBlockM + min(r + u2, r_hi - 1);
            const float amax = __uint_as_float(__ldcg(g1.row_amax + prow));
            sc2[u2] = fmaxf(__fdiv_rn(amax, 448.0f), 1.0e-4f);
            inv[u2] = __fdiv_rn(1.0f, sc2[u2]);
            const uint4* src = reinterpret_cast<const uint4*>(g1.act_bf16 + prow * inter);
#pragma unroll
            for (int k = 0; k < 8; ++k) { const int v = k * 32 + lane; if (v < vecs) buf[u2][k] = __ldcg(src + v); }
        }
#pragma unroll
        for (int u2 = 0; u2 < 2; ++u2) {
            if (r + u2 >= r_hi) continue;
            const int64_t prow = static_cast<int64_t>(mb) * kBlockM + r + u2;
            const uint4* src = reinterpret_cast<const uint4*>(g1.act_bf16 + prow * inter);
            uint2* dst = reinterpret_cast<uint2*>(fp.act_fp8 + prow * inter);
            for (int v0 = 0; v0 < vecs; v0 += 32 * 8) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int v = v0 + k * 32 + lane;
                    if (v < vecs) {
                        const uint4 d = (v0 == 0) ? buf[u2][k] : __ldcg(src + v);
                        uint2 o;
                        o.x = pack4_e4m3(bf16_lo(d.x) * inv[u2], bf16_hi(d.x) * inv[u2], bf16_lo(d.y) * inv[u2], bf16_hi(d.y) * inv[u2]);
                        o.y = pack4_e4m3(bf16_lo(d.z) * inv[u2], bf16_hi(d.z) * inv[u2], bf16_lo(d.w) * inv[u2], bf16_hi(d.w) * inv[u2]);
                        dst[v] = o;
                    }
                }
            }
            if (lane == 0) { fp.act_scale_w[prow] = sc2[u2]; g1.row_amax[prow] = 0u; }
        }
    }
    __syncwarp();
    if (lane == 0) {
        __threadfence();
        red_release_gpu_add(fp.l2_ready + mb, 1);     // GEMM2 producers wait for 4
        red_release_gpu_add(fp.grid_sync + MM_SYNC_UNITS_DONE, 1);
    }
}

__global__ void __launch_bounds__(kFusedThreads, 1)
mega_moe_fused_kernel(const __grid_constant__ CUtensorMap tm_pool, const __grid_constant__ CUtensorMap tm_w1,
                      const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_w2,
                      const __grid_constant__ FusedParams fp) {
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
    int* s_misc = reinterpret_cast<int*>(tail + 16);       // [0] number of m-blocks, [1] ok flag of block-wide waits, [2] rows to receive,
                                                           // [4] leading tiles of this CTA whose dependency the scout has confirmed
    volatile int* tile_ring = reinterpret_cast<volatile int*>(tail + 48);   // kTileRing x {sequence number, tile}
    FusedRouteSmem& rs = *reinterpret_cast<FusedRouteSmem*>(smem_gen);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tid = threadIdx.x, nthr = blockDim.x;
    // timeline of CTA 0 (tenths of a microsecond since kernel entry) in the spare status words, for tuning:
    // [5] plan ready, [6] rows pushed, [7] producer done, [8] MMA done, [9] epilogue done, [10] all ranks done, [11] reduced,
    // [12] helper pushes done, [13] helper requantisation done, [14] / [15] producer's own polling for GEMM1 arrivals / GEMM2 requantisation
    const uint64_t t_entry = global_timer_ns();
    auto stamp = [&](int slot) { if (blockIdx.x == 0) status[slot] = static_cast<int>((global_timer_ns() - t_entry) / 100); };
    const bool traced = fp.trace != nullptr && static_cast<int>(blockIdx.x) == fp.trace_cta;
    auto trace = [&](int j, int slot, long long v) { if (traced && j < fp.trace_tiles) fp.trace[j * kTraceWords + slot] = v; };

    // ------------------------------------------------------------------ phase 0: barriers, TMEM, call identity
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), kEpilogueWarps); }
        *abort_flag = 0;
        s_misc[0] = 0; s_misc[1] = ld_acquire_gpu(status) == 0 ? 1 : 0; s_misc[2] = 0; s_misc[4] = 0;
        for (int i = 0; i < kTileRing; ++i) tile_ring[2 * i] = -1;
        fence_barrier_init();
        prefetch_tensormap(&tm_pool); prefetch_tensormap(&tm_w1); prefetch_tensormap(&tm_act); prefetch_tensormap(&tm_w2);
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    // the epoch words are only rewritten at the very end of the kernel, after every CTA has passed the grid barrier
    const int epoch = reinterpret_cast<const int*>(rp.scratch + rp.cl.epoch)[0] + (fp.gemm_only ? 0 : 1);
    const int fused_calls = fp.grid_sync[1];
    const int n_tokens = route_num_tokens(rp);
    const int n_routes = n_tokens * rp.K;
    for (int e = tid; e < rp.E; e += nthr) { rs.hist[e] = 0; rs.before[e] = 0; }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int arrive_total_slot = static_cast<int>(rp.sl.pool_rows / MM_BLOCK_M);   // last word of the arrival array

    if (!fp.gemm_only) {
    // While the routing steps below run (some 20 us of dependent round trips), start pulling the weights of the first GEMM1
    // tiles into L2.  Which expert a tile belongs to is not known yet; with few tokens (the regime of this mode) every local
    // expert that has rows has ONE m-block, so tile t most likely is expert t / nb1 -- a wrong guess only costs L2 traffic.
    if (tid == 0) {
        const int nb1_ = fp.g1.n_blocks, kb_ = fp.g1.kdim / kBlockK;
        for (int t = blockIdx.x; t < 96; t += gridDim.x) {          // 96 tiles of 1 MiB: what L2 can hold on to until they are used
            const int e = t / nb1_;
            if (e >= rp.E_loc) break;
            const uint8_t* wt = fp.w1_tiled + static_cast<int64_t>(t) * kb_ * kBBytes;     // tile t of [expert][n block][k block][256][128]
            for (int kb = 0; kb < kb_; ++kb)
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(wt + static_cast<int64_t>(kb) * kBBytes), "r"(kBBytes) : "memory");
        }
    }
    // ------------------------------------------------------------------ phase 1: local histogram, publish counts
    // This CTA pushes the contiguous share [lo, hi) of the rank's routes; `before` counts, per expert, the valid routes
    // in front of the share, so the CTA can number its routes without talking to the other CTAs.
    const int per_cta = (n_routes + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    const int lo = min(static_cast<int>(blockIdx.x) * per_cta, n_routes), hi = min(lo + per_cta, n_routes);
    const int64_t* idx = reinterpret_cast<const int64_t*>(rp.sym + rp.sl.topk_idx);
    const float* tw = reinterpret_cast<const float*>(rp.sym + rp.sl.topk_weights);
    for (int i = tid; i < n_routes; i += nthr) {
        const int64_t e64 = idx[i];
        if (e64 >= 0 && e64 < rp.E && tw[i] != 0.0f) {
            atomicAdd(&rs.hist[static_cast<int>(e64)], 1);
            if (i < lo) atomicAdd(&rs.before[static_cast<int>(e64)], 1);
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
    if (tid < rp.R && s_misc[1]) {
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
            fp.plan[MM_PLAN_MBLOCKS] = run / MM_BLOCK_M;   // every CTA writes the same values
            fp.plan[MM_PLAN_ROWS_PADDED] = run;
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
    __threadfence();
    __syncthreads();
    if (tid == 0) stamp(5);

    // ------------------------------------------------------------------ phase 3: push this CTA's share of the rows
    if (s_misc[1]) {
        int* dest_row = reinterpret_cast<int*>(rp.scratch + rp.cl.dest_row);
        // 3a. one warp numbers the share's routes in route order: a route's pool row on the owner is the expert's base for
        //     this rank + the rank's earlier routes to that expert (those before the share, then those inside it).
        if (warp == 0) {
            for (int i0 = lo; i0 < hi; i0 += 32) {
                const int i = i0 + lane;
                int e = -1;
                if (i < hi) {
                    const int64_t e64 = idx[i];
                    if (e64 >= 0 && e64 < rp.E && tw[i] != 0.0f) e = static_cast<int>(e64);
                }
                const unsigned same = __match_any_sync(0xffffffffu, e);
                const int ahead = __popc(same & ((1u << lane) - 1u));
                int row = -1;
                if (e >= 0) row = rs.dest[e] + rs.before[e] + ahead;
                __syncwarp();
                if (e >= 0 && ahead == 0) rs.before[e] += __popc(same);
                __syncwarp();
                if (row >= rp.sl.pool_rows) row = -1;          // cannot happen with worst-case sizing; never write out of bounds
                if (i < hi) dest_row[i] = row;
            }
        }
        __syncthreads();
        // 3b. all warps copy rows (H bytes of fp8 + 16 bytes of metadata each) into the owners' pools
        const uint8_t* x = rp.sym + rp.sl.x;
        const float* x_sf = reinterpret_cast<const float*>(rp.sym + rp.sl.x_sf);
        const int warps_per_cta = nthr >> 5;
        for (int i = lo + warp; i < hi; i += warps_per_cta) {
            const int row = dest_row[i];
            if (row < 0) continue;
            const int e = static_cast<int>(idx[i]);
            const int token = i / rp.K, slot = i - token * rp.K;
            uint8_t* peer = reinterpret_cast<uint8_t*>(rp.peers[e / rp.E_loc]);
            push_two_rows(x + static_cast<int64_t>(token) * rp.H, peer + rp.sl.pool_x + static_cast<int64_t>(row) * rp.H, nullptr, nullptr,
                          rp.H, lane);
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
        fence_rows_pushed(rp.R > 1);
        for (int i0 = lo + warp; i0 < hi; i0 += 32 * warps_per_cta) {
            const int i = i0 + lane * warps_per_cta;
            if (i < hi) {
                const int row = dest_row[i];
                if (row >= 0) {
                    const int e = static_cast<int>(idx[i]);
                    int* arr = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(rp.peers[e / rp.E_loc]) + rp.sl.pool_arrive);
                    signal_row_arrived(arr + row / MM_BLOCK_M, rp.R > 1);
                    signal_row_arrived(arr + arrive_total_slot, rp.R > 1);
                }
            }
        }
    }
    } else if (tid == 0) {
        s_misc[0] = s_misc[1] ? fp.plan[MM_PLAN_MBLOCKS] : 0;      // the plan was made by route_plan_kernel
        s_misc[2] = fp.plan[MM_PLAN_ROWS_EXPECTED];
    }
    // the routing scratch is dead from here on; the operand ring (same shared memory) is written by TMA next
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) stamp(6);
    const int num_mblocks = s_misc[0];
    const bool healthy = s_misc[1] != 0;
    const int rows_expected = s_misc[2];

    // ------------------------------------------------------------------ phase 4: the tile loop
    const GemmParams& g1 = fp.g1;
    const GemmParams& g2 = fp.g2;
    const int nb1 = g1.n_blocks, nb2 = g2.n_blocks;
    const WaveOrder order_init(num_mblocks, max(1, fp.wave_mblocks), nb1, nb2, (fp.policy & 4) == 0);
    const int tiles_all = healthy ? num_mblocks * (nb1 + nb2) : 0;
    const int requant_units = healthy ? num_mblocks * 4 : 0;
    const int* arrive = reinterpret_cast<const int*>(rp.sym + rp.sl.pool_arrive);

    if (warp == 0) {
        // -------------------------------------------------------------- TMA producer (one thread)
        if (lane == 0) {
        int stage = 0; uint32_t phase = 0;
        bool alive = true;
        // once every row has arrived (every m-block is requantised) no further per-tile polling is needed
        bool all_arrived = false, all_ready = false;
        WaveOrder order = order_init;
        int local_i = -1;                                   // index of the tile in this CTA's sequence
        uint64_t polled_g1 = 0, polled_g2 = 0;              // time this thread itself spent polling for GEMM1 / GEMM2 tiles (tuning aid)
        int* tile_head = fp.grid_sync + MM_SYNC_TILE_HEAD;
        const bool static_tiles = (fp.policy & 8) != 0;      // measurement aid: round-robin assignment instead of claiming
        int tile = tiles_all > 0 ? (static_tiles ? static_cast<int>(blockIdx.x) : atomicAdd(tile_head, 1)) : tiles_all;
        for (; tile < tiles_all && alive;) {
            // claimed one ahead: needed only when this tile's loads are issued
            const int next_tile = static_tiles ? tile + static_cast<int>(gridDim.x) : atomicAdd(tile_head, 1);
            ++local_i;
            ring_publish(tile_ring, local_i, tile);
            int kind, mb, nb;
            order.seek(tile, kind, mb, nb);
            trace(local_i, TR_TILE, static_cast<long long>(tile) | (static_cast<long long>(kind) << 32));
            trace(local_i, TR_PROD_BEGIN, clock64());
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
                mbar_arrive_expect_tx(full_bar(stage), kStageBytes);
                tma_load_2d(a_dst + kABytes, tb, 0, (b_tile0 + kb) * kBlockN, full_bar(stage));   // weights first
                if (kb == 0) {
                    // The token operand of this m-block must be complete before TMA may read it.  Normally the scout (an
                    // epilogue lane that polls ahead while it waits for accumulators) has confirmed that already, and this
                    // thread, whose loads the tensor pipe is waiting for, only reads a shared-memory word; otherwise it polls.
                    const bool confirmed = local_i < *reinterpret_cast<volatile int*>(s_misc + 4);
                    if (!confirmed && !(second ? all_ready : all_arrived)) {
                        int seen = 0;
                        bool ok = true;
                        const uint64_t t_poll = global_timer_ns();
                        if (second) {
                            all_ready = ld_acquire_gpu(fp.grid_sync + MM_SYNC_UNITS_DONE) - requant_units >= 0;
                            if (!all_ready) ok = wait_flag_ge(fp.l2_ready + mb, 4, false, status, g.timeout_ns, &seen);
                        } else {
                            all_arrived = load_arrivals(arrive + arrive_total_slot, rp.R > 1) - rows_expected >= 0;
                            if (!all_arrived) ok = wait_flag_ge(arrive + mb, g.mblock_valid[mb], rp.R > 1, status, rp.barrier_timeout_ns, &seen);
                        }
                        if (second) polled_g2 += global_timer_ns() - t_poll; else polled_g1 += global_timer_ns() - t_poll;
                        if (!ok) {
                            report_status(rp.scratch, rp.cl, MM_ERR_GRID_BARRIER_TIMEOUT, second ? 2 : 1, mb, second ? 4 : g.mblock_valid[mb], seen);
                            *abort_flag = 1;
                            alive = false;
                        }
                    }
                    // rows were written with ordinary stores (by other SMs or GPUs) and their completion was observed with an
                    // acquire load (here, or by the scout, whose result came through shared memory): order all that before
                    // the TMA reads
                    __threadfence_block();
                    asm volatile("fence.proxy.async;" ::: "memory");
                    trace(local_i, TR_PROD_DEP, clock64());
                }
                // issue the token tile even on failure so that the stage's byte count completes and nobody is left waiting
                tma_load_2d(a_dst, ta, kb * kBlockK, mb * kBlockM, full_bar(stage));
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
                if (!alive) break;
            }
            trace(local_i, TR_PROD_END, clock64());
            tile = next_tile;
        }
        ring_publish(tile_ring, local_i + 1, -1);                // no more tiles for this CTA
        stamp(7);
        if (blockIdx.x == 0) { status[14] = static_cast<int>(polled_g1 / 100); status[15] = static_cast<int>(polled_g2 / 100); }
        }
        __syncwarp();
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer (one thread)
        if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_f8(kBlockM, kBlockN);
        int stage = 0; uint32_t phase = 0;
        int acc = 0; uint32_t acc_phase = 0;
        bool alive = true;
        WaveOrder order = order_init;
        for (int j = 0; alive; ++j) {
            const int tile = ring_wait(tile_ring, j, abort_flag, rp.barrier_timeout_ns);
            if (tile < 0) break;
            int kind, mb, nb;
            order.seek(tile, kind, mb, nb);
            const GemmParams& g = kind == WaveOrder::kG2 ? g2 : g1;
            const int k_blocks = g.kdim / kBlockK;
            trace(j, TR_MMA_BEGIN, clock64());
            if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, g.timeout_ns)) { alive = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * kBlockN;
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag, g.timeout_ns)) { alive = false; break; }
                tc_fence_after();
                if (kb == 0) trace(j, TR_MMA_FIRST, clock64());
                const uint32_t a_src = smem_base + stage * kStageBytes;
                const uint64_t da = umma_desc_k_sw128(a_src);
                const uint64_t db = umma_desc_k_sw128(a_src + kABytes);
#pragma unroll
                for (int k = 0; k < kBlockK / 32; ++k) umma_f8(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
                umma_commit(empty_bar(stage));
                if (kb == k_blocks - 1) umma_commit(tfull_bar(acc));
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            trace(j, TR_MMA_END, clock64());
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        stamp(8);
        }
        __syncwarp();
    } else if (warp < kFusedFirstEpilogueWarp) {
        // -------------------------------------------------------------- helpers
        // Two jobs:
        // (a) gemm_only: push this rank's rows in send-list order.  Chunks of the list are claimed with an atomic counter, so
        //     the helper warps of the whole grid walk it front to back together.  After a chunk's rows are written: warp
        //     barrier, one system-scope fence, then one arrival per row on the owner (per m-block and in total).
        // (b) requantisation units, claimed in m-block order by the helper warps of all CTAs: once every GEMM1 tile of the
        //     m-block is stored (each of the 8 epilogue warps of each of its nb1 tiles counts once), turn a quarter of its bf16 rows
        //     into e4m3 with one scale per row (deep_gemm/include/deep_gemm/impls/mega_moe_dcu_tiles.cuh:672-733) and count
        //     the quarter towards l2_ready[m-block].
        // Both loops are kept as simple as this on purpose: merged into one loop the compiler spills the row buffers and the
        // helper warps fall behind the tile loop (measured).
        const int n_send = (fp.gemm_only && healthy) ? fp.plan[MM_PLAN_SEND] : 0;
        const int l1_target = nb1 * kEpilogueWarps;

        int* requant_head = fp.grid_sync + MM_SYNC_REQUANT_HEAD;
        // (a) push: walk the send list until it is exhausted.  Only warp 2 of a CTA pushes (policy bit 0: both do), so that
        //     warp 3 requantises from the start and GEMM2 tiles never wait for the push to finish.
        const bool pusher = (fp.policy & 1) != 0 || warp == 2;
        for (int it = 0; pusher; ++it) {
            const int chunk = it < 2 ? kPushChunkStart : kPushChunk;
            int j0 = 0;
            if (lane == 0) j0 = atomicAdd(fp.grid_sync + MM_SYNC_PUSH_HEAD, chunk);
            j0 = __shfl_sync(0xffffffffu, j0, 0);
            if (j0 >= n_send) break;
            push_chunk(fp, j0, chunk, n_send, lane);
        }
        if (warp == 2 && lane == 0) stamp(12);
        // (b) requantisation: claim the units in order and wait for each
        while (true) {
            int u = 0;
            if (lane == 0) u = atomicAdd(requant_head, 1);
            u = __shfl_sync(0xffffffffu, u, 0);
            if (u >= requant_units) break;
            int ok = 1;
            if (lane == 0) {
                int seen = 0;
                if (!wait_flag_ge(fp.l1_done + (u >> 2), l1_target, false, status, g1.timeout_ns, &seen, 200)) {
                    report_status(rp.scratch, rp.cl, MM_ERR_GRID_BARRIER_TIMEOUT, 4, u >> 2, l1_target, seen);
                    ok = 0;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            requant_unit(fp, u, lane);
        }
        if (warp == 2 && lane == 0) stamp(13);
    } else {
        // -------------------------------------------------------------- epilogue (eight warps)
        const int ew = warp - kFusedFirstEpilogueWarp;
        const int q = warp & 3;                       // TMEM lane quarter this warp may read
        const int half = ew >> 2;                     // which half of the tile's output columns
        const int et = q * 32 + lane;
        uint8_t* my_staging = staging_gen + ew * kStagingWarpBytes;
        const bool do_clamp = g1.clamp < 3.0e38f;
        int acc = 0; uint32_t acc_phase = 0;
        bool alive = true;
        WaveOrder order = order_init;
        // Until this CTA's first accumulator is complete the epilogue warps have nothing to do: they help the helper warps
        // push rows (gemm_only), which gets most of a single GPU's rows into the pool within the first tile's time.
        if (fp.gemm_only && healthy && (fp.policy & 2)) {
            const int n_send = fp.plan[MM_PLAN_SEND];
            while (true) {
                int j0 = n_send;
                if (lane == 0 && !mbar_try_wait(tfull_bar(0), 0)) j0 = atomicAdd(fp.grid_sync + MM_SYNC_PUSH_HEAD, kPushChunkStart);
                j0 = __shfl_sync(0xffffffffu, j0, 0);
                if (j0 >= n_send) break;
                push_chunk(fp, j0, kPushChunkStart, n_send, lane);
            }
        }
        // Scout: one lane checks, without blocking, whether the dependencies of this CTA's NEXT tiles are met (arrival
        // counter of a GEMM1 tile's m-block, requantisation count of a GEMM2 tile's) and publishes how many leading tiles
        // are confirmed.  It polls while the epilogue waits for an accumulator, so the producer warp does not have to put a
        // global-memory round trip in front of every tile.  Counters only grow during a call: a confirmation stays valid.
        const bool is_scout = warp == kFusedFirstEpilogueWarp && lane == 0;
        WaveOrder scout_order = order_init;
        int scout_n = 0, scout_polls = 0;                    // tiles of this CTA confirmed so far (in ring order)
        bool scout_all_arrived = false, scout_all_ready = false;
        auto scout_step = [&](int j_epilogue) {
            if (scout_n < j_epilogue) scout_n = j_epilogue;   // tiles the epilogue has reached were loaded: nothing left to confirm
            for (int n = 0; n < 2; ++n) {
                const volatile int* slot = tile_ring + 2 * (scout_n & (kTileRing - 1));
                if (slot[0] != scout_n) break;                // not published yet
                __threadfence_block();
                const int t = slot[1];
                if (t < 0) break;
                int kind, mb, nb;
                scout_order.seek(t, kind, mb, nb);
                bool ok;
                if (kind == WaveOrder::kG2) {
                    if (!scout_all_ready && (scout_polls++ & 7) == 0) scout_all_ready = ld_acquire_gpu(fp.grid_sync + MM_SYNC_UNITS_DONE) - requant_units >= 0;
                    ok = scout_all_ready || ld_acquire_gpu(fp.l2_ready + mb) - 4 >= 0;
                } else {
                    if (!scout_all_arrived && (scout_polls++ & 7) == 0) scout_all_arrived = load_arrivals(arrive + arrive_total_slot, rp.R > 1) - rows_expected >= 0;
                    ok = scout_all_arrived || load_arrivals(arrive + mb, rp.R > 1) - g1.mblock_valid[mb] >= 0;
                }
                if (!ok) break;
                ++scout_n;
            }
            __threadfence_block();
            *reinterpret_cast<volatile int*>(s_misc + 4) = scout_n;
        };
        int pending_mb = -1;
        for (int local_i = 0; alive; ++local_i) {
            if (*abort_flag != 0) break;
            const int tile = ring_wait(tile_ring, local_i, abort_flag, rp.barrier_timeout_ns);
            if (tile < 0) break;
            int kind, mb, nb;
            order.seek(tile, kind, mb, nb);
            const bool second = kind == WaveOrder::kG2;
            const GemmParams& g = second ? g2 : g1;
            const int e = g.mblock_expert[mb];
            const int valid = g.mblock_valid[mb];
            const int row = mb * kBlockM + et;
            const bool row_ok = et < valid;
            float* sc = scales_gen + acc * kBlockN;
            {
                const int st = ew * 32 + lane;
                const float* ws = g.w_scale + static_cast<int64_t>(e) * g.w_rows_per_expert;
                if (!second) {
                    sc[st] = st < 128 ? ws[nb * 128 + st] : ws[g.w_rows_per_expert / 2 + nb * 128 + (st - 128)];
                } else {
                    const int c0 = nb * kBlockN + st;
                    sc[st] = c0 < g.n_out ? ws[c0] : 0.0f;
                }
            }
            named_bar_sync(1, kEpilogueThreads);
            if (is_scout) scout_step(local_i);
            __syncwarp();
            // Things done here cost nothing while the tensor pipe is the bottleneck (the accumulator is not complete yet):
            // count the previous GEMM1 tile's share towards its m-block (the fence waits for this warp's stores), and, if the
            // scout has confirmed this tile's dependency, fetch the row's metadata before the accumulator wait instead of after.
            if (pending_mb >= 0) {
                if (lane == 0) { __threadfence(); red_release_gpu_add(fp.l1_done + pending_mb, 1); }
                pending_mb = -1;
            }
            const bool early = local_i < *reinterpret_cast<volatile int*>(s_misc + 4);
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            float a_scale = 0.0f;
            if (early && row_ok) {
                __threadfence_block();
                raw = __ldcg(reinterpret_cast<const uint4*>(g.meta + row));
                if (second) a_scale = __ldcg(g.act_scale + row);
            }
            if (is_scout) trace(local_i, TR_EPI_BEGIN, clock64());
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, g.timeout_ns)) { alive = false; break; }
            tc_fence_after();
            if (is_scout) trace(local_i, TR_EPI_FULL, clock64());
            // the accumulator is complete, so the m-block's rows (and, for GEMM2, its activation scales) are in place
            float row_scale = 0.0f, route_w = 0.0f;
            uint8_t* out_ptr = nullptr;
            if (row_ok) {
                if (!early) {
                    raw = __ldcg(reinterpret_cast<const uint4*>(g.meta + row));
                    if (second) a_scale = __ldcg(g.act_scale + row);
                }
                if (!second) {
                    row_scale = __uint_as_float(raw.x);
                    route_w = __uint_as_float(raw.y);
                } else {
                    row_scale = a_scale;
                    out_ptr = combine_row_ptr(g, static_cast<int>(raw.w), static_cast<int>(raw.z));
                }
            }
            if (!second) epilogue_math<0>(g1, tmem_base, sc, my_staging, lane, q, half, acc, mb, nb, valid, row, row_ok, row_scale, route_w, out_ptr, do_clamp);
            else         epilogue_math<1>(g2, tmem_base, sc, my_staging, lane, q, half, acc, mb, nb, valid, row, row_ok, row_scale, route_w, out_ptr, do_clamp);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (is_scout) trace(local_i, TR_EPI_END, clock64());
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }

            // this warp's share of a GEMM1 tile (bf16 values, row amax) is stored: it is counted towards the m-block's total at
            // the next idle point (above), or right after the loop
            if (!second) pending_mb = mb;
        }
        if (pending_mb >= 0 && lane == 0) { __threadfence(); red_release_gpu_add(fp.l1_done + pending_mb, 1); }
    }

    fence_rows_pushed(rp.R > 1);      // the combine stores of this CTA's GEMM2 tiles, before anybody is told they are done
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
        // after a failure this rank stays silent: its peers' own bounded waits expire and each records a status
        if (tid < rp.R && ld_acquire_gpu(status) == 0) {
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
    if (ld_acquire_gpu(status) == 0) {      // after a failure y stays untouched
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
                        if (ok[j]) buf[j] = __ldcg(comb + (static_cast<int64_t>(t) * rp.K + s) * vecs + v);
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
        for (int i = blockIdx.x * nthr + tid; i < num_mblocks; i += gridDim.x * nthr) { arr[i] = 0; fp.l2_ready[i] = 0; fp.l1_done[i] = 0; }
        if (blockIdx.x == 0 && tid == 0) {
            arr[arrive_total_slot] = 0;
            fp.grid_sync[2] = 0;
            fp.grid_sync[MM_SYNC_REQUANT_HEAD] = 0;
            fp.grid_sync[MM_SYNC_PUSH_HEAD] = 0;
            fp.grid_sync[MM_SYNC_TILE_HEAD] = 0;
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
