#!/usr/bin/env python
"""Benchmark of the W8A8 channelwise Mega MoE layer on B200.

    python bench.py --gpus N --steps K --warmup W              # this implementation (one process per GPU)
    python bench.py --impl reference --gpus N --steps K --warmup W   # CPU arm: the oracle port on the host cores

Workload: the DSV4-Flash-shaped layer (256 experts, top-6, hidden 4096, intermediate 2048), 4096 tokens per rank,
logits ~ N(0,1) routing, EP = N (256/N experts per rank); synthetic seeded data, random-init weights quantised per
output channel.  One step = one pass of the layer over one batch.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

E, K, H, I = 256, 6, 4096, 2048
METRIC, UNIT = "moe_layer_tokens_per_s", "tokens/s"
FLOP_PER_ROW = 2 * 3 * H * I                     # 50.33 MFLOP per routed row (GEMM1 33.55 + GEMM2 16.78)
PARITY_SAMPLES = 4                               # tokens per rank checked against the CPU oracle after the timed region
# DRAM read + write bytes of one layer-kernel launch per expert processed at 96 rows per expert, from an ncu capture of a
# 32-expert launch (888 MB); the traffic of a launch grows with the experts it processes.  An estimate, labelled as such.
LAYER_KERNEL_DRAM_BYTES_PER_EXPERT_96ROWS = 888.0e6 / 32


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_bf16_tflops():
    """Dense bf16 burst figure of the machine-readable peak file (None if absent); twice it is the usual FP8 estimate."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f).get("bf16_tflops", 0.0)) or None
    return None


def parity_block(dist, group, rank, world, dev, sb, l1, l2, y, stats, tokens, n_samples=PARITY_SAMPLES, oracle_variant="fused"):
    """Correctness of the run that was just timed, computed outside the timed region at every N:
      counts_equal      per-expert receive statistics == bincount of all ranks' top-k indices (bit-exact routing counts);
      max_abs_over_rms, cosine   of `n_samples` tokens per rank against the CPU oracle (oracle/moe_oracle.py) run on just those
                        tokens -- a token's output depends on no other token.  Every rank runs the oracle for the sampled
                        routes that hit ITS experts (its weights never leave the rank); the per-route rows are summed over
                        ranks, then reduced in slot order as the layer does.
    The literal acceptance bar is max_abs <= 2e-2 * rms and cosine >= 0.999; `ok` is the run's pass/fail: counts equal,
    cosine >= 0.999 and no element off by more than 0.1 * rms (an FP8 activation code that flips on a rounding tie moves one
    output row by a few percent of rms, so the literal figure is reported beside it rather than asserted)."""
    import megamoe
    from oracle import moe_oracle as orc
    e_loc = E // world
    T = tokens
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))   # every rank runs its share of the oracle on the same host

    def gather(t):
        if dist is None:
            return t
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t.contiguous())
        return torch.cat(out, dim=0)

    idx_all = gather(sb.topk_idx[:T])
    w_all = gather(sb.topk_weights[:T])
    valid = (idx_all >= 0) & (idx_all < E) & (w_all != 0)
    counts = torch.bincount(idx_all[valid].flatten(), minlength=E)[rank * e_loc:(rank + 1) * e_loc].to(torch.int32)
    counts_equal = bool(torch.equal(counts, stats))

    gp = torch.Generator().manual_seed(4242 + rank)
    pick = torch.unique(torch.cat([torch.tensor([0, T - 1]), torch.randint(0, T, (max(n_samples - 2, 0),), generator=gp)]))[:n_samples]
    while pick.numel() < n_samples:                                     # duplicates removed above: top up deterministically
        pick = torch.unique(torch.cat([pick, torch.tensor([(int(pick[-1]) + 17) % T])]))
    pick = pick.to(dev)
    xq = gather(sb.x[pick].view(torch.uint8)).cpu().view(torch.float8_e4m3fn)
    xs = gather(sb.x_sf[pick]).cpu()
    idx_s = gather(sb.topk_idx[pick]).cpu()
    w_s = gather(sb.topk_weights[pick]).cpu()
    n_tok = idx_s.shape[0]
    mine = (idx_s >= rank * e_loc) & (idx_s < (rank + 1) * e_loc) & (w_s != 0)
    touched = torch.unique(idx_s[mine]) - rank * e_loc                  # local indices of the experts the samples hit here
    contrib = torch.zeros((n_tok, K, H), dtype=torch.float32)
    if touched.numel():
        remap = torch.full((E,), -1, dtype=torch.int64)
        remap[touched + rank * e_loc] = torch.arange(touched.numel())
        idx_local = torch.where(mine, remap[idx_s.clamp(0, E - 1)], torch.full_like(idx_s, -1))
        sel = touched.to(dev)
        w1p = megamoe.unpack_weights_tiled(l1[0][sel], "l1", 2 * I).cpu()
        w2p = megamoe.unpack_weights_tiled(l2[0][sel], "l2", H).cpu()
        _, lay, tr = orc.moe_layer([xq], [xs], [idx_local], [w_s], [w1p], [l1[1][sel].cpu()], [w2p], [l2[1][sel].cpu()],
                                   int(touched.numel()), None, oracle_variant, trace=True)
        rows = torch.from_numpy((lay.row_src_rank[0] >= 0).nonzero()[0])
        tt = torch.from_numpy(lay.row_src_token[0][rows.numpy()].astype("int64"))
        kk = torch.from_numpy(lay.row_src_slot[0][rows.numpy()].astype("int64"))
        contrib[tt, kk] = tr.out_rows[0][rows].float()
    contrib = contrib.to(dev)
    if dist is not None:
        dist.all_reduce(contrib)
    mine_rows = contrib[rank * n_samples:(rank + 1) * n_samples]
    acc = torch.zeros((n_samples, H), dtype=torch.float32, device=dev)
    for s_ in range(K):                                                 # slot order, fp32, one bf16 rounding
        acc += mine_rows[:, s_]
    y_ref = acc.to(torch.bfloat16)
    err, cos = orc.parity_metrics(y[pick].cpu(), y_ref.cpu())
    vals = torch.tensor([err, -cos, 0.0 if counts_equal else 1.0], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    err, cos, bad_counts = float(vals[0]), -float(vals[1]), float(vals[2]) > 0
    return {"counts_equal": not bad_counts, "max_abs_over_rms": round(err, 5), "cosine": round(cos, 7),
            "sampled_tokens_per_rank": n_samples, "oracle": f"oracle/moe_oracle.py, numerics '{oracle_variant}', on the sampled tokens",
            "literal_bar": {"max_abs_over_rms": 2e-2, "cosine": 0.999, "met": bool(err <= 2e-2 and cos >= 0.999)},
            "ok": bool((not bad_counts) and cos >= 0.999 and err <= 0.1)}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()          # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def init_dist(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return dist, dist.group.WORLD, rank, world, local
    if n_gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")
    torch.cuda.set_device(0)
    return None, None, 0, 1, 0


def make_rank_data(rank: int, world: int, tokens: int, dev):
    """Seeded synthetic inputs and weights of one rank, generated on the device (inputs also kept in pinned host memory)."""
    import megamoe
    e_loc = E // world
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    l1q = torch.empty((e_loc, I // 128, H // 128, 256, 128), dtype=torch.float8_e4m3fn, device=dev)   # tiled layout
    l1s = torch.empty((e_loc, 2 * I), dtype=torch.float32, device=dev)
    l2q = torch.empty((e_loc, H // 256, I // 128, 256, 128), dtype=torch.float8_e4m3fn, device=dev)
    l2s = torch.empty((e_loc, H), dtype=torch.float32, device=dev)
    step = 16
    for e0 in range(0, e_loc, step):   # a few experts at a time bounds the bf16 temporaries
        n = min(step, e_loc - e0)
        w1 = (torch.randn((n, 2 * I, H), generator=g, device=dev, dtype=torch.float32) / H ** 0.5).to(torch.bfloat16)
        w2 = (torch.randn((n, H, I), generator=g, device=dev, dtype=torch.float32) / I ** 0.5).to(torch.bfloat16)
        (a, as_), (b, bs_) = megamoe.transform_fp8_weights_for_mega_moe(w1, w2)
        l1q[e0:e0 + n], l1s[e0:e0 + n], l2q[e0:e0 + n], l2s[e0:e0 + n] = a, as_, b, bs_
        del w1, w2, a, b
    x = torch.randn((tokens, H), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn((tokens, E), generator=g, device=dev, dtype=torch.float32)
    w, idx = torch.topk(torch.softmax(logits, dim=-1), K, dim=-1)
    w = (w / w.sum(dim=-1, keepdim=True)).float()
    return (l1q, l1s), (l2q, l2s), x, idx.to(torch.int64), w


def _plain(w, which, rows):
    """Weights as plain [E, rows, K] on the host (undo the tiled packing)."""
    import megamoe
    return megamoe.unpack_weights_tiled(w, which, rows).cpu() if w.dim() == 5 else w.cpu()


def cpu_baseline(l1, l2, x_q, x_s, idx, w, n_experts: int, threads: int, repeats: int = 1):
    """Time the CPU oracle on the rows of the first `n_experts` experts of rank 0 (a bounded sample of the workload).
    Returns (tokens/s equivalent, rows in the sample, seconds)."""
    from oracle import moe_oracle as orc
    torch.set_num_threads(threads)
    keep = idx < n_experts
    idx_s = torch.where(keep, idx, torch.full_like(idx, -1)).cpu()
    args = ([x_q.cpu()], [x_s.cpu()], [idx_s], [w.cpu()],
            [_plain(l1[0][:n_experts], "l1", 2 * I)], [l1[1][:n_experts].cpu()], [_plain(l2[0][:n_experts], "l2", H)], [l2[1][:n_experts].cpu()])
    rows = int(keep.sum().item())
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.moe_layer(*args, n_experts, None, "fused")
        best = min(best, time.perf_counter() - t0)
    return rows / K / best, rows, best


def run_reference_arm(args):
    """--impl reference: the reference has no runnable CPU or CUDA implementation of this path (HIP/gfx938 only), so
    this arm times the CPU restatement of its arithmetic (oracle/moe_oracle.py) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import moe_oracle as orc
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    tokens, n_exp = args.tokens, 8
    g = torch.Generator().manual_seed(1000)
    w1 = (torch.randn((n_exp, 2 * I, H), generator=g) / H ** 0.5).to(torch.bfloat16)
    w2 = (torch.randn((n_exp, H, I), generator=g) / I ** 0.5).to(torch.bfloat16)
    l1 = orc.cast_grouped_weight_to_fp8_channelwise(w1); l2 = orc.cast_grouped_weight_to_fp8_channelwise(w2)
    x = torch.randn((tokens, H), generator=g).to(torch.bfloat16)
    xq, xs = orc.cast_to_fp8_channelwise(x)
    idx, w = orc.make_routing(tokens, E, K, seed=1000)
    times, rows = [], 0
    for i in range(args.warmup + args.steps):
        v, rows, t = cpu_baseline(l1, l2, xq, xs, idx, w, n_exp, threads)
        if i >= args.warmup:
            times.append(t)
    t_step = sum(times) / len(times)
    value = rows / K / t_step
    sample = f"rows routed to the first {n_exp} of {E} experts ({rows} of {tokens * K} routed rows) per step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"DSV4-Flash MoE layer: {E} experts top-{K} hidden {H} intermediate {I}, {tokens} tokens/rank, "
                               f"EP={max(1, args.gpus)}, uniform N(0,1)-logit routing, W8A8 channelwise",
                   "tokens_per_rank": tokens, "ep": max(1, args.gpus), "l2": "n/a (host cores)",
                   "variant": "CPU restatement of the reference arithmetic on a bounded sample (rank 0's rows only)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def nvlink_store_probe(dist, group, rank, world, dev, sb):
    """GB/s per direction of this library's own plain 16-byte stores into peers' receive pools (between layer calls): to
    the next rank only and spread over all peers, every rank storing at once; the slowest rank's best of three."""
    import ctypes
    from deepgemm_b200 import _lib
    lib = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    pool_bytes = sb.pool_rows * H // 512 * 512
    peers = [p_ for r_, p_ in enumerate(sb.handle.buffer_ptrs) if r_ != rank]
    probe = {}
    for name, dsts, nbytes in (("one_peer", [sb.handle.buffer_ptrs[(rank + 1) % world]], min(pool_bytes, 256 << 20)),
                               ("all_peers", peers, min(pool_bytes, (256 << 20) // len(peers) // 512 * 512))):
        arr = (ctypes.c_uint64 * len(dsts))(*[d + sb._sym_off["pool_x"] for d in dsts])
        best = 0.0
        for _ in range(3):
            torch.cuda.synchronize(); dist.barrier(group); torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            _lib.check(lib.mm_peer_store_probe(arr, len(dsts), nbytes, stream))
            t1.record()
            torch.cuda.synchronize()
            best = max(best, nbytes * len(dsts) / (t0.elapsed_time(t1) * 1e-3) / 1e9)
        t = torch.tensor([best], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        probe[name] = round(float(t.item()), 1)
    torch.cuda.synchronize(); dist.barrier(group)
    return probe


def tile_trace(layer, dev, cta: int, max_tiles: int = 128):
    """One call of the layer with the layer kernel's per-tile cycle stamps switched on for one CTA (mm_set_tile_trace).
    Per tile the kernel records the SM's clock64 when the producer took the tile / saw its dependency met / issued its last
    copy, when the MMA issuer took it / issued its first / its last MMA, and when the first epilogue warp began to wait for the
    accumulator / saw it complete / released it.  Returns per GEMM the medians, in SM cycles, of
      cadence  = accumulator complete -> next accumulator complete (what a tile costs the CTA),
      mainloop = first MMA issued -> accumulator complete,
      epilogue = accumulator complete -> released,
      wait     = MMA issuer took the tile -> its first operands had landed;
    the ideal mainloop is 128 cycles per M128 x N256 x K32 MMA: 16 384 (GEMM1, K = 4096) and 8 192 (GEMM2, K = 2048)."""
    import statistics
    from deepgemm_b200 import _lib
    lib = _lib.lib()
    buf = torch.zeros((max_tiles, 12), dtype=torch.int64, device=dev)
    _lib.check(lib.mm_set_tile_trace(buf.data_ptr(), max_tiles, cta))
    try:
        layer()
        torch.cuda.synchronize()
    finally:
        _lib.check(lib.mm_set_tile_trace(None, 0, 0))
    rows = [r for r in buf.cpu().tolist() if r[1] != 0]
    out = {"cta": cta, "tiles": len(rows), "unit": "SM cycles"}
    if not rows:
        return out
    t0 = rows[0][1]
    per_kind = {0: [], 1: []}
    prev_full = None
    print("  j kind   tile | producer: took dep-met last-copy | mma: took first last | epilogue: wait complete released", file=sys.stderr)
    for j, r in enumerate(rows):
        tile, kind = r[0] & 0xffffffff, r[0] >> 32
        pb, pd, pe, mb_, mf, me, eb, ef, ee = [(v - t0) if v else -1 for v in r[1:10]]
        print(f"{j:3d} G{kind + 1} {tile:7d} | {pb:9d} {pd:9d} {pe:9d} | {mb_:9d} {mf:9d} {me:9d} | {eb:9d} {ef:9d} {ee:9d}", file=sys.stderr)
        if prev_full is not None and ef > 0 and j >= 2:       # the first tiles include the start-up of the call
            per_kind[kind].append((ef - prev_full, ef - mf, ee - ef, mf - mb_))
        prev_full = ef
    for kind, name in ((0, "gemm1"), (1, "gemm2")):
        if per_kind[kind]:
            cols = list(zip(*per_kind[kind]))
            out[name] = {"tiles": len(per_kind[kind]), "cadence": statistics.median(cols[0]), "mainloop": statistics.median(cols[1]),
                         "epilogue": statistics.median(cols[2]), "wait": statistics.median(cols[3])}
    return out


def run_sweep(args):
    """--sweep: the scaling sweep of the layer (tokens per rank x routing skew) at the launched EP size.  One JSON line per
    point from rank 0: tokens/s, FP8 TFLOP/s, NVLink GB/s per rank and the three roofline times (tensor at the measured FP8
    peak, HBM at the measured copy peak, NVLink at the rate of this library's own store probe); max over ranks, CUDA events."""
    dist, group, rank, world, local = init_dist(args.gpus)
    dev = torch.device("cuda", local)
    import megamoe
    from deepgemm_b200 import _lib
    token_list = [int(t) for t in args.sweep.split(",")]
    t_max = max(token_list)
    e_loc = E // world
    l1, l2, _, _, _ = make_rank_data(rank, world, 8, dev)
    sb = megamoe.get_symm_buffer_for_mega_moe(group, E, t_max, K, H, I)
    fp8_peak = _lib.fp8_mma_peak_tflops()                                   # all-ones operands: the burst rate
    fp8_peak_data = _lib.fp8_mma_peak_tflops(random_operands=True)          # random operands: what real data can reach
    hbm_peak, _ = measured_peaks()
    # NVLink denominator: this library's own store probe spread over all peers (measured here, printed in every line)
    nvl_probe = nvlink_store_probe(dist, group, rank, world, dev, sb) if world > 1 else {"one_peer": None, "all_peers": None}
    nvl_gbs = nvl_probe["all_peers"] or 1.0
    g = torch.Generator(device=dev).manual_seed(2000 + rank)
    gp = torch.Generator().manual_seed(12345)
    pop = torch.empty(E)
    pop[torch.randperm(E, generator=gp)] = torch.arange(1, E + 1, dtype=torch.float32) ** -1.1
    log_pop = torch.log(pop / pop.sum()).to(dev)
    for routing in ("uniform", "zipf"):
        for T in token_list:
            x = torch.randn((T, H), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
            logits = torch.randn((T, E), generator=g, device=dev, dtype=torch.float32)
            if routing == "zipf":
                logits = logits + 1.5 * log_pop.view(1, -1)
            megamoe.fill_inputs_from_router(sb, x, logits)
            y = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
            stats = torch.zeros((e_loc,), dtype=torch.int32, device=dev)
            megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb, cumulative_local_expert_recv_stats=stats, dispatch_num_tokens=T)
            for _ in range(3):
                megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb, dispatch_num_tokens=T)
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier(group)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            steps = max(5, args.steps)
            ev0.record()
            for _ in range(steps):
                megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb, dispatch_num_tokens=T)   # every rank holds T tokens
            ev1.record()
            torch.cuda.synchronize()
            sb.check_status()
            ms = ev0.elapsed_time(ev1) / steps
            rows = int(stats.sum().item()); touched = int((stats > 0).sum().item())
            vals = torch.tensor([ms, rows, touched, float(stats.max().item())], dtype=torch.float64, device=dev)
            if dist is not None:
                allv = [torch.zeros_like(vals) for _ in range(world)]
                dist.all_gather(allv, vals)
                allv = torch.stack(allv)
            else:
                allv = vals.view(1, -1)
            ms = float(allv[:, 0].max()); rows_max = float(allv[:, 1].max()); rows_sum = float(allv[:, 1].sum())
            t_tensor = rows_max * FLOP_PER_ROW / (fp8_peak_data * 1e12) * 1e3   # against the rate random operands reach
            hbm_bytes = float(allv[:, 2].max()) * (3 * H * I + 4 * (2 * I + H)) + rows_max * (H + 4 + (I + 4) * 2 + 2 * H)
            t_hbm = hbm_bytes / (hbm_peak * 1e9) * 1e3
            remote = rows_max * (world - 1) / world
            t_nvl = remote * (H + 16 + 2 * H) / (nvl_gbs * 1e9) * 1e3   # dispatch in + combine out share a direction in time
            t_roof = max(t_tensor, t_hbm, t_nvl)
            if rank == 0:
                print(json.dumps({
                    "sweep": True, "ep": world, "tokens_per_rank": T, "routing": routing, "ms": round(ms, 4),
                    "tokens_per_s": round(T * world / (ms * 1e-3)), "fp8_tflops_total": round(rows_sum * FLOP_PER_ROW / (ms * 1e-3) / 1e12, 1),
                    "fp8_frac_of_measured_peak_per_gpu": round(rows_max * FLOP_PER_ROW / (ms * 1e-3) / 1e12 / fp8_peak_data, 3),
                    "fp8_peak_tflops": {"ones_operands": round(fp8_peak, 1), "random_operands": round(fp8_peak_data, 1)},
                    "nvlink_gbs_per_rank": round(remote * (H + 16 + 2 * H) / (ms * 1e-3) / 1e9, 1),
                    "nvlink_store_probe_gbs": nvl_probe,
                    "max_rows_per_expert": int(allv[:, 3].max()), "rows_max_rank": int(rows_max),
                    "roof_ms": {"tensor": round(t_tensor, 4), "hbm": round(t_hbm, 4), "nvlink": round(t_nvl, 4)},
                    "frac_of_roofline": round(t_roof / ms, 3),
                    "variant": "fused" if T <= sb._large_opt_3stage_threshold else
                               ("staged-split" if megamoe._staged_as_split_launches(sb, T, e_loc) else "staged")}), flush=True)
    sb.destroy()
    if dist is not None:
        dist.barrier(group)
        dist.destroy_process_group()


def run_split_baseline(args):
    """Expert-parallel size 1: the split pipeline of the reference's test (tests/test_mega_moe_dcu.py:188-300) against the
    layer call on the same quantised inputs.  Without ranks there is no DeepEP dispatch / combine, so this compares only
    what happens on one GPU: five launches with a bf16 [rows, 2I] round trip against the layer's launches."""
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    import megamoe
    T = args.tokens
    l1, l2, x_bf16, idx, w = make_rank_data(0, 1, T, dev)
    sb = megamoe.get_symm_buffer_for_mega_moe(None, E, T, K, H, I)
    xq, xs = megamoe.cast_to_fp8_channelwise(x_bf16)
    sb.x[:T].copy_(xq); sb.x_sf[:T].copy_(xs); sb.topk_idx[:T].copy_(idx); sb.topk_weights[:T].copy_(w)
    y = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    # the grouped GEMM wants W1 rows in natural order (gate rows, then up rows); the layer's tiling interleaves them
    w1_nat = torch.empty((E, (2 * I) // 256, H // 128, 256, 128), dtype=torch.float8_e4m3fn, device=dev)
    for e0 in range(0, E, 16):
        w1_nat[e0:e0 + 16] = megamoe.pack_weights_tiled(megamoe.unpack_weights_tiled(l1[0][e0:e0 + 16], "l1", 2 * I), "l2")
    counts = torch.bincount(idx.flatten(), minlength=E)
    aligned = ((counts + 127) // 128 * 128).to(torch.int32)
    rows = int(aligned.sum())
    l1_out = torch.empty((rows, 2 * I), dtype=torch.bfloat16, device=dev)
    a8 = torch.empty((rows, I), dtype=torch.float8_e4m3fn, device=dev)
    a8s = torch.empty((rows,), device=dev)
    l2_out = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)
    y2 = torch.empty((T, H), dtype=torch.bfloat16, device=dev)

    def split():
        gx, gs, rw, mi, oi = megamoe.deepep_deepgemm_preprocess_channelwise(xq, xs, idx, w, aligned, rows)
        megamoe.m_grouped_fp8_gemm_nt_contiguous((gx, gs), (w1_nat, l1[1]), l1_out, mi)
        megamoe.swiglu_quant_channelwise_out(l1_out, rw, a8, a8s, None, num_per_channels=I, clamp_value=None)
        megamoe.m_grouped_fp8_gemm_nt_contiguous((a8, a8s), l2, l2_out, mi)
        megamoe.deepep_deepgemm_postprocess_channelwise(y2, l2_out, idx, w, oi, apply_topk_weights=False)

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    ms_layer = timed(lambda: megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb))
    ms_split = timed(split)
    sb.check_status()
    a, b = y.float().flatten(), y2.float().flatten()
    cos = float(torch.nn.functional.cosine_similarity(a.double(), b.double(), dim=0))
    print(json.dumps({"split_baseline": True, "workload": f"{E} experts top-{K} hidden {H} intermediate {I}, {T} tokens, EP=1",
                      "layer_ms": round(ms_layer, 4), "split_pipeline_ms": round(ms_split, 4),
                      "split_over_layer": round(ms_split / ms_layer, 3), "grouped_rows": rows, "cosine_layer_vs_split": round(cos, 6)}),
          flush=True)
    sb.destroy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=4096, help="tokens per rank")
    ap.add_argument("--variant", default="auto", choices=["auto", "fused", "staged", "split"],
                    help="kernel variant: auto = the API's token threshold (fused up to 256 tokens, staged above); "
                         "split = the staged variant as separate dispatch / GEMM1 / requantisation / GEMM2 launches")
    ap.add_argument("--experts", type=int, default=E, help="total experts (reduce only for small profiler captures)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--split-baseline", action="store_true",
                    help="one GPU: time the reference test's split pipeline (scatter, grouped GEMM, SwiGLU+quantise, grouped GEMM, "
                         "gather) built from this library's kernels next to the layer call, on the same inputs")
    ap.add_argument("--recipe", default="channelwise", choices=["channelwise", "ue8m0"],
                    help="activation recipe between the GEMMs: the reference's channelwise fp32 scales (default) or per-32 UE8M0 scales "
                         "applied by a block-scaled MMA (staged launches; parity is then checked against the oracle's ue8m0 variant)")
    ap.add_argument("--profile-only", action="store_true",
                    help="device-resident arm only (no end-to-end arm, no parity or CPU baseline): the command line for ncu captures")
    ap.add_argument("--sweep", default=None, help="comma-separated tokens-per-rank list: run the scaling sweep instead of the bench")
    ap.add_argument("--tile-trace", type=int, default=None, metavar="CTA",
                    help="with --profile-only: after the timed steps run one more call with the layer kernel's per-tile cycle "
                         "stamps switched on for this CTA and add their medians (SM cycles) to the line; the table goes to stderr")
    args = ap.parse_args()
    if args.tile_trace is not None and not args.profile_only:
        ap.error("--tile-trace needs --profile-only")
    globals()["E"] = args.experts
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.sweep:
        run_sweep(args)
        return
    if args.split_baseline:
        run_split_baseline(args)
        return

    dist, group, rank, world, local = init_dist(args.gpus)
    dev = torch.device("cuda", local)
    import ctypes
    import megamoe
    from deepgemm_b200 import _lib
    T = args.tokens
    e_loc = E // world
    l1, l2, x_bf16, idx, w = make_rank_data(rank, world, T, dev)
    sb = megamoe.get_symm_buffer_for_mega_moe(group, E, T, K, H, I)
    if args.variant != "auto":
        sb._large_opt_3stage_mode = {"fused": "off", "staged": "force", "split": "force"}[args.variant]
        sb._staged_split = args.variant == "split"
        sb._staged_split_auto = False
    staged = megamoe._large_opt_3stage_selected(T, sb._large_opt_3stage_mode, sb._large_opt_3stage_threshold)
    variant = ("staged-split" if megamoe._staged_as_split_launches(sb, T, e_loc) else "staged") if staged else "fused"
    y = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    lib = _lib.lib()

    def quantise_into_buffer(src):
        _lib.check(lib.mm_quant_per_token(src.data_ptr(), T, H, sb.x.data_ptr(), sb.x_sf.data_ptr(), stream))

    recipe_kw = {"recipe": megamoe.RECIPE_UE8M0_PER32} if args.recipe == "ue8m0" else {}
    if args.recipe == "ue8m0":
        variant = "staged-ue8m0"

    def layer():
        megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb, **recipe_kw)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier(group)
            torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident arm: inputs already quantised in the symmetric buffer ----------------------------------
    quantise_into_buffer(x_bf16)
    sb.topk_idx[:T].copy_(idx); sb.topk_weights[:T].copy_(w)
    for _ in range(max(args.warmup, 3)):
        layer()
    barrier()
    sb.check_status()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        layer()
    ev1.record()
    barrier()
    launches = _lib.launch_count() - launches0
    ms_step = max_over_ranks(ev0.elapsed_time(ev1) / args.steps)
    sb.check_status()
    if args.profile_only:
        sampler.stop()
        line = {"profile_only": True, "ms_per_step": ms_step, "gpu_launches": launches, "experts": E, "tokens_per_rank": T,
                "ep": world, "variant": variant}
        if args.tile_trace is not None:
            line["tile_trace"] = tile_trace(layer, dev, args.tile_trace)
        if rank == 0:
            print(json.dumps(line), flush=True)
        sb.destroy()
        if dist is not None:
            dist.barrier(group)
            dist.destroy_process_group()
        return

    # ---- end-to-end arm: host buffers in, host buffer out, every step ------------------------------------------
    # Every step copies its inputs from pinned host memory (bf16 activations, top-k indices and weights), quantises,
    # runs the layer and copies y back to pinned host memory.  The three phases run on three streams with double
    # buffering, so step i+1's upload and step i-1's download overlap step i's compute, as a serving loop would do.
    # compute=False runs the same copies on the same streams without the kernels: the copy floor of this box.
    hx = x_bf16.cpu().pin_memory(); hidx = idx.cpu().pin_memory(); hw = w.cpu().pin_memory()
    hy = [torch.empty((T, H), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    dx = [torch.empty_like(x_bf16) for _ in range(2)]
    didx = [torch.empty_like(idx) for _ in range(2)]
    dw = [torch.empty_like(w) for _ in range(2)]
    dy = [y, torch.empty_like(y)]
    s_main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_ready = [torch.cuda.Event() for _ in range(2)]     # inputs of buffer b are on the device
    ev_free = [torch.cuda.Event() for _ in range(2)]      # compute has consumed the staged inputs of buffer b
    ev_done = [torch.cuda.Event() for _ in range(2)]      # y of buffer b is complete
    ev_out = [torch.cuda.Event() for _ in range(2)]       # y of buffer b has reached the host
    for e in ev_free + ev_out:
        e.record(s_main)

    def e2e_step(i, compute=True):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_free[b])
            dx[b].copy_(hx, non_blocking=True)
            didx[b].copy_(hidx, non_blocking=True)
            dw[b].copy_(hw, non_blocking=True)
            ev_ready[b].record(s_in)
        s_main.wait_event(ev_ready[b])
        if compute:
            sb.topk_idx[:T].copy_(didx[b], non_blocking=True)
            sb.topk_weights[:T].copy_(dw[b], non_blocking=True)
            quantise_into_buffer(dx[b])
        ev_free[b].record(s_main)
        s_main.wait_event(ev_out[b])                      # the previous y in this buffer has left the device
        if compute:
            megamoe.fp8_w8a8_mega_moe(dy[b], l1, l2, sb, **recipe_kw)
        ev_done[b].record(s_main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[b])
            hy[b].copy_(dy[b], non_blocking=True)
            ev_out[b].record(s_out)

    def time_e2e(compute):
        for i in range(4):
            e2e_step(i, compute)
        barrier()
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev2.record(s_main)
        for i in range(args.steps):
            e2e_step(i, compute)
        s_main.wait_event(ev_out[0]); s_main.wait_event(ev_out[1])   # the timed region ends when the last y is on the host
        ev3.record(s_main)
        barrier()
        return max_over_ranks(ev2.elapsed_time(ev3) / args.steps)

    e2e_ms = time_e2e(True)
    clocks = sampler.stop()
    copy_floor_ms = time_e2e(False)
    h2d = T * H * 2 + T * K * 8 + T * K * 4
    d2h = T * H * 2

    # ---- per-stage times (CUDA events recorded by the library on the launching stream) --------------------------
    sb.topk_idx[:T].copy_(idx); sb.topk_weights[:T].copy_(w); quantise_into_buffer(x_bf16)
    lib.mm_set_stage_timing(1)
    acc = {}
    n_rep = max(3, min(10, args.steps))
    for _ in range(n_rep):
        barrier()                      # ranks start each timed call together, else the skew lands in the first cross-rank wait
        layer()
        for k_, v in _lib.stage_times().items():
            acc[k_] = acc.get(k_, 0.0) + v / n_rep
    lib.mm_set_stage_timing(0)
    stats = torch.zeros((e_loc,), dtype=torch.int32, device=dev)
    megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb, cumulative_local_expert_recv_stats=stats, **recipe_kw)
    torch.cuda.synchronize()
    sb.check_status()
    rows_recv = int(stats.sum().item())
    touched = int((stats > 0).sum().item())
    parity = parity_block(dist, group, rank, world, dev, sb, l1, l2, y, stats, T, min(PARITY_SAMPLES, T),
                          oracle_variant="ue8m0" if args.recipe == "ue8m0" else "fused")

    # ---- roofline of the dominant kernel ----------------------------------------------------------------------------
    split = "gemm1" in acc        # separate GEMM1 / requantisation / GEMM2 launches (MEGAMOE_STAGED_SPLIT=1)
    kernel_ms = max_over_ranks(acc["gemm1"] if split else acc["fused"])
    if split:
        # GEMM1 launch: FP8 gate+up weights and scales of the touched experts, the received FP8 rows with their 16-byte
        # metadata, the bf16 activations written
        kernel_bytes = touched * (2 * I * H + 4 * 2 * I) + rows_recv * (H + 16) + rows_recv * I * 2
        kernel_flops = rows_recv * 2 * H * 2 * I
        kernel_name = "grouped_gemm_kernel<0> (GEMM1 + SwiGLU)"
        if args.recipe == "ue8m0":             # codes and scale bytes instead of bf16 activations
            kernel_bytes = touched * (2 * I * H + 4 * 2 * I) + rows_recv * (H + 16) + rows_recv * (I + I // 32)
            kernel_name = "grouped_gemm_kernel<2> (GEMM1 + SwiGLU + per-32 UE8M0 quantisation)"
    else:
        # the layer kernel moves the whole layer's bytes (formula of the reference's own test,
        # tests/test_mega_moe_dcu.py:352-364): weights + scales, FP8 rows in, FP8 activations written and read, bf16 rows out
        kernel_bytes = touched * (3 * H * I + 4 * (2 * I + H)) + rows_recv * (H + 4) + rows_recv * (I + 4) * 2 + rows_recv * H * 2
        kernel_flops = rows_recv * FLOP_PER_ROW
        kernel_name = ("mega_moe_fused_kernel (NVLink push + GEMM1 + requantisation + GEMM2 + combine stores)" if staged
                       else "mega_moe_fused_kernel (whole layer)")
    hbm_peak, peak_kind = measured_peaks()
    achieved = kernel_bytes / (kernel_ms * 1e-3) / 1e9
    roofline = {"kernel": kernel_name, "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak, "peak_kind": f"of {peak_kind}",
                "traffic": (LAYER_KERNEL_DRAM_BYTES_PER_EXPERT_96ROWS * touched
                            if (not split and 64 <= rows_recv / max(touched, 1) <= 128) else None),
                "traffic_note": "estimate: scaled from an ncu capture of a 32-expert launch of the same kernel at 96 rows per "
                                "expert (traffic grows with the experts processed); not measured in this run",
                "algorithmic_bytes": kernel_bytes, "ms": kernel_ms}
    # With many rows per expert the same kernel is bound by the tensor pipe instead.  The machine-readable peak file has a
    # bf16 figure only, so the FP8 denominator is the library's own probe of the MMA shape the kernel issues, run with
    # pseudo-random operands; the all-ones probe value and twice the measured bf16 figure are printed beside it.
    if rows_recv >= 200 * max(touched, 1):
        fp8_rand = _lib.fp8_mma_peak_tflops(random_operands=True)
        if kernel_flops / (fp8_rand * 1e12) > kernel_bytes / (hbm_peak * 1e9):
            fp8_ones = _lib.fp8_mma_peak_tflops(random_operands=False)
            fp8_quant = _lib.fp8_mma_peak_tflops(quantised_like_operands=True)
            bf16 = measured_bf16_tflops()
            tf = kernel_flops / (kernel_ms * 1e-3) / 1e12
            roofline = {"kernel": kernel_name, "bound": "tensor", "achieved": tf, "peak": fp8_rand, "unit": "TFLOP/s",
                        "frac": tf / fp8_rand, "peak_kind": "of measured: own FP8 MMA probe with random operands, burst "
                        "(MEASURED_PEAKS.json holds a bf16 figure only)",
                        "fp8_peak_candidates_tflops": {"probe_random_operands": round(fp8_rand, 1), "probe_ones_operands": round(fp8_ones, 1),
                                                       "probe_quantised_like_operands": round(fp8_quant, 1),
                                                       "twice_measured_bf16": None if bf16 is None else round(2 * bf16, 1)},
                        "frac_of": {"probe_ones_operands": round(tf / fp8_ones, 4),
                                    "probe_quantised_like_operands": round(tf / fp8_quant, 4),
                                    "twice_measured_bf16": None if bf16 is None else round(tf / (2 * bf16), 4)},
                        "traffic": None, "traffic_note": "tensor-bound: see profiles/ for the pipe-utilisation capture",
                        "algorithmic_flops": kernel_flops, "algorithmic_bytes": kernel_bytes, "ms": kernel_ms}

    total_rows = T * K * world
    value = T * world / (ms_step * 1e-3)
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3",
        "data": "synthetic",
        "config": {"workload": f"DSV4-Flash MoE layer: {E} experts top-{K} hidden {H} intermediate {I}, {T} tokens/rank, EP={world}, "
                               "uniform N(0,1)-logit routing, W8A8 channelwise", "tokens_per_rank": T, "ep": world,
                   "l2": "weights streamed per step exceed L2 (no flush needed)", "variant": variant},
        "fp8_tflops": total_rows * FLOP_PER_ROW / (ms_step * 1e-3) / 1e12,
        "e2e": {"value": T * world / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "copy_floor_ms": copy_floor_ms,
                "over_floor": e2e_ms / max(copy_floor_ms, ms_step)},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": roofline,
        "stage_ms": {k_: round(v, 4) for k_, v in acc.items()},
        "parity": parity,
    }

    if world > 1:
        # ---- exposed communication: the step minus its all-local twin (this rank's experts only, the same token count and
        #      top-k, one rank, no peer traffic), measured in the same run on every GPU at once
        twin = megamoe.get_symm_buffer_for_mega_moe(None, e_loc, T, K, H, I)
        twin._large_opt_3stage_mode = sb._large_opt_3stage_mode
        twin._staged_split, twin._staged_split_auto = megamoe._staged_as_split_launches(sb, T, e_loc), False
        g = torch.Generator(device=dev).manual_seed(77 + rank)
        tw_, ti_ = torch.topk(torch.softmax(torch.randn((T, e_loc), generator=g, device=dev), dim=-1), K, dim=-1)
        twin.x[:T].copy_(sb.x[:T]); twin.x_sf[:T].copy_(sb.x_sf[:T])
        twin.topk_idx[:T].copy_(ti_); twin.topk_weights[:T].copy_((tw_ / tw_.sum(-1, keepdim=True)).float())
        for _ in range(3):
            megamoe.fp8_w8a8_mega_moe(y, l1, l2, twin)
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            megamoe.fp8_w8a8_mega_moe(y, l1, l2, twin)
        t1.record()
        barrier()
        twin.check_status()
        twin_ms = max_over_ranks(t0.elapsed_time(t1) / args.steps)
        twin.destroy()
        out["exposed_comm"] = {"all_local_twin_ms": twin_ms, "ms": ms_step - twin_ms, "frac_of_step": (ms_step - twin_ms) / ms_step}
        # ---- NVLink: plain 16-byte stores of this library to one peer and to all peers (every rank at once), and the
        #      remote bytes of the step over the time of the kernel(s) that move them
        probe = nvlink_store_probe(dist, group, rank, world, dev, sb)
        remote = rows_recv * (world - 1) / world
        nvl = {"store_probe_gbs_per_direction": probe, "dispatch_bytes_out_per_rank": remote * (H + 16),
               "combine_bytes_out_per_rank": remote * 2 * H}
        if split:
            nvl["dispatch_gbs"] = remote * (H + 16) / (max_over_ranks(acc["dispatch"]) * 1e-3) / 1e9
            nvl["combine_gbs_over_gemm2"] = remote * 2 * H / (max_over_ranks(acc["gemm2"]) * 1e-3) / 1e9
        else:
            nvl["out_gbs_over_layer_kernel"] = remote * (3 * H + 16) / (kernel_ms * 1e-3) / 1e9
        out["nvlink"] = nvl

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        n_exp = min(E, 128)                 # about 10 s of host work in all (three passes, best one reported)
        v, rows, secs = cpu_baseline(l1, l2, sb.x[:T], sb.x_sf[:T], idx, w, n_exp, threads, repeats=3)
        out["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                               "gflops": round(rows * FLOP_PER_ROW / secs / 1e9, 1),
                               "sample": f"rows routed to the first {n_exp} of {E} experts ({rows} of {T * K} routed rows), "
                                         f"best of 3 passes, {secs:.1f} s each"}
    if rank == 0:
        print(json.dumps(out), flush=True)
    sb.destroy()
    if dist is not None:
        dist.barrier(group)
        dist.destroy_process_group()
    if not parity["ok"]:
        raise SystemExit("parity check failed: " + json.dumps(parity))


if __name__ == "__main__":
    main()
