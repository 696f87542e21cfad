"""Expert-parallel parity on 2..8 GPUs of one node: one process per GPU, NVLink push dispatch and remote combine.

Skipped when fewer than two GPUs are visible.  Each child runs its rank through the megamoe API and compares every
stage with the CPU oracle evaluated for all ranks (the shapes are small enough for every child to do that).
"""
import os
import socket

import numpy as np
import pytest
import torch

import moe_case as mc

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, cfg):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from deepgemm_b200 import _lib
        _lib.lib().mm_set_timeouts(20000, 4000)
        tokens = cfg["tokens"][:world]
        case = mc.make_case(world, cfg["E"], cfg["K"], cfg["H"], cfg["I"], tokens, seed=cfg["seed"], zipf=cfg.get("zipf", False),
                            invalid_fraction=cfg.get("invalid", 0.0))
        ys, lay, tr = mc.run_oracle(case, cfg.get("clamp"), "fused", trace=True)
        stats = torch.zeros((cfg["E"] // world,), dtype=torch.int32, device="cuda")
        # ranks hold different token counts: one dispatch_num_tokens for all of them keeps the variant choice uniform
        uniform = dict(dispatch_num_tokens=max(tokens))
        y, sb = mc.run_cuda_rank(case, rank, group=dist.group.WORLD, clamp=cfg.get("clamp"), keep=True,
                                 t_max=max(max(tokens), 1), stats=stats, variant=cfg.get("variant"), **uniform)
        f = mc.compare_stages(case, rank, sb, lay, tr, log=lambda *_: None)
        for key in ("x_q_equal", "x_s_equal", "dest_row_equal", "totals_equal", "pool_off_equal", "plan_rows_equal",
                    "pool_rows_equal", "pool_meta_equal"):
            assert f[key], f"rank {rank}: {key}"
        e_loc = cfg["E"] // world
        assert stats.cpu().tolist() == lay.totals[rank * e_loc:(rank + 1) * e_loc].tolist()
        if lay.totals[rank * e_loc:(rank + 1) * e_loc].sum():
            assert f["act_q_mismatch_frac"] < 1e-3 and f["act_scale_max_rel"] < 1e-2, (rank, f)
        mc.assert_end_to_end_close(y, ys[rank], f"rank {rank}")
        # a second call on the same buffers reproduces the first bit for bit
        y2, _ = mc.run_cuda_rank(case, rank, group=dist.group.WORLD, clamp=cfg.get("clamp"), sb=sb, variant=cfg.get("variant"),
                                 **uniform)
        assert torch.equal(y.view(torch.int16), y2.view(torch.int16)), f"rank {rank}: not deterministic"
        sb.destroy()
    finally:
        dist.barrier()
        dist.destroy_process_group()


def _recipe_worker(rank, world, port, cfg):
    """End-to-end parity of a recipe other than the default on several ranks (the stage-by-stage helpers above read the
    channelwise recipe's intermediates)."""
    import torch.distributed as dist
    import megamoe
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from deepgemm_b200 import _lib
        _lib.lib().mm_set_timeouts(20000, 4000)
        tokens = cfg["tokens"][:world]
        case = mc.make_case(world, cfg["E"], cfg["K"], cfg["H"], cfg["I"], tokens, seed=cfg["seed"], invalid_fraction=cfg.get("invalid", 0.0))
        ys, lay, _ = mc.run_oracle(case, cfg.get("clamp"), cfg["oracle"])
        e_loc = cfg["E"] // world
        stats = torch.zeros((e_loc,), dtype=torch.int32, device="cuda")
        y, sb = mc.run_cuda_rank(case, rank, group=dist.group.WORLD, clamp=cfg.get("clamp"), keep=True, t_max=max(max(tokens), 1),
                                 stats=stats, recipe=getattr(megamoe, cfg["recipe"]), dispatch_num_tokens=max(tokens))
        assert stats.cpu().tolist() == lay.totals[rank * e_loc:(rank + 1) * e_loc].tolist()
        mc.assert_end_to_end_close(y, ys[rank], f"rank {rank}")
        y2, _ = mc.run_cuda_rank(case, rank, group=dist.group.WORLD, clamp=cfg.get("clamp"), sb=sb, recipe=getattr(megamoe, cfg["recipe"]),
                                 dispatch_num_tokens=max(tokens))
        assert torch.equal(y.view(torch.int16), y2.view(torch.int16)), f"rank {rank}: not deterministic"
        sb.destroy()
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_ep2_ue8m0_recipe_uneven_tokens():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    cfg = dict(E=16, K=4, H=1024, I=512, tokens=[300, 77], seed=28, invalid=0.1, clamp=10.0, recipe="RECIPE_UE8M0_PER32", oracle="ue8m0")
    mp.spawn(_recipe_worker, args=(2, _free_port(), cfg), nprocs=2, join=True)


def _run(world, cfg):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), cfg), nprocs=world, join=True)


def test_ep2_small():
    _run(2, dict(E=8, K=2, H=512, I=256, tokens=[128, 128], seed=20, variant="staged"))


def test_ep2_small_fused_variant():
    _run(2, dict(E=8, K=2, H=512, I=256, tokens=[128, 100], seed=20, variant="fused"))


def test_ep2_dsv4_shaped_fused_variant():
    _run(2, dict(E=32, K=6, H=4096, I=2048, tokens=[300, 256], seed=23, variant="fused"))


def test_ep8_decode_shaped_fused_variant():
    _run(8, dict(E=64, K=6, H=1024, I=512, tokens=[128, 0, 64, 128, 1, 17, 96, 128], seed=26, variant="fused"))


def test_ep2_uneven_tokens_invalid_routes_clamp():
    _run(2, dict(E=16, K=4, H=512, I=256, tokens=[133, 7], seed=21, invalid=0.2, clamp=10.0))


def test_ep2_one_rank_without_tokens():
    _run(2, dict(E=8, K=2, H=512, I=256, tokens=[0, 200], seed=22))


def test_ep2_dsv4_shaped():
    _run(2, dict(E=32, K=6, H=4096, I=2048, tokens=[300, 256], seed=23))


def test_ep4_skewed():
    _run(4, dict(E=32, K=6, H=1024, I=512, tokens=[200, 0, 77, 130], seed=24, zipf=True, variant="staged"))


def test_ep8_token_list_like_the_reference_cli():
    # the reference test's explicit per-rank list, e.g. 0,133,0,... (tests/test_mega_moe_dcu.py:405-419)
    _run(8, dict(E=64, K=6, H=1024, I=512, tokens=[0, 133, 0, 64, 128, 1, 17, 96], seed=25, variant="staged"))


def _graph_worker(rank, world, port, cfg):
    """CUDA-graph bucket replay across ranks: one capture per rank at the bucket size, replays with device-side token
    counts that differ per rank and per replay, zero included (tests/test_mega_moe_dcu.py:563-715)."""
    import torch.distributed as dist
    import megamoe
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from deepgemm_b200 import _lib
        _lib.lib().mm_set_timeouts(20000, 4000)
        E, K, H, I, bucket = cfg["E"], cfg["K"], cfg["H"], cfg["I"], cfg["bucket"]
        full = mc.make_case(world, E, K, H, I, [bucket] * world, seed=cfg["seed"])
        sb = megamoe.get_symm_buffer_for_mega_moe(dist.group.WORLD, E, bucket, K, H, I)
        l1, l2 = megamoe.transform_fp8_weights_for_mega_moe(full.w1_bf16[rank].cuda(), full.w2_bf16[rank].cuda())
        xq, xs = megamoe.cast_to_fp8_channelwise(full.x_bf16[rank].cuda())
        sb.x[:bucket].copy_(xq); sb.x_sf[:bucket].copy_(xs)
        sb.topk_idx[:bucket].copy_(full.idx[rank].cuda()); sb.topk_weights[:bucket].copy_(full.w[rank].cuda())
        y = torch.zeros((bucket, H), dtype=torch.bfloat16, device="cuda")
        flag = {"staged": dict(stages_fused_cuda_graph=True), "fused": dict(big_fused_cuda_graph=True)}[cfg["variant"]]
        megamoe.fp8_mega_moe(y, l1, l2, sb, **flag)           # warm-up outside capture (same call on every rank)
        torch.cuda.synchronize(); dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            megamoe.fp8_mega_moe(y, l1, l2, sb, **flag)
        for counts in cfg["replays"]:
            n = counts[rank]
            y.fill_(7.0)
            sb.cuda_graph_num_tokens.fill_(n)
            torch.cuda.synchronize(); dist.barrier()
            graph.replay()
            torch.cuda.synchronize()
            sb.check_status()
            case = mc.make_case(world, E, K, H, I, [bucket] * world, seed=cfg["seed"])
            for r in range(world):       # the oracle sees each rank's prefix
                case.tokens[r] = counts[r]
                for name in ("x_bf16", "x_q", "x_s", "idx", "w"):
                    getattr(case, name)[r] = getattr(case, name)[r][:counts[r]]
            ys, _, _ = mc.run_oracle(case)
            mc.assert_end_to_end_close(y[:n].cpu(), ys[rank], f"rank {rank} replay {counts}")
            assert bool((y[n:] == 7.0).all()), "rows past the device-side token count must not be written"
        sb.destroy()
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("variant", ["staged", "fused"])
def test_ep2_graph_bucket_replay_with_per_rank_token_counts(variant):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    cfg = dict(E=8, K=2, H=512, I=256, bucket=96, seed=27, variant=variant, replays=[[96, 96], [40, 77], [0, 13], [96, 0]])
    mp.spawn(_graph_worker, args=(2, _free_port(), cfg), nprocs=2, join=True)


# ------------------------------------------------------------------------------------------------------------------
# The full DSV4-Flash shape on 8 GPUs (256 experts, top-6, hidden 4096, intermediate 2048), as the reference's own test
# runs it (tests/test_mega_moe_dcu.py:405-419,729-744).  The CPU oracle cannot run 100k+ routes in test time, so each rank
# checks a handful of its tokens against the oracle run on just those tokens (a token's output depends on no other
# token; every owner evaluates the sampled routes that hit its experts, bench.parity_block), and the per-expert receive
# counts against a bincount of all ranks' indices.
def _dsv4_worker(rank, world, port, cfg):
    import torch.distributed as dist
    import megamoe
    import bench
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from deepgemm_b200 import _lib
        _lib.lib().mm_set_timeouts(20000, 4000)
        dev = torch.device("cuda", rank)
        E, K, H, I = bench.E, bench.K, bench.H, bench.I
        T, cap = cfg["tokens"], cfg["capacity"]
        group = dist.group.WORLD
        l1, l2, x, _, _ = bench.make_rank_data(rank, world, T, dev)
        g = torch.Generator(device=dev).manual_seed(3000 + rank)
        logits = torch.randn((T, E), generator=g, device=dev, dtype=torch.float32)
        if cfg.get("zipf"):
            gp = torch.Generator().manual_seed(12345)
            pop = torch.empty(E)
            pop[torch.randperm(E, generator=gp)] = torch.arange(1, E + 1, dtype=torch.float32) ** -1.1
            logits = logits + 1.5 * torch.log(pop / pop.sum()).to(dev).view(1, -1)
        sb = megamoe.get_symm_buffer_for_mega_moe(group, E, cap, K, H, I)
        megamoe.fill_inputs_from_router(sb, x, logits)
        e_loc = E // world
        stats = torch.zeros((e_loc,), dtype=torch.int32, device=dev)
        y = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device=dev)
        mc.poison_work_buffers(sb)
        megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb, cumulative_local_expert_recv_stats=stats)
        sb.check_status()
        assert not torch.isnan(y.float()).any(), f"rank {rank}: NaN in y (a row or slot was not written)"
        par = bench.parity_block(dist, group, rank, world, dev, sb, l1, l2, y, stats, T, cfg.get("samples", 4))
        assert par["counts_equal"] and par["ok"], (rank, par)
        if rank == 0:
            print(f"parity {cfg}: {par}", flush=True)
        if cfg.get("max_rows_per_expert_at_least"):
            m = torch.tensor([float(stats.max())], device=dev)
            dist.all_reduce(m, op=dist.ReduceOp.MAX)
            assert float(m) >= cfg["max_rows_per_expert_at_least"], "the skewed routing produced no hot expert"
        if cfg.get("graph_bucket"):
            # the same tokens through the fused kernel as a CUDA-graph bucket of `capacity` rows with a device-side count
            big = torch.full((cap, H), 7.0, dtype=torch.bfloat16, device=dev)
            sb.cuda_graph_num_tokens.fill_(T)
            megamoe.fp8_mega_moe(big, l1, l2, sb, big_fused_cuda_graph=True)   # warm-up outside capture
            torch.cuda.synchronize(); dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                megamoe.fp8_mega_moe(big, l1, l2, sb, big_fused_cuda_graph=True)
            big.fill_(7.0)
            torch.cuda.synchronize(); dist.barrier()
            graph.replay()
            torch.cuda.synchronize()
            sb.check_status()
            assert torch.equal(big[:T].view(torch.int16), y.view(torch.int16)), f"rank {rank}: graph replay differs from the eager call"
            assert bool((big[T:] == 7.0).all()), "rows past the device-side token count must not be written"
        sb.destroy()
    finally:
        dist.barrier()
        dist.destroy_process_group()


def _run_dsv4(cfg):
    if torch.cuda.device_count() < 8:
        pytest.skip("needs 8 GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_dsv4_worker, args=(8, _free_port(), cfg), nprocs=8, join=True)


def test_ep8_dsv4_decode_128_tokens_capacity_8192_fused_and_graph_bucket():
    """EP8 decode regime: 128 tokens per rank in a buffer of 8192 -- the fused kernel by the default rule, then replayed as
    an 8192-row CUDA-graph bucket with a device-side count of 128."""
    _run_dsv4(dict(tokens=128, capacity=8192, graph_bucket=True))


def test_ep8_dsv4_prefill_16384_tokens_zipf_staged():
    """EP8 prefill regime: 16384 tokens per rank, Zipf(1.1)-skewed routing (hot experts several times the mean load)."""
    _run_dsv4(dict(tokens=16384, capacity=16384, zipf=True, max_rows_per_expert_at_least=6000))
