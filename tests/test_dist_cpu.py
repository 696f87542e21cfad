"""Multi-process host logic on CPU (gloo, world size 2): handle exchange order, and the rank-sharded view of the
routing plan -- every rank derives the same plan from the all-gathered count vectors, which is what the device-side
count exchange relies on."""
import os
import socket
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    from deepgemm_b200.megamoe import _gather_handles
    from oracle import moe_oracle as orc
    group = dist.group.WORLD
    handles = _gather_handles(group, bytes([rank]) * 64)
    assert [h[0] for h in handles] == list(range(world)) and all(len(h) == 64 for h in handles)
    # each rank only knows its own routing; the plan must come out identical everywhere
    E, K, T = 16, 4, [50, 13][rank]
    idx, w = orc.make_routing(T, E, K, seed=40 + rank)
    mine = np.bincount(idx.numpy().ravel(), minlength=E).astype(np.int64)
    gathered = [torch.zeros(E, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(mine))
    counts = torch.stack(gathered).numpy()
    totals = counts.sum(0)
    padded = (totals + 127) // 128 * 128
    e_loc = E // world
    pool_off = np.concatenate([np.concatenate([[0], np.cumsum(padded[o * e_loc:(o + 1) * e_loc])[:-1]]) for o in range(world)])
    dest_base = pool_off + counts[:rank].sum(0)
    # compare with the full-knowledge oracle (both ranks' routing regenerated locally)
    all_idx, all_w = zip(*[orc.make_routing([50, 13][r], E, K, seed=40 + r) for r in range(world)])
    lay = orc.route_layout([i.numpy() for i in all_idx], [x.numpy() for x in all_w], E)
    assert np.array_equal(lay.counts, counts) and np.array_equal(lay.pool_off, pool_off)
    first_rows = np.array([lay.dest_row[rank][idx.numpy() == e].min() if (idx.numpy() == e).any() else -1 for e in range(E)])
    has = first_rows >= 0
    assert np.array_equal(first_rows[has], dest_base[has])
    q.put((rank, pool_off.tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_world2_handle_exchange_and_plan_agreement():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = dict(q.get() for _ in range(2))
    assert got[0] == got[1]


def test_reference_arm_prints_one_line_on_rank0_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "0"], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip() == ""
