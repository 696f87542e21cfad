"""Routing layout: the vectorised restatement against the plain C restatement, and its invariants."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc


def _routing(R, E, K, tokens, seed, invalid=0.0, zipf=False):
    idx, w = [], []
    for r in range(R):
        i_, w_ = orc.make_routing(tokens[r], E, K, seed=seed + r, zipf=zipf)
        if invalid and tokens[r]:
            g = torch.Generator().manual_seed(seed + 50 + r)
            m = torch.rand(i_.shape, generator=g)
            i_ = torch.where(m < invalid / 3, torch.full_like(i_, -1), i_)
            i_ = torch.where((m >= invalid / 3) & (m < 2 * invalid / 3), torch.full_like(i_, E + 3), i_)
            w_ = torch.where((m >= 2 * invalid / 3) & (m < invalid), torch.zeros_like(w_), w_)
        idx.append(i_.numpy()); w.append(w_.numpy())
    return idx, w


@pytest.mark.parametrize("R,E,K,tokens,invalid,zipf", [
    (1, 8, 2, [256], 0.0, False),
    (2, 8, 2, [100, 37], 0.2, False),
    (4, 32, 6, [0, 133, 0, 64], 0.1, True),
    (8, 256, 6, [128] * 8, 0.0, False),
    (8, 256, 6, [17, 0, 300, 1, 0, 5, 64, 2], 0.3, True),
    (1, 4, 4, [0], 0.0, False),
])
def test_numpy_layout_matches_c(R, E, K, tokens, invalid, zipf):
    idx, w = _routing(R, E, K, tokens, 7, invalid, zipf)
    lay = orc.route_layout(idx, w, E)
    counts, totals, pool_off, dest = orc.c_route_layout(idx, w, E)
    assert np.array_equal(lay.counts, counts)
    assert np.array_equal(lay.totals, totals)
    assert np.array_equal(lay.pool_off, pool_off)
    for r in range(R):
        assert np.array_equal(lay.dest_row[r], dest[r])


def test_layout_invariants():
    R, E, K = 4, 32, 6
    idx, w = _routing(R, E, K, [200, 0, 77, 130], 11, 0.15, True)
    lay = orc.route_layout(idx, w, E)
    E_loc = E // R
    # counts follow the reference's bincount rule over valid routes (tests/test_mega_moe_dcu.py:310-316)
    for r in range(R):
        v = (idx[r] >= 0) & (idx[r] < E) & (w[r] != 0)
        assert np.array_equal(lay.counts[r], np.bincount(idx[r][v], minlength=E))
        assert np.all((lay.dest_row[r] >= 0) == v)
    for o in range(R):
        rows = np.concatenate([lay.dest_row[r][(idx[r] // E_loc == o) & (lay.dest_row[r] >= 0)] for r in range(R)])
        assert len(np.unique(rows)) == len(rows)                       # a pool row is used once
        assert lay.pool_rows[o] % 128 == 0
        for le in range(E_loc):
            e = o * E_loc + le
            assert lay.pool_off[e] % 128 == 0
            seg = np.sort(rows[(rows >= lay.pool_off[e]) & (rows < lay.pool_off[e] + lay.totals[e])])
            assert np.array_equal(seg, np.arange(lay.pool_off[e], lay.pool_off[e] + lay.totals[e]))
        # rows of one expert are ordered by (source rank, token, slot)
        sr, st, ss = lay.row_src_rank[o], lay.row_src_token[o], lay.row_src_slot[o]
        for le in range(E_loc):
            e = o * E_loc + le
            s = slice(lay.pool_off[e], lay.pool_off[e] + lay.totals[e])
            key = sr[s].astype(np.int64) * 10 ** 9 + st[s].astype(np.int64) * 100 + ss[s]
            assert np.all(np.diff(key) > 0)


def test_empty_ranks_and_all_invalid():
    idx = [np.zeros((0, 2), np.int64), np.full((5, 2), -1, np.int64)]
    w = [np.zeros((0, 2), np.float32), np.ones((5, 2), np.float32)]
    lay = orc.route_layout(idx, w, 4)
    assert lay.totals.sum() == 0 and lay.pool_rows == [0, 0]
    assert np.all(lay.dest_row[1] == -1)
