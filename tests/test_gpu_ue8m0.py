"""The UE8M0 recipe (recipe=megamoe.RECIPE_UE8M0_PER32) against the CPU oracle's "ue8m0" variant.

The activation recipe of the reference's Blackwell Mega MoE kernel -- e4m3 codes with one power-of-two scale per
(row, 32 columns), produced in the GEMM1 tile and applied by a block-scaled MMA in GEMM2
(deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:839-870,1023-1057) -- with FP8 weights and channelwise weight
scales.  Checked stage by stage, like the channelwise recipe:
  * codes and scale bytes the GEMM1 epilogue wrote: equal to the oracle's on all but a few blocks (a block scale flips when
    the block's amax sits on a power-of-two boundary and the two GEMM1 sums differ in the last bit);
  * GEMM2 + combine, isolated: the oracle's tail fed with the CUDA path's own codes and scale bytes, literal bar;
  * end to end against the oracle.
"""
import numpy as np
import pytest
import torch

import moe_case as mc
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu


def _cuda_codes_and_scales(sb, case, n):
    """FP8 codes [n, I] and scale bytes [n, I / 32] as the GEMM1 epilogue left them in the scratch buffer."""
    I = case.I
    q = sb.scratch_view("act_fp8", (sb.pool_rows, I), torch.uint8)[:n].cpu()
    atoms = sb.scratch_view("act_sf", (sb.pool_rows // 128, I // 128, 32, 4, 4), torch.uint8)[:n // 128].cpu()
    # atom byte (r0, r1, kb) belongs to row r1 * 32 + r0 of the m-block and to column block 4 * stage + kb
    sf = atoms.permute(0, 3, 2, 1, 4).reshape(n, I // 32)
    return q, sf


def _check(case, clamp=None):
    import megamoe
    ys, lay, _ = mc.run_oracle(case, clamp, "ue8m0", trace=True)
    y, sb = mc.run_cuda_rank(case, 0, clamp=clamp, keep=True, recipe=megamoe.RECIPE_UE8M0_PER32)
    try:
        n = lay.pool_rows[0]
        valid = np.nonzero(lay.row_src_rank[0] >= 0)[0]
        vr = torch.from_numpy(valid)
        q, sf = _cuda_codes_and_scales(sb, case, n)
        # ---- GEMM1 + quantisation against the oracle's codes and scale bytes
        H, I, K = case.H, case.I, case.K
        st, ss = lay.row_src_token[0], lay.row_src_slot[0]
        ref_q = torch.zeros((n, I), dtype=torch.uint8); ref_sf = torch.zeros((n, I // 32), dtype=torch.uint8)
        comb = torch.zeros((K, case.tokens[0], H))
        for e in range(case.E):
            cnt = int(lay.totals[e])
            if not cnt:
                continue
            rows = np.arange(lay.pool_off[e], lay.pool_off[e] + cnt)
            ri = torch.from_numpy(rows)
            tt = torch.from_numpy(st[rows].astype(np.int64)); kk = torch.from_numpy(ss[rows].astype(np.int64))
            a = case.x_q[0][tt].float() * case.x_s[0][tt].view(-1, 1)
            gu = a @ (case.w1_q[0][e].float() * case.w1_s[0][e].view(-1, 1)).t()
            g, u = gu[:, :I], gu[:, I:]
            if clamp is not None:
                g = g.clamp(-clamp, clamp); u = u.clamp(-clamp, clamp)
            act = g * torch.sigmoid(g) * u * case.w[0][tt, kk].view(-1, 1)
            rq, rsf = orc.ue8m0_block_quant(act)
            ref_q[ri] = rq.view(torch.uint8); ref_sf[ri] = rsf
            # ---- GEMM2 + combine of the oracle, fed with the CUDA path's codes and scale bytes
            a2 = (q[ri].view(torch.float8_e4m3fn).float().reshape(cnt, I // 32, 32) * orc.ue8m0_to_float(sf[ri]).unsqueeze(2)).reshape(cnt, I)
            out = ((a2 @ case.w2_q[0][e].float().t()) * case.w2_s[0][e].view(1, -1)).to(torch.bfloat16).float()
            comb[kk, tt] = out
        if valid.size:
            sf_mismatch = (sf[vr] != ref_sf[vr]).float().mean().item()
            assert sf_mismatch < 2e-3, f"scale bytes differ from the oracle on {sf_mismatch:.2%} of the blocks"
            same = (sf[vr] == ref_sf[vr]).repeat_interleave(32, dim=1)
            q_mismatch = ((q[vr] != ref_q[vr]) & same).float().mean().item()
            assert q_mismatch < 2e-2, f"FP8 codes differ from the oracle on {q_mismatch:.2%} of the elements with equal scales"
            y_tail = comb.sum(dim=0).to(torch.bfloat16)
            mc.assert_layer_close(y, y_tail, "UE8M0 GEMM2 + combine")
        mc.assert_end_to_end_close(y, ys[0], "UE8M0 end to end")
        return y
    finally:
        sb.destroy()


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; run them with -m gpu on a B200")


def test_ue8m0_small_config():
    _check(mc.make_case(1, 8, 2, 512, 256, [256], seed=0))


def test_ue8m0_invalid_routes_clamp_and_ragged_blocks():
    _check(mc.make_case(1, 8, 4, 384, 384, [201], seed=50, invalid_fraction=0.2), clamp=10.0)


def test_ue8m0_dsv4_shaped_slice():
    _check(mc.make_case(1, 16, 6, 4096, 2048, [512], seed=51))


def test_ue8m0_is_deterministic_and_differs_from_the_channelwise_recipe():
    import megamoe
    case = mc.make_case(1, 8, 2, 512, 256, [200], seed=52)
    a, sb = mc.run_cuda_rank(case, 0, keep=True, recipe=megamoe.RECIPE_UE8M0_PER32)
    b, _ = mc.run_cuda_rank(case, 0, sb=sb, recipe=megamoe.RECIPE_UE8M0_PER32)
    c, _ = mc.run_cuda_rank(case, 0, sb=sb)
    sb.destroy()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert not torch.equal(a.view(torch.int16), c.view(torch.int16))
    err, cos = orc.parity_metrics(a, c)
    assert cos > 0.995, (err, cos)
