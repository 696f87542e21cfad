"""The reference test's SPLIT baseline rebuilt from this library's pieces on one B200
(tests/test_mega_moe_dcu.py:188-300: scatter -> grouped GEMM -> SwiGLU + quantise -> grouped GEMM -> gather), checked
piece by piece against the CPU oracle and end to end against the oracle's "staged" numerics."""
import numpy as np
import pytest
import torch

import moe_case as mc
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

K, H, I = 6, 4096, 2048          # DSV4-Flash layer dimensions


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")


def _grouped_layout(counts, gen):
    """m_indices of a contiguous layout: every expert's rows padded to 128, plus one all-padding block at the end."""
    mi = []
    for e, c in enumerate(counts):
        pad = (c + 127) // 128 * 128
        mi += [e] * c + [-1] * (pad - c)
    mi += [-1] * 128
    return torch.tensor(mi, dtype=torch.int32)


@pytest.mark.parametrize("n,k", [(512, 256), (384, 512), (4096, 2048)])
def test_m_grouped_gemm_against_fp32_reference(n, k):
    import megamoe
    g = torch.Generator().manual_seed(31)
    counts = [200, 0, 128, 1, 77, 300]
    mi = _grouped_layout(counts, g)
    rows = mi.numel()
    a = torch.randn((rows, k), generator=g)
    aq, as_ = orc.cast_to_fp8_channelwise(a.to(torch.bfloat16))
    w = (torch.randn((len(counts), n, k), generator=g) / k ** 0.5).to(torch.bfloat16)
    wq, ws = orc.cast_grouped_weight_to_fp8_channelwise(w)
    d = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    megamoe.m_grouped_fp8_gemm_nt_contiguous((aq.cuda(), as_.cuda()), (wq.cuda(), ws.cuda()), d, mi.cuda(), check=True)
    d = d.cpu()
    valid = mi >= 0
    assert bool(torch.isnan(d[~valid].float()).all()), "padding rows must be left untouched"
    ref = torch.empty((rows, n))
    for e in range(len(counts)):
        m = mi == e
        ref[m] = (aq[m].float() * as_[m].view(-1, 1)) @ (wq[e].float() * ws[e].view(-1, 1)).t()
    got = d[valid].float(); want = ref[valid]
    # fp32 accumulation in another order, then one bf16 rounding: within one bf16 ulp of the reference
    tol = want.abs() * 2.0 ** -7 + 1e-3 * want.abs().mean()
    assert bool(((got - want).abs() <= tol).all()), float(((got - want).abs() - tol).max())
    # tiled weights are accepted as they are
    d2 = torch.zeros_like(d, device="cuda")
    megamoe.m_grouped_fp8_gemm_nt_contiguous((aq.cuda(), as_.cuda()), (megamoe.pack_weights_tiled(wq.cuda(), "l2"), ws.cuda()),
                                             d2, mi.cuda())
    assert torch.equal(d2.cpu()[valid].view(torch.int16), d[valid].view(torch.int16))


def test_m_grouped_gemm_reports_a_block_that_mixes_experts():
    import megamoe
    from deepgemm_b200 import _lib
    mi = torch.tensor([0] * 100 + [1] * 28 + [1] * 128, dtype=torch.int32)     # first block holds two experts
    aq = torch.zeros((256, 128), dtype=torch.float8_e4m3fn, device="cuda")
    wq = torch.zeros((2, 128, 128), dtype=torch.float8_e4m3fn, device="cuda")
    d = torch.zeros((256, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.MegaMoeError):
        megamoe.m_grouped_fp8_gemm_nt_contiguous((aq, torch.ones(256, device="cuda")), (wq, torch.ones((2, 128), device="cuda")),
                                                 d, mi.cuda(), check=True)
    with pytest.raises(RuntimeError):       # rows not padded to 128
        megamoe.m_grouped_fp8_gemm_nt_contiguous((aq[:200], torch.ones(200, device="cuda")), (wq, torch.ones((2, 128), device="cuda")),
                                                 d[:200], mi[:200].cuda())


@pytest.mark.parametrize("clamp", [None, 10.0, 0.5])
def test_swiglu_quant_matches_the_oracle(clamp):
    from megamoe.dcu_megamoe_large_opt.K2_fused.k2_fused import swiglu_quant_channelwise_out     # the reference's import path
    g = torch.Generator().manual_seed(32)
    rows, inter = 333, 768
    x = (torch.randn((rows, 2 * inter), generator=g) * 3).to(torch.bfloat16)
    w = torch.rand((rows,), generator=g)
    w[::7] = 0.0                                    # routes without weight
    x[5] = 0                                        # an all-zero row: the 1e-4 floor
    o8 = torch.empty((rows, inter), dtype=torch.float8_e4m3fn, device="cuda")
    os_ = torch.empty((rows,), device="cuda")
    ob = torch.empty((rows, inter), dtype=torch.bfloat16, device="cuda")
    ret = swiglu_quant_channelwise_out(x.cuda(), w.cuda(), o8, os_, ob, num_per_channels=inter, output_bf16=True, clamp_value=clamp)
    assert len(ret) == 3 and ret[1].shape == (1, rows)
    aq, s2, act = orc.swiglu_quant_channelwise(x.float(), w, clamp)
    # scales: the fast exponential moves amax by a few ulp at most
    assert torch.allclose(os_.cpu(), s2, rtol=2e-6, atol=0)
    zero = w == 0
    assert bool((o8.cpu().view(torch.uint8)[zero] == 0).all()) and bool((os_.cpu()[zero] == np.float32(1e-4) / np.float32(448)).all())
    got = o8.cpu().float(); want = aq.float()
    differ = got != want
    assert float(differ.float().mean()) < 2e-3                       # rounding ties that the last ulp of exp() flips
    assert bool(((got - want).abs()[differ] <= want.abs()[differ] * 0.126 + 2 ** -9).all())     # one code step
    assert torch.allclose(ob.cpu().float(), act, rtol=2 ** -7, atol=1e-30)
    # rows whose combine pointer is 0 are skipped when no bf16 copy is requested
    o8.zero_(); os_.fill_(-1.0)
    ptrs = torch.ones((rows,), dtype=torch.int64); ptrs[10:20] = 0
    swiglu_quant_channelwise_out(x.cuda(), w.cuda(), o8, os_, None, num_per_channels=inter, clamp_value=clamp, row_combine_ptrs=ptrs.cuda())
    assert bool((os_.cpu()[10:20] == -1.0).all()) and bool((os_.cpu()[20:30] > 0).all())
    with pytest.raises(ValueError):
        swiglu_quant_channelwise_out(x.cuda(), w.cuda(), o8, os_, None, num_per_channels=inter // 2)


@pytest.mark.parametrize("shape", [(8, 2, 512, 256, 300, None), (16, 6, 4096, 2048, 256, 10.0)])
def test_split_baseline_pipeline_matches_the_staged_oracle(shape):
    """Scatter, GEMM1, SwiGLU + quantise, GEMM2, gather on one rank == the oracle's "staged" numerics, and close to the
    fused layer (whose numerics differ slightly: bf16 rounding point, clamp sidedness)."""
    import megamoe
    E, K, H, I, T, clamp = shape
    case = mc.make_case(1, E, K, H, I, [T], seed=33)
    idx, w = case.idx[0], case.w[0]
    counts = torch.bincount(idx[idx >= 0].flatten(), minlength=E)
    aligned = ((counts + 127) // 128 * 128).to(torch.int32)
    rows = int(aligned.sum())
    gx, gs, rw, mi, oi = megamoe.deepep_deepgemm_preprocess_channelwise(
        case.x_q[0].cuda(), case.x_s[0].cuda(), idx.cuda(), w.cuda(), aligned.cuda(), rows)
    l1_out = torch.empty((rows, 2 * I), dtype=torch.bfloat16, device="cuda")
    megamoe.m_grouped_fp8_gemm_nt_contiguous((gx, gs), (case.w1_q[0].cuda(), case.w1_s[0].cuda()), l1_out, mi, check=True)
    a8 = torch.empty((rows, I), dtype=torch.float8_e4m3fn, device="cuda")
    a8s = torch.empty((rows,), device="cuda")
    megamoe.swiglu_quant_channelwise_out(l1_out, rw, a8, a8s, None, num_per_channels=I, clamp_value=clamp)
    l2_out = torch.empty((rows, H), dtype=torch.bfloat16, device="cuda")
    megamoe.m_grouped_fp8_gemm_nt_contiguous((a8, a8s), (case.w2_q[0].cuda(), case.w2_s[0].cuda()), l2_out, mi)
    y = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    megamoe.deepep_deepgemm_postprocess_channelwise(y, l2_out, idx.cuda(), w.cuda(), oi, apply_topk_weights=False)
    ys, _, _ = mc.run_oracle(case, clamp, "staged")
    mc.assert_end_to_end_close(y.cpu(), ys[0], "split baseline vs staged oracle")
    y_fused, _ = mc.run_cuda_rank(case, 0, clamp=clamp)
    _, cos = orc.parity_metrics(y.cpu(), y_fused)
    assert cos > 0.999, cos


def test_layer_against_split_baseline_with_the_reference_tests_recipe():
    """The reference's own correctness check (tests/test_mega_moe_dcu.py:484-497, 729-744): inputs N(0,1) * 0.05,
    weights N(0,1) * 0.05, unsorted top-k of random scores with a softmax over the selected scores, clamp 10, the layer
    against the split baseline: max |difference| <= 0.0035 (its --atol) and identical per-expert receive statistics on top
    of a random initial value."""
    import megamoe
    E, T = 16, 512
    g = torch.Generator(device="cuda").manual_seed(41)
    x = torch.randn((T, H), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16) * 0.05
    w1 = torch.randn((E, 2 * I, H), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16) * 0.05
    w2 = torch.randn((E, H, I), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16) * 0.05
    scores = torch.randn((T, E), generator=g, device="cuda")
    tw, ti = torch.topk(scores, K, dim=-1, largest=True, sorted=False)
    tw = torch.softmax(tw.float(), dim=-1)
    xq, xs = megamoe.cast_to_fp8_channelwise(x)
    l1, l2 = megamoe.transform_fp8_weights_for_mega_moe(w1, w2, layout="native")
    stats0 = torch.randint(0, 100, (E,), dtype=torch.int32, device="cuda")

    # fused layer
    sb = megamoe.get_symm_buffer_for_mega_moe(None, E, T, K, H, I)
    sb.x[:T].copy_(xq); sb.x_sf[:T].copy_(xs); sb.topk_idx[:T].copy_(ti); sb.topk_weights[:T].copy_(tw)
    y = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    stats = stats0.clone()
    megamoe.fp8_mega_moe(y, l1, l2, sb, cumulative_local_expert_recv_stats=stats, activation_clamp=10.0)
    sb.check_status()

    # split baseline (tests/test_mega_moe_dcu.py:188-300 without the DeepEP transport, which is the identity on one rank)
    counts = torch.bincount(ti.flatten(), minlength=E)
    aligned = ((counts + 127) // 128 * 128).to(torch.int32)
    rows = int(aligned.sum())
    gx, gs, rw, mi, oi = megamoe.deepep_deepgemm_preprocess_channelwise(xq, xs, ti, tw, aligned, rows)
    l1_out = torch.empty((rows, 2 * I), dtype=torch.bfloat16, device="cuda")
    megamoe.m_grouped_fp8_gemm_nt_contiguous((gx, gs), l1, l1_out, mi)
    a8 = torch.empty((rows, I), dtype=torch.float8_e4m3fn, device="cuda"); a8s = torch.empty((rows,), device="cuda")
    l2_out = torch.empty((rows, H), dtype=torch.bfloat16, device="cuda")
    megamoe.swiglu_quant_channelwise_out(l1_out, rw, a8, a8s, l2_out, num_per_channels=I, output_bf16=False, clamp_value=10.0)
    megamoe.m_grouped_fp8_gemm_nt_contiguous((a8, a8s), l2, l2_out, mi)
    y_base = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    megamoe.deepep_deepgemm_postprocess_channelwise(y_base, l2_out, ti, tw, oi, apply_topk_weights=False)
    stats_base = stats0 + counts.to(torch.int32)

    diff = (y.float() - y_base.float()).abs()
    assert float(diff.max()) <= 0.0035, float(diff.max())
    assert torch.equal(stats, stats_base)
    assert float(y_base.float().abs().max()) > 0.01            # the tolerance is not vacuous
    sb.destroy()
