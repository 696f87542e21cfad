"""Full-size parity on one B200: the DSV4-Flash-shaped layer (256 experts, top-6, hidden 4096, intermediate 2048, 4096
tokens, EP1 -- the benchmark workload).  The CPU oracle cannot run all of it in seconds, so the checks are
  * bit-exact integer results against torch on the device: per-expert receive counts == bincount, every token->slot
    entry unique and inside its expert's segment, segments aligned to 128 rows;
  * size-independent properties of the outputs: doubling all route weights doubles y bit for bit, permuting the tokens
    permutes y bit for bit, a second call reproduces the first;
  * the oracle on a SAMPLE: all rows routed to four experts are recomputed on the CPU from the quantised inputs and
    compared, route by route, with what the CUDA path stored in the combine buffer.
"""
import numpy as np
import pytest
import torch

import moe_case as mc
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

E, K, H, I, T = 256, 6, 4096, 2048, 4096


def _make():
    import megamoe
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(7)
    l1q = torch.empty((E, I // 128, H // 128, 256, 128), dtype=torch.float8_e4m3fn, device=dev)
    l1s = torch.empty((E, 2 * I), dtype=torch.float32, device=dev)
    l2q = torch.empty((E, H // 256, I // 128, 256, 128), dtype=torch.float8_e4m3fn, device=dev)
    l2s = torch.empty((E, H), dtype=torch.float32, device=dev)
    for e0 in range(0, E, 32):
        w1 = (torch.randn((32, 2 * I, H), generator=g, device=dev) / H ** 0.5).to(torch.bfloat16)
        w2 = (torch.randn((32, H, I), generator=g, device=dev) / I ** 0.5).to(torch.bfloat16)
        (a, as_), (b, bs_) = megamoe.transform_fp8_weights_for_mega_moe(w1, w2)
        l1q[e0:e0 + 32], l1s[e0:e0 + 32], l2q[e0:e0 + 32], l2s[e0:e0 + 32] = a, as_, b, bs_
        del w1, w2, a, b
    x = torch.randn((T, H), generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn((T, E), generator=g, device=dev)
    return (l1q, l1s), (l2q, l2s), x, logits


def test_dsv4_flash_ep1_4096_tokens():
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    import megamoe
    l1, l2, x, logits = _make()
    sb = megamoe.get_symm_buffer_for_mega_moe(None, E, T, K, H, I)
    megamoe.fill_inputs_from_router(sb, x, logits)
    idx = sb.topk_idx[:T].clone(); w = sb.topk_weights[:T].clone()
    stats = torch.zeros((E,), dtype=torch.int32, device="cuda")
    y = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb, cumulative_local_expert_recv_stats=stats)
    sb.check_status()

    # ---- routing layout, bit-exact against torch on the device
    counts = torch.bincount(idx.flatten(), minlength=E).to(torch.int32)
    assert torch.equal(stats, counts)
    off = sb.scratch_view("expert_off", (E,), torch.int32)
    padded = (counts + 127) // 128 * 128
    assert torch.equal(off, (torch.cumsum(padded, 0) - padded).to(torch.int32))
    dest = sb.scratch_view("dest_row", (sb.num_max_tokens_per_rank, K), torch.int32)[:T]
    flat = dest.flatten().long()
    assert flat.unique().numel() == T * K
    e_flat = idx.flatten()
    assert bool(((flat >= off[e_flat].long()) & (flat < (off[e_flat] + counts[e_flat]).long())).all())
    # rows of one expert are in (token, slot) order: the row index grows with the route index inside each expert
    order = torch.argsort(e_flat * (T * K) + torch.arange(T * K, device="cuda"))
    same = e_flat[order][1:] == e_flat[order][:-1]
    assert bool((flat[order][1:][same] > flat[order][:-1][same]).all())

    # ---- sampled oracle: every row of four experts, compared per route through the combine buffer
    comb = sb.symm_view("combine", (sb.num_max_tokens_per_rank, K, H), torch.bfloat16)
    xq, xs = sb.x[:T].cpu(), sb.x_sf[:T].cpu()
    idx_c, w_c = idx.cpu(), w.cpu()
    for e in (0, 77, 130, 255):
        tt, kk = torch.nonzero(idx_c == e, as_tuple=True)
        w1 = megamoe.unpack_weights_tiled(l1[0][e:e + 1], "l1", 2 * I)[0].cpu().float() * l1[1][e].cpu().view(-1, 1)
        w2 = megamoe.unpack_weights_tiled(l2[0][e:e + 1], "l2", H)[0].cpu().float() * l2[1][e].cpu().view(-1, 1)
        a = xq[tt].float() * xs[tt].view(-1, 1)
        gu = a @ w1.t()
        g_, u_ = gu[:, :I], gu[:, I:]
        act = (g_ * torch.sigmoid(g_) * u_ * w_c[tt, kk].view(-1, 1)).to(torch.bfloat16).float()
        s2 = (act.abs().amax(dim=1) / 448.0).clamp(min=1e-4)
        aq = (act * (1.0 / s2).view(-1, 1)).to(torch.float8_e4m3fn).float()
        ref = ((aq * s2.view(-1, 1)) @ w2.t()).to(torch.bfloat16)
        got = comb[tt.cuda(), kk.cuda()].cpu()
        mc.assert_end_to_end_close(got, ref, f"routes of expert {e}")

    # ---- size-independent properties
    y1 = y.clone()
    megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb)
    assert torch.equal(y.view(torch.int16), y1.view(torch.int16)), "a second call differs"
    sb.topk_weights[:T].copy_(w * 2)
    megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb)
    assert torch.equal(y.view(torch.int16), (y1.float() * 2).to(torch.bfloat16).view(torch.int16)), "doubling the weights"
    perm = torch.randperm(T, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    sb.x[:T].copy_(sb.x[:T][perm].clone()); sb.x_sf[:T].copy_(sb.x_sf[:T][perm].clone())
    sb.topk_idx[:T].copy_(idx[perm]); sb.topk_weights[:T].copy_(w[perm])
    megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb)
    sb.check_status()
    assert torch.equal(y.view(torch.int16), y1[perm].view(torch.int16)), "permuting the tokens"
    assert not torch.isnan(y.float()).any()
    sb.destroy()


def test_large_token_count_offsets_beyond_4_gib():
    """131072 tokens x top-6 on 32 DSV4-shaped experts: 786k pool rows, so the byte offsets into the pool (3.2 GB), the
    bf16 activations (3.2 GB) and the combine buffer (6.4 GB) pass 2^31 and 2^32.  Counts are checked bit-exactly against
    torch; the outputs of sampled tokens (first, last, random) against the CPU oracle run on just those tokens -- a
    token's output does not depend on the other tokens."""
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    import megamoe
    e, t = 32, 131072
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(9)
    w1 = (torch.randn((e, 2 * I, H), generator=g, device=dev) / H ** 0.5).to(torch.bfloat16)
    w2 = (torch.randn((e, H, I), generator=g, device=dev) / I ** 0.5).to(torch.bfloat16)
    l1, l2 = megamoe.transform_fp8_weights_for_mega_moe(w1, w2)
    del w1, w2
    sb = megamoe.get_symm_buffer_for_mega_moe(None, e, t, K, H, I)
    for t0 in range(0, t, 16384):                                     # fill in slices to bound the temporaries
        x = torch.randn((16384, H), generator=g, device=dev).to(torch.bfloat16)
        logits = torch.randn((16384, e), generator=g, device=dev)
        xq, xs = megamoe.cast_to_fp8_channelwise(x)
        wts, idx = torch.topk(torch.softmax(logits, dim=-1), K, dim=-1)
        sb.x[t0:t0 + 16384].copy_(xq); sb.x_sf[t0:t0 + 16384].copy_(xs)
        sb.topk_idx[t0:t0 + 16384].copy_(idx); sb.topk_weights[t0:t0 + 16384].copy_(wts / wts.sum(-1, keepdim=True))
        del x, logits, xq, xs
    stats = torch.zeros((e,), dtype=torch.int32, device=dev)
    y = torch.full((t, H), float("nan"), dtype=torch.bfloat16, device=dev)
    megamoe.fp8_w8a8_mega_moe(y, l1, l2, sb, cumulative_local_expert_recv_stats=stats)
    sb.check_status()
    assert torch.equal(stats, torch.bincount(sb.topk_idx[:t].flatten(), minlength=e).to(torch.int32))
    assert int(stats.sum()) == t * K and not torch.isnan(y.float()).any()
    dest = sb.scratch_view("dest_row", (sb.num_max_tokens_per_rank, K), torch.int32)[:t]
    assert dest.flatten().long().unique().numel() == t * K and int(dest.max()) * H > 2 ** 31

    pick = torch.cat([torch.arange(16), torch.arange(t - 16, t),
                      torch.randint(0, t, (32,), generator=torch.Generator().manual_seed(3))]).to(dev)
    w1p = megamoe.unpack_weights_tiled(l1[0], "l1", 2 * I).cpu()
    w2p = megamoe.unpack_weights_tiled(l2[0], "l2", H).cpu()
    ys, _, _ = orc.moe_layer([sb.x[pick].cpu()], [sb.x_sf[pick].cpu()], [sb.topk_idx[pick].cpu()], [sb.topk_weights[pick].cpu()],
                             [w1p], [l1[1].cpu()], [w2p], [l2[1].cpu()], e, None, "fused")
    mc.assert_end_to_end_close(y[pick].cpu(), ys[0], "sampled tokens of the 131072-token call")
    sb.destroy()
