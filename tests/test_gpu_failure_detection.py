"""Bounded device-side waits: a cross-rank signal that never arrives ends in an error status, not in a hang.

The failure is made benignly: rank 0 of a two-rank layout runs alone on one GPU; its peer's buffer is a second local
allocation whose signal words nothing ever writes.  Every wait gives up after the configured limit (100 ms here),
records {code, phase, rank, expected, observed} in the status words and the kernels return; the CUDA context stays
usable and a clean single-rank call succeeds afterwards.  (The reference aborts the process after 6e10 cycles:
deep_gemm/include/deep_gemm/comm/mega_moe_dcu.cuh:85-89.)
"""
import ctypes

import pytest
import torch

import moe_case as mc

pytestmark = pytest.mark.gpu


def test_missing_peer_signal_times_out_with_status_and_context_survives(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    from deepgemm_b200 import _lib
    lib = built_lib
    R, E, T, K, H, I = 2, 8, 384, 2, 512, 256
    off, nbytes = _lib.symm_buffer_layout(R, E, T, K, H, I)
    soff, sbytes = _lib.scratch_layout(R, E, T, K, H, I)
    local = torch.zeros((nbytes,), dtype=torch.int8, device="cuda")
    phantom = torch.zeros((nbytes,), dtype=torch.int8, device="cuda")   # a peer that never runs
    scratch = torch.zeros((sbytes,), dtype=torch.int8, device="cuda")
    peers = (ctypes.c_uint64 * 16)(local.data_ptr(), phantom.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.mm_init_buffers(local.data_ptr(), scratch.data_ptr(), peers, 0, R, E, T, K, H, I, stream))
    _lib.check(lib.mm_set_timeouts(100, 100))
    try:
        case = mc.make_case(1, 4, 2, H, I, [64], seed=30)      # rank 0 owns experts 0..3 of the 8
        dev = torch.device("cuda")
        import megamoe
        w1q, w2q = megamoe.pack_weights_tiled(case.w1_q[0].to(dev), "l1"), megamoe.pack_weights_tiled(case.w2_q[0].to(dev), "l2")
        w1s, w2s = case.w1_s[0].to(dev), case.w2_s[0].to(dev)
        local[off["x"]:off["x"] + 64 * H].copy_(case.x_q[0].view(torch.int8).flatten().to(dev))
        local[off["x_sf"]:off["x_sf"] + 64 * 4].view(torch.float32).copy_(case.x_s[0].to(dev))
        local[off["topk_idx"]:off["topk_idx"] + 64 * K * 8].view(torch.int64).copy_(case.idx[0].flatten().to(dev))
        local[off["topk_weights"]:off["topk_weights"] + 64 * K * 4].view(torch.float32).copy_(case.w[0].flatten().to(dev))
        y = torch.zeros((64, H), dtype=torch.bfloat16, device=dev)
        _lib.check(lib.mm_fp8_w8a8_mega_moe(y.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), None,
                                            local.data_ptr(), scratch.data_ptr(), peers, 0, R, T, 4, 64, K, H, I, float("inf"),
                                            _lib.MODE_STAGED, None, stream))
        out = (ctypes.c_int32 * 5)()
        _lib.check(lib.mm_read_status(scratch.data_ptr(), stream, out))
        assert out[0] == 1, f"expected a rank-barrier timeout status, got {list(out)}"
        assert out[1] == 0 and out[2] == 1, "the first wait to expire is the count exchange, waiting on rank 1"
        assert out[3] == 1 and out[4] == 0        # expected epoch 1, observed 0
        torch.cuda.synchronize()                   # the context is alive
    finally:
        _lib.check(lib.mm_set_timeouts(10000, 4000))
    # a clean single-rank call afterwards
    case = mc.make_case(1, 8, 2, 512, 256, [64], seed=31)
    y, _ = mc.run_cuda_rank(case, 0)
    mc.assert_layer_close(y, mc.run_oracle(case)[0][0], "call after a timed-out one")
