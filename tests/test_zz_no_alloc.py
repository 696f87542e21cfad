"""mm_fp8_w8a8_mega_moe_static -- the layer for callers that may not allocate device memory.

A serving process that gave all of its HBM to its own arena, or a code path where cudaMalloc (which synchronises the
whole device) is off limits, cannot provide the two work buffers the regular entry point needs.  The static variant
keeps them in a fixed-size device array inside the library.  This test calls it through the C ABI with nothing but
input and output pointers and requires the same bits as the regular entry point, on two calls in a row with
different shapes (the second call finds the first call's leftovers in the shared work area), and checks that a shape
that does not fit is refused with a message instead of overrunning the area.

Collected last on purpose: a failure here cannot hide results of the other tests in a stop-at-first-failure run.
"""
import ctypes

import pytest
import torch

import moe_case as mc

pytestmark = pytest.mark.gpu


def _static_call(lib, case, clamp):
    import megamoe
    from deepgemm_b200 import _lib
    dev = torch.device("cuda")
    T = case.tokens[0]
    (w1, s1), (w2, s2) = megamoe.transform_fp8_weights_for_mega_moe(case.w1_bf16[0].to(dev), case.w2_bf16[0].to(dev))
    xq, xs = megamoe.cast_to_fp8_channelwise(case.x_bf16[0].to(dev))
    idx, w = case.idx[0].to(dev).contiguous(), case.w[0].to(dev).contiguous()
    y = torch.full((T, case.H), float("nan"), dtype=torch.bfloat16, device=dev)
    stats = torch.zeros((case.E,), dtype=torch.int32, device=dev)
    _lib.check(lib.mm_fp8_w8a8_mega_moe_static(
        y.data_ptr(), xq.data_ptr(), xs.data_ptr(), idx.data_ptr(), w.data_ptr(), w1.data_ptr(), s1.data_ptr(), w2.data_ptr(),
        s2.data_ptr(), stats.data_ptr(), T, case.E, case.K, case.H, case.I, float("inf") if clamp is None else clamp,
        torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    out = (ctypes.c_int32 * 5)()
    _lib.check(lib.mm_fp8_w8a8_mega_moe_static_status(torch.cuda.current_stream().cuda_stream, out))
    assert out[0] == 0, f"a bounded wait expired inside the static call: {list(out)}"
    return y.cpu(), stats.cpu()


def test_static_work_area_variant_matches_regular_entry_point(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    cases = [(mc.make_case(1, 8, 2, 512, 256, [256], seed=40), None),
             (mc.make_case(1, 4, 3, 384, 128, [77], seed=41, invalid_fraction=0.2), 10.0)]
    for case, clamp in cases:
        stats_ref = torch.zeros((case.E,), dtype=torch.int32, device="cuda")
        y_ref, _ = mc.run_cuda_rank(case, 0, clamp=clamp, stats=stats_ref)           # regular entry point, own buffers
        y, stats = _static_call(built_lib, case, clamp)                               # static work area, no buffers
        assert torch.equal(y.view(torch.int16), y_ref.view(torch.int16)), "static variant differs from the regular entry point"
        assert torch.equal(stats, stats_ref.cpu())
        mc.assert_layer_close(y, mc.run_oracle(case, clamp)[0][0], "static variant vs oracle")


def test_static_variant_leaves_free_device_memory_unchanged(built_lib):
    """What the entry point is for: a caller whose arena owns all of HBM.  Once the kernels' code is resident (first
    call), further calls must not take or give back a single byte of device memory."""
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    import megamoe
    from deepgemm_b200 import _lib
    dev = torch.device("cuda")
    case = mc.make_case(1, 8, 2, 512, 256, [200], seed=42)
    (w1, s1), (w2, s2) = megamoe.transform_fp8_weights_for_mega_moe(case.w1_bf16[0].to(dev), case.w2_bf16[0].to(dev))
    xq, xs = megamoe.cast_to_fp8_channelwise(case.x_bf16[0].to(dev))
    idx, w = case.idx[0].to(dev).contiguous(), case.w[0].to(dev).contiguous()
    y = torch.empty((200, case.H), dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        _lib.check(built_lib.mm_fp8_w8a8_mega_moe_static(
            y.data_ptr(), xq.data_ptr(), xs.data_ptr(), idx.data_ptr(), w.data_ptr(), w1.data_ptr(), s1.data_ptr(), w2.data_ptr(),
            s2.data_ptr(), None, 200, case.E, case.K, case.H, case.I, float("inf"), stream))
        torch.cuda.synchronize()

    call()                                              # loads the kernels' code, resolves the work area's address
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory changed across static calls: {free_before} -> {free_after}"
    y_ref, _ = mc.run_cuda_rank(case, 0)                 # regular entry point with its own buffers: the same bits
    assert torch.equal(y.cpu().view(torch.int16), y_ref.view(torch.int16)), "static variant differs from the regular entry point"


def test_static_variant_refuses_shapes_beyond_its_work_area(built_lib):
    dummy = ctypes.c_void_p(256)
    rc = built_lib.mm_fp8_w8a8_mega_moe_static(dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy, None,
                                               4096, 256, 6, 4096, 2048, float("inf"), None)
    assert rc != 0
    msg = built_lib.mm_last_error().decode()
    assert "work memory" in msg and "mm_fp8_w8a8_mega_moe" in msg
