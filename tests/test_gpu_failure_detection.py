"""Bounded device-side waits: a cross-rank signal that never arrives ends in an error status, not in a hang.

The failure is made benignly: rank 0 of a two-rank layout runs alone on one GPU; its peer's buffer is a second local
allocation whose signal words nothing ever writes.  Every wait gives up after the configured limit (100 ms here),
records {code, phase, rank, expected, observed} in the status words and the kernels return; every later launch of the
call sees the status and returns at once, so y and the local combine buffer stay untouched; the CUDA context stays
usable and a clean single-rank call succeeds afterwards.  (The reference aborts the process after 6e10 cycles:
deep_gemm/include/deep_gemm/comm/mega_moe_dcu.cuh:85-89.)
"""
import ctypes

import pytest
import torch

import moe_case as mc

pytestmark = pytest.mark.gpu

R, E, T, K, H, I = 2, 8, 384, 2, 512, 256
BAR_COUNTS, BAR_DISPATCH, BAR_COMBINE = 0, 1, 2
LIBRARY_DEFAULT_TIMEOUTS = (30000, 4000)


class _PhantomPeer:
    """Rank 0 of a two-rank layout with a peer that never runs."""

    def __init__(self, lib):
        from deepgemm_b200 import _lib
        import megamoe
        self.lib, self._lib = lib, _lib
        self.off, nbytes = _lib.symm_buffer_layout(R, E, T, K, H, I)
        _, sbytes = _lib.scratch_layout(R, E, T, K, H, I)
        self.local = torch.zeros((nbytes,), dtype=torch.int8, device="cuda")
        self.phantom = torch.zeros((nbytes,), dtype=torch.int8, device="cuda")
        self.scratch = torch.zeros((sbytes,), dtype=torch.int8, device="cuda")
        self.peers = (ctypes.c_uint64 * 16)(self.local.data_ptr(), self.phantom.data_ptr())
        self.stream = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.mm_init_buffers(self.local.data_ptr(), self.scratch.data_ptr(), self.peers, 0, R, E, T, K, H, I, self.stream))
        case = mc.make_case(1, 4, 2, H, I, [64], seed=30)      # rank 0 owns experts 0..3 of the 8
        dev = torch.device("cuda")
        self.w1q = megamoe.pack_weights_tiled(case.w1_q[0].to(dev), "l1"); self.w2q = megamoe.pack_weights_tiled(case.w2_q[0].to(dev), "l2")
        self.w1s, self.w2s = case.w1_s[0].to(dev), case.w2_s[0].to(dev)
        off = self.off
        self.local[off["x"]:off["x"] + 64 * H].copy_(case.x_q[0].view(torch.int8).flatten().to(dev))
        self.local[off["x_sf"]:off["x_sf"] + 64 * 4].view(torch.float32).copy_(case.x_s[0].to(dev))
        self.local[off["topk_idx"]:off["topk_idx"] + 64 * K * 8].view(torch.int64).copy_(case.idx[0].flatten().to(dev))
        self.local[off["topk_weights"]:off["topk_weights"] + 64 * K * 4].view(torch.float32).copy_(case.w[0].flatten().to(dev))
        self.combine = self.local[off["combine"]:off["combine"] + K * T * H * 2].view(torch.int16)
        self.combine.fill_(0x1234)
        self.y = torch.full((64, H), 7.0, dtype=torch.bfloat16, device=dev)

    def pretend_peer_signalled(self, bar):
        """Write a far-future epoch into the local slot of barrier `bar` for rank 1, as if the peer had arrived there
        (its count-matrix row stays zero: it sends no rows)."""
        slot = self.off["signals"] + (bar * 16 + 1) * 4
        self.local[slot:slot + 4].view(torch.int32).fill_(1 << 20)

    def call(self, mode):
        self._lib.check(self.lib.mm_fp8_w8a8_mega_moe(
            self.y.data_ptr(), self.w1q.data_ptr(), self.w1s.data_ptr(), self.w2q.data_ptr(), self.w2s.data_ptr(), None,
            self.local.data_ptr(), self.scratch.data_ptr(), self.peers, 0, R, T, 4, 64, K, H, I, float("inf"), mode, None, self.stream))
        out = (ctypes.c_int32 * 5)()
        self._lib.check(self.lib.mm_read_status(self.scratch.data_ptr(), self.stream, out))
        torch.cuda.synchronize()                   # the context is alive
        return list(out)

    def assert_outputs_untouched(self):
        assert bool((self.y == 7.0).all()), "y was written after a bounded wait had expired"
        assert bool((self.combine == 0x1234).all()), "the local combine buffer was written after a bounded wait had expired"


@pytest.fixture()
def short_timeouts(built_lib):
    from deepgemm_b200 import _lib
    _lib.check(built_lib.mm_set_timeouts(100, 100))
    yield built_lib
    _lib.check(built_lib.mm_set_timeouts(*LIBRARY_DEFAULT_TIMEOUTS))


def _clean_call_afterwards():
    case = mc.make_case(1, 8, 2, 512, 256, [64], seed=31)
    y, _ = mc.run_cuda_rank(case, 0)
    mc.assert_layer_close(y, mc.run_oracle(case)[0][0], "call after a timed-out one")


@pytest.mark.parametrize("mode_name", ["staged", "split", "fused"])
def test_missing_peer_counts_time_out_with_status_and_nothing_is_written(short_timeouts, mode_name):
    """The first cross-rank wait of every variant is the count exchange: it expires waiting on rank 1, the plan stays
    empty and no later stage touches y or the combine buffer."""
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    from deepgemm_b200 import _lib
    mode = {"staged": _lib.MODE_STAGED, "split": _lib.MODE_STAGED_SPLIT, "fused": _lib.MODE_FUSED}[mode_name]
    ph = _PhantomPeer(short_timeouts)
    out = ph.call(mode)
    assert out[0] == 1, f"expected a rank-barrier timeout status, got {out}"
    assert out[1] == BAR_COUNTS and out[2] == 1, "the first wait to expire is the count exchange, waiting on rank 1"
    assert out[3] == 1 and out[4] == 0        # expected epoch 1, observed 0
    ph.assert_outputs_untouched()
    _clean_call_afterwards()


def test_missing_peer_at_the_dispatch_barrier_of_the_split_launches(short_timeouts):
    """Counts 'arrive' (pre-set signal, zero rows from the peer), the rows are dispatched, then the dispatch barrier
    expires; the GEMMs, the requantisation and the reduce see the status and leave y and the combine buffer alone."""
    from deepgemm_b200 import _lib
    ph = _PhantomPeer(short_timeouts)
    ph.pretend_peer_signalled(BAR_COUNTS)
    out = ph.call(_lib.MODE_STAGED_SPLIT)
    assert out[0] == 1 and out[1] == BAR_DISPATCH and out[2] == 1, out
    ph.assert_outputs_untouched()
    _clean_call_afterwards()


@pytest.mark.parametrize("mode_name", ["staged", "fused"])
def test_missing_peer_at_the_combine_barrier(short_timeouts, mode_name):
    """Counts 'arrive' and the local rows are processed (the combine buffer IS written by this rank's own GEMM2), then the
    wait for the peer's 'combine stores done' expires: the reduce does not run and y stays untouched."""
    from deepgemm_b200 import _lib
    ph = _PhantomPeer(short_timeouts)
    ph.pretend_peer_signalled(BAR_COUNTS)
    out = ph.call(_lib.MODE_STAGED if mode_name == "staged" else _lib.MODE_FUSED)
    assert out[0] == 1 and out[1] == BAR_COMBINE and out[2] == 1, out
    assert bool((ph.y == 7.0).all()), "y was written although the combine barrier had expired"
    _clean_call_afterwards()
