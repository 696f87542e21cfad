"""ctypes binding of libmegamoe_b200.so (the C ABI declared in include/megamoe_b200.h).

There is no fallback: if the shared object is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_uint64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmegamoe_b200.so")

# enum mirrors of include/megamoe_b200.h
SYM_NAMES = ["peer_ptrs", "signals", "runtime_num_tokens", "count_matrix", "x", "x_sf", "topk_idx", "topk_weights",
             "pool_x", "pool_meta", "combine", "pool_rows"]
SCR_NAMES = ["status", "epoch", "plan", "block_counts", "dest_base", "expert_total", "expert_off", "mblock_expert",
             "mblock_valid", "dest_row", "row_amax", "act_scale", "act_bf16", "act_fp8", "send_base", "send_list", "l1_done",
             "l2_ready", "grid_sync", "act_sf", "route_blocks"]
MODE_STAGED, MODE_FUSED, MODE_STAGED_SPLIT, MODE_STAGED_UE8M0 = 0, 1, 2, 3
MAX_RANKS = 16
BLOCK_M = 128

STATUS_NAMES = {0: "ok", 1: "rank barrier timeout", 2: "GEMM pipeline timeout", 3: "receive pool overflow",
                4: "grid barrier timeout", 5: "m-grouped GEMM: a 128-row block mixes experts or has a hole"}

# every symbol the header declares, with its signature
_SIGNATURES = {
    "mm_last_error": (c_char_p, []),
    "mm_token_alignment": (c_int, []),
    "mm_symm_buffer_layout": (c_int, [c_int] * 6 + [POINTER(c_int64), POINTER(c_int64)]),
    "mm_scratch_layout": (c_int, [c_int] * 6 + [POINTER(c_int64), POINTER(c_int64)]),
    "mm_ipc_alloc": (c_int, [c_int64, POINTER(c_void_p), c_void_p]),
    "mm_ipc_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "mm_ipc_close": (c_int, [c_void_p]),
    "mm_ipc_free": (c_int, [c_void_p]),
    "mm_init_buffers": (c_int, [c_void_p, c_void_p, POINTER(c_uint64), c_int] + [c_int] * 6 + [c_void_p]),
    "mm_quant_per_token": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
    "mm_deepep_scatter_channelwise": (c_int, [c_void_p] * 11 + [c_int] * 6 + [c_void_p]),
    "mm_deepep_gather_channelwise": (c_int, [c_void_p] * 5 + [c_int] * 5 + [c_void_p]),
    "mm_m_grouped_fp8_gemm_nt_contiguous": (c_int, [c_void_p] * 6 + [c_int] * 4 + [c_void_p, c_void_p]),
    "mm_swiglu_quant_channelwise": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_float, c_void_p]),
    "mm_fp8_mma_peak_probe": (c_int, [c_int, c_int, c_int, c_void_p, c_void_p, POINTER(ctypes.c_double)]),
    "mm_peer_store_probe": (c_int, [POINTER(c_uint64), c_int, c_int64, c_void_p]),
    "mm_router_topk_quant": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "mm_fp8_w8a8_mega_moe": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     POINTER(c_uint64), c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                     c_int, c_void_p, c_void_p]),
    "mm_read_status": (c_int, [c_void_p, c_void_p, POINTER(c_int32)]),
    "mm_set_timeouts": (c_int, [c_int, c_int]),
    "mm_set_tuning": (c_int, [c_int, c_int]),
    "mm_set_tile_trace": (c_int, [c_void_p, c_int, c_int]),
    "mm_tile_order": (c_int, [c_int, c_int, c_int, c_int, c_int, POINTER(c_int32)]),
    "mm_build_config": (c_int, [ctypes.c_char_p, c_int]),
    "mm_launch_count": (c_int64, []),
    "mm_fp8_w8a8_mega_moe_static": (c_int, [c_void_p] * 10 + [c_int] * 5 + [c_float, c_void_p]),
    "mm_fp8_w8a8_mega_moe_static_status": (c_int, [c_void_p, POINTER(c_int32)]),
    "mm_set_stage_timing": (c_int, [c_int]),
    "mm_get_stage_times": (c_int, [POINTER(c_float), c_int]),
}
STAGE_NAMES = ["route_count", "route_exchange", "route_plan", "dispatch", "barrier_dispatch", "gemm1", "requant", "gemm2",
               "barrier_combine", "reduce", "fused"]
EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


class MegaMoeError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Load the shared object (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MegaMoeError(
                f"{LIB_PATH} is missing: build it with `python -m deepgemm_b200.build` "
                "(there is no CPU or PyTorch fallback for this operator)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        msg = lib().mm_last_error()
        raise MegaMoeError(f"libmegamoe_b200 error {rc}: {msg.decode() if msg else '?'}")


def symm_buffer_layout(R, E, T, K, H, I):
    offs = (c_int64 * len(SYM_NAMES))()
    total = c_int64()
    check(lib().mm_symm_buffer_layout(R, E, T, K, H, I, offs, ctypes.byref(total)))
    return dict(zip(SYM_NAMES, offs)), total.value


def scratch_layout(R, E, T, K, H, I):
    offs = (c_int64 * len(SCR_NAMES))()
    total = c_int64()
    check(lib().mm_scratch_layout(R, E, T, K, H, I, offs, ctypes.byref(total)))
    return dict(zip(SCR_NAMES, offs)), total.value


def build_config() -> dict:
    import json
    buf = ctypes.create_string_buffer(1024)
    check(lib().mm_build_config(buf, 1024))
    return json.loads(buf.value.decode())


def stage_times() -> dict:
    """Durations (ms) of the stages of the last layer call made with stage timing on."""
    buf = (c_float * len(STAGE_NAMES))()
    check(lib().mm_get_stage_times(buf, len(STAGE_NAMES)))
    return {n: float(v) for n, v in zip(STAGE_NAMES, buf) if v >= 0}


def fp8_mma_peak_tflops(iters: int = 20000, repeats: int = 5, random_operands: bool = False, cta_pair: bool = False,
                        quantised_like_operands: bool = False) -> float:
    """Dense FP8 tensor-core rate (TFLOP/s) measured with the library's probe kernel on the current device (best of repeats).
    random_operands: pseudo-random e4m3 data of magnitude below 2 instead of all ones; quantised_like_operands: e4m3 codes
    with the exponent fields per-row quantisation of N(0,1) data produces.  Both draw more power than all ones, so under
    the board's power cap the clock and the rate are lower (the cycle count per MMA is the same)."""
    import torch
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    flops = ctypes.c_double()
    best = 0.0
    for _ in range(repeats + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        check(lib().mm_fp8_mma_peak_probe(iters, 2 if quantised_like_operands else int(random_operands), int(cta_pair), status.data_ptr(), stream,
                                          ctypes.byref(flops)))
        e1.record()
        torch.cuda.synchronize()
        best = max(best, flops.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    if int(status.item()) != 0:
        raise MegaMoeError("the FP8 peak probe timed out")
    return best


def launch_count() -> int:
    return int(lib().mm_launch_count())
