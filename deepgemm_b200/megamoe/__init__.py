"""B200 (sm_100a) implementation of the `megamoe` Python API of yuguo-Jack/DeepGEMM.

Same public names, argument meaning and error behaviour as the reference package (megamoe/__init__.py:461-473);
underneath, every step runs as hand-written CUDA in libmegamoe_b200.so, called through its C ABI with raw
pointers.  There is no CPU or PyTorch fallback: CUDA tensors are required and a missing library is an error.

Differences a caller can observe (all supersets of the reference behaviour):
  * any EP size in 1..16 and any shape with hidden % 128 == 0, intermediate % 128 == 0, top-k <= 32 is accepted
    (the reference accepts only EP8 / 256 experts / top-6 / 4096 / 2048: csrc/kernels/mega_moe_fused_hip.cu:94-119);
  * `transform_fp8_weights_for_mega_moe` returns weights packed in 256x128-byte tiles (one TMA box = 32 contiguous KiB);
    plain `[E_loc, rows, K]` weights and the reference's Marlin layout `[E_loc, rows/16, K*16]` are also accepted and
    re-packed once;
  * `group=None` builds a single-rank buffer without torch.distributed;
  * device-side waits are bounded: `SymmBuffer.check_status()` reports a timeout instead of aborting the process.
"""
from __future__ import annotations

import ctypes
import math
import os
import weakref
from types import SimpleNamespace
from typing import Optional, Tuple

import torch

from .. import _lib

__version__ = "0.1"

_LARGE_OPT_FORCE_VALUES = {"1", "true", "yes", "on", "large_opt", "3stage"}
_LARGE_OPT_AUTO_VALUES = {"auto", "threshold", "adaptive"}
_LARGE_OPT_ENV = "MEGAMOE_DCU_USE_LARGE_OPT_3STAGE"
_LARGE_OPT_THRESHOLD_ENV = "MEGAMOE_DCU_LARGE_OPT_3STAGE_TOKEN_THRESHOLD"
# The reference switches at 128 tokens (megamoe/__init__.py:22).  Measured on B200 (2 ranks, DSV4-Flash shape) the fused
# variant still wins at 192-256 tokens per rank (5-6 %), ties near 512 and loses beyond, or earlier with skewed routing.
_LARGE_OPT_DEFAULT_THRESHOLD = 256
# un-prefixed aliases of the reference's environment variables
_ALIASES = {_LARGE_OPT_ENV: "MEGAMOE_USE_STAGED", _LARGE_OPT_THRESHOLD_ENV: "MEGAMOE_STAGED_TOKEN_THRESHOLD"}

# Kind of staged variant, snapshotted per buffer: by default the routing kernels are followed by ONE launch that pushes rows
# over NVLink, runs GEMM1, requantises and runs GEMM2 with per-m-block dependencies; MEGAMOE_STAGED_SPLIT=1 selects separate
# dispatch / barrier / GEMM1 / requantisation / GEMM2 launches instead.  All ranks of a group must use the same setting.
_STAGED_SPLIT_ENV = "MEGAMOE_STAGED_SPLIT"
# Recipe value of fp8_mega_moe for the activation recipe of the reference's Blackwell Mega MoE kernel (deep_gemm/mega/__init__.py:105-142,
# deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:1023-1057): the SwiGLU output is quantised inside the GEMM1 tile
# to e4m3 with one power-of-two (UE8M0) scale per (row, 32 columns) and GEMM2 applies the scales with a block-scaled MMA.
# The default recipe (1, 1, 32) is the reference's W8A8 channelwise one.  Weights are FP8 with channelwise scales in both.
RECIPE_UE8M0_PER32 = "ue8m0_per32"
_FUSED_AVAILABLE = True


def _align(value: int, alignment: int) -> int:
    return ((value + alignment - 1) // alignment) * alignment


def _env(name: str, default: str) -> str:
    v = os.getenv(name)
    if v is None and name in _ALIASES:
        v = os.getenv(_ALIASES[name])
    return default if v is None else v


def _large_opt_3stage_mode() -> str:
    """megamoe/__init__.py:25-31."""
    value = _env(_LARGE_OPT_ENV, "auto").strip().lower()
    if value in _LARGE_OPT_FORCE_VALUES:
        return "force"
    if value in _LARGE_OPT_AUTO_VALUES:
        return "auto"
    return "off"


def _large_opt_3stage_threshold() -> int:
    return int(_env(_LARGE_OPT_THRESHOLD_ENV, str(_LARGE_OPT_DEFAULT_THRESHOLD)))


def _large_opt_3stage_selected(num_tokens: int, mode: str, threshold: int) -> bool:
    """megamoe/__init__.py:38-43: staged when forced, or in auto mode above the threshold."""
    if mode == "force":
        return True
    if mode == "auto":
        return num_tokens > threshold
    return False


def _eager_variant_is_staged(mode: str, threshold: int, y_tokens: int, dispatch_num_tokens: Optional[int]) -> bool:
    """Variant of an eager (non-graph) call, decided exactly as the reference does (megamoe/__init__.py:398-404): on
    dispatch_num_tokens if given, else on y.size(0).  Every rank of a group must run the same variant (the staged launches
    and the fused kernel signal one another differently), so when ranks hold different token counts the caller passes one
    dispatch_num_tokens to all of them -- the reference's contract (README.md:165-177).  A mismatch does not deadlock here:
    the bounded waits expire and SymmBuffer.check_status() reports it."""
    tokens = y_tokens if dispatch_num_tokens is None else int(dispatch_num_tokens)
    return _large_opt_3stage_selected(tokens, mode, threshold)


def _staged_as_split_launches(sb, tokens: int, e_loc: int) -> bool:
    """Kind of staged variant.  The single layer kernel (in-kernel NVLink push, GEMM1, requantisation and GEMM2 tiles with
    per-m-block dependencies) is the default.  Separate launches are used when MEGAMOE_STAGED_SPLIT=1 was set at buffer
    creation, and when an expert is expected to hold two 128-row blocks (144 < tokens * top-k / local experts <= 256): there
    the CTA-pair GEMM kernels of the split launches are about 10 % faster (measured on B200).  `tokens` is the count the
    fused/staged choice was made on, so all ranks agree under the same caller contract."""
    if sb._staged_split:
        return True
    routes = int(tokens) * sb.num_topk
    return sb._staged_split_auto and 144 * e_loc < routes <= 256 * e_loc


def _is_current_stream_capturing() -> bool:
    checker = getattr(torch.cuda, "is_current_stream_capturing", None)
    return bool(checker()) if checker is not None else False


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (this package has no CPU path)")


# ------------------------------------------------------------------------------------------------ quantisation
def cast_to_fp8_channelwise(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row FP8 e4m3 cast: scale = clamp(amax,1e-4)/448 (megamoe/__init__.py:51-56), bit-exact, as one kernel."""
    if x.dim() != 2:
        raise ValueError("channelwise FP8 cast expects a 2D tensor")
    _require_cuda(x, "x")
    if x.dtype != torch.bfloat16:
        raise TypeError("cast_to_fp8_channelwise expects bfloat16 input")
    rows, k = x.shape
    if k % 8 != 0:
        raise ValueError("the row length must be a multiple of 8")
    x = x.contiguous()
    out = torch.empty((rows, k), dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mm_quant_per_token(x.data_ptr(), rows, k, out.data_ptr(), scale.data_ptr(), _stream_ptr()))
    return out, scale


def cast_grouped_weight_to_fp8_channelwise(weights: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per output row of every expert (megamoe/__init__.py:59-78)."""
    if weights.dim() != 3:
        raise ValueError("MegaMoE grouped weights must be 3D tensors")
    g, rows, k = weights.shape
    q, s = cast_to_fp8_channelwise(weights.reshape(g * rows, k))
    return q.reshape(g, rows, k), s.reshape(g, rows)


def weight8bit_nt_kpack2_marlin(weight: torch.Tensor, k_tile: int = 16, n_tile: int = 16) -> torch.Tensor:
    """The reference's 16x16 tile permutation [E,R,K] -> [E,R/16,K*16] (megamoe/__init__.py:81-98).  Kept so that
    callers holding Marlin-packed checkpoints interoperate; the B200 kernels themselves read the plain layout."""
    if weight.dim() != 3:
        raise ValueError("MegaMoE Marlin weight layout expects a 3D grouped weight tensor")
    if k_tile != 16 or n_tile != 16:
        raise ValueError("DCU W8A8 MegaMoE currently supports only 16x16 kpack2 Marlin tiles")
    g, rows, k = weight.shape
    if rows % n_tile != 0 or k % k_tile != 0:
        raise ValueError("DCU W8A8 MegaMoE Marlin weights require rows and K divisible by 16")
    return (weight.view(torch.uint8).reshape(g, rows // n_tile, n_tile, k // k_tile, k_tile).permute(0, 1, 3, 2, 4)
            .contiguous().reshape(g, rows // n_tile, k * n_tile).view(weight.dtype))


def _marlin_inverse(weight: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    g = weight.shape[0]
    return (weight.view(torch.uint8).reshape(g, rows // 16, k // 16, 16, 16).permute(0, 1, 3, 2, 4)
            .contiguous().reshape(g, rows, k).view(weight.dtype))


def pack_weights_tiled(weight: torch.Tensor, which: str) -> torch.Tensor:
    """Pack a grouped FP8 weight tensor [E, rows, K] into the order the GEMM kernels stream it from HBM:
    [E][n block][K/128][256 rows][128 bytes], one contiguous 32 KiB block per (output tile, k block).

    which="l1": gate+up weights [E, 2I, K]; n block j holds gate rows [128j, 128j+128) followed by the matching up
                rows [I+128j, I+128j+128), so one output tile yields 128 complete SwiGLU results.
    which="l2": down weights [E, H, K]; n block j holds rows [256j, 256j+256) (zero rows past H when H % 256 == 128).
    It plays the role the 16x16 Marlin packing plays for the reference's MMAC kernels (megamoe/__init__.py:81-98)."""
    if weight.dim() != 3:
        raise ValueError("expected a grouped [E, rows, K] weight tensor")
    if which not in ("l1", "l2"):
        raise ValueError("which must be 'l1' or 'l2'")
    g, rows, k = weight.shape
    if rows % 128 != 0 or k % 128 != 0 or (which == "l1" and rows % 256 != 0):
        raise ValueError("rows and K must be multiples of 128 (L1 rows: of 256)")
    src = weight.view(torch.uint8)
    if which == "l1":
        nb = rows // 256
        out = torch.empty((g, nb, k // 128, 256, 128), dtype=torch.uint8, device=weight.device)
        for e in range(g):   # one expert at a time bounds the temporary
            # [2 (gate/up), nb, 128, kt, 128] -> [nb, kt, 2, 128, 128]
            out[e].view(nb, k // 128, 2, 128, 128).copy_(src[e].reshape(2, nb, 128, k // 128, 128).permute(1, 3, 0, 2, 4))
    else:
        nb = (rows + 255) // 256
        out = torch.zeros((g, nb, k // 128, 256, 128), dtype=torch.uint8, device=weight.device)
        full = rows // 256
        for e in range(g):
            if full:
                out[e, :full].copy_(src[e, :full * 256].reshape(full, 256, k // 128, 128).permute(0, 2, 1, 3))
            if rows % 256:
                out[e, full, :, :128].copy_(src[e, full * 256:].reshape(128, k // 128, 128).permute(1, 0, 2))
    return out.view(weight.dtype)


def unpack_weights_tiled(weight: torch.Tensor, which: str, rows: int) -> torch.Tensor:
    """Inverse of pack_weights_tiled: back to [E, rows, K]."""
    g, nb, kt = weight.shape[:3]
    src = weight.view(torch.uint8)
    if which == "l1":
        out = src.reshape(g, nb, kt, 2, 128, 128).permute(0, 3, 1, 4, 2, 5).reshape(g, 2 * nb * 128, kt * 128)
    else:
        out = src.permute(0, 1, 3, 2, 4).reshape(g, nb * 256, kt * 128)[:, :rows]
    return out.contiguous().view(weight.dtype)


def transform_fp8_weights_for_mega_moe(l1_weights: torch.Tensor, l2_weights: torch.Tensor, layout: str = "tiled"):
    """bf16 [E_loc,2I,H], [E_loc,H,I] -> ((w1_fp8, s1[E_loc,2I]), (w2_fp8, s2[E_loc,H])) (megamoe/__init__.py:280-289).
    layout="tiled" (default) packs for the B200 kernels (see pack_weights_tiled); "native" keeps [E_loc, rows, K];
    "marlin" applies the reference's permutation.  fp8_mega_moe accepts all three."""
    l1_fp8, l1_scale = cast_grouped_weight_to_fp8_channelwise(l1_weights)
    l2_fp8, l2_scale = cast_grouped_weight_to_fp8_channelwise(l2_weights)
    if layout == "marlin":
        return (weight8bit_nt_kpack2_marlin(l1_fp8), l1_scale), (weight8bit_nt_kpack2_marlin(l2_fp8), l2_scale)
    if layout == "tiled":
        return (pack_weights_tiled(l1_fp8, "l1"), l1_scale), (pack_weights_tiled(l2_fp8, "l2"), l2_scale)
    if layout != "native":
        raise ValueError("layout must be 'tiled', 'native' or 'marlin'")
    return (l1_fp8, l1_scale), (l2_fp8, l2_scale)


def get_mega_moe_hip_build_config() -> dict:
    """csrc/apis/mega_dcu.hpp:28-39 + megamoe/__init__.py:101-110 (name kept for drop-in use)."""
    config = _lib.build_config()
    config["large_opt_3stage_env"] = _LARGE_OPT_ENV
    config["large_opt_3stage_auto_values"] = sorted(_LARGE_OPT_AUTO_VALUES)
    config["large_opt_3stage_threshold_env"] = _LARGE_OPT_THRESHOLD_ENV
    config["large_opt_3stage_default_threshold"] = _LARGE_OPT_DEFAULT_THRESHOLD
    config["large_opt_3stage_shape"] = "any EP<=16, hidden%128==0, intermediate%128==0, topk<=32"
    config["cuda_graph_max_tokens_source"] = "requested num_max_tokens_per_rank"
    config["cuda_graph_execution"] = "explicit_big_fused_or_large_opt_3stage"
    config["fused_variant_available"] = _FUSED_AVAILABLE
    return config


# ------------------------------------------------------------------------------------------------ symmetric buffer
class _DeviceMemory:
    """Exposes a raw device allocation to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|i1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _view(buffer: torch.Tensor, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
    n = int(math.prod(shape)) * torch.empty((), dtype=dtype).element_size()
    return buffer[offset:offset + n].view(dtype).view(*shape)


def _gather_handles(group, payload: bytes):
    """All-gather one opaque handle per rank; entry r of the result is rank r's handle (megamoe/__init__.py:178-181)."""
    import torch.distributed as dist
    gathered = [None] * group.size()
    dist.all_gather_object(gathered, (group.rank(), payload), group)
    out = [None] * group.size()
    for r, raw in gathered:
        out[r] = raw
    if any(h is None for h in out):
        raise RuntimeError("handle exchange is incomplete: a rank did not contribute")
    return out


class SymmBuffer:
    """Peer-mapped buffer + local scratch of one rank (megamoe/__init__.py:113-249)."""

    def __init__(self, group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                 intermediate_hidden: int, use_fp8_dispatch: bool = True, activation: str = "swiglu",
                 cuda_graph_max_tokens_per_rank: Optional[int] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("megamoe (B200) needs a CUDA device")
        if activation != "swiglu":
            raise ValueError("only swiglu is supported")
        if not use_fp8_dispatch:
            raise ValueError("only FP8 dispatch is supported")
        self.group = group
        self.num_experts = int(num_experts)
        self.num_max_tokens_per_rank = int(num_max_tokens_per_rank)
        self.num_topk = int(num_topk)
        self.hidden = int(hidden)
        self.intermediate_hidden = int(intermediate_hidden)
        self._large_opt_3stage_mode = _large_opt_3stage_mode()
        self._large_opt_3stage_threshold = _large_opt_3stage_threshold()
        self._staged_split = os.getenv(_STAGED_SPLIT_ENV, "auto").strip().lower() in _LARGE_OPT_FORCE_VALUES
        self._staged_split_auto = os.getenv(_STAGED_SPLIT_ENV, "auto").strip().lower() in _LARGE_OPT_AUTO_VALUES
        self.cuda_graph_max_tokens_per_rank = int(cuda_graph_max_tokens_per_rank
                                                  if cuda_graph_max_tokens_per_rank is not None
                                                  else num_max_tokens_per_rank)
        if (self.cuda_graph_max_tokens_per_rank <= 0
                or self.cuda_graph_max_tokens_per_rank > self.num_max_tokens_per_rank):
            raise ValueError(f"cuda_graph_max_tokens_per_rank must be in 1..{self.num_max_tokens_per_rank}")

        self.num_ranks = 1 if group is None else group.size()
        self.rank = 0 if group is None else group.rank()
        dims = (self.num_ranks, self.num_experts, self.num_max_tokens_per_rank, self.num_topk, self.hidden,
                self.intermediate_hidden)
        self._dims = dims
        self._sym_off, num_bytes = _lib.symm_buffer_layout(*dims)
        self._scr_off, scratch_bytes = _lib.scratch_layout(*dims)
        self.device = torch.device("cuda", torch.cuda.current_device())
        lib = _lib.lib()
        self._owned_ptr = None
        self._peer_mapped = []
        if self.num_ranks == 1:
            self.buffer = torch.empty((num_bytes,), dtype=torch.int8, device=self.device)
            buffer_ptr = self.buffer.data_ptr()
            buffer_ptrs = [buffer_ptr]
        else:
            import torch.distributed as dist
            ptr = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            _lib.check(lib.mm_ipc_alloc(num_bytes, ctypes.byref(ptr), handle))
            buffer_ptr = int(ptr.value)
            self._owned_ptr = buffer_ptr
            self.buffer = torch.as_tensor(_DeviceMemory(buffer_ptr, num_bytes), device=self.device)
            buffer_ptrs = [0] * self.num_ranks
            for r, raw in enumerate(_gather_handles(group, bytes(handle.raw))):
                if r == self.rank:
                    buffer_ptrs[r] = buffer_ptr
                else:
                    peer = ctypes.c_void_p()
                    _lib.check(lib.mm_ipc_open(ctypes.create_string_buffer(raw, 64), ctypes.byref(peer)))
                    buffer_ptrs[r] = int(peer.value)
                    self._peer_mapped.append(int(peer.value))
        self.route_scratch = torch.empty((scratch_bytes,), dtype=torch.int8, device=self.device)
        sig = self._sym_off["signals"]
        self.handle = SimpleNamespace(buffer_ptrs=buffer_ptrs, buffer_ptr=buffer_ptr,
                                      signal_ptrs=[p + sig for p in buffer_ptrs], signal_buffer_ptr=buffer_ptr + sig)
        self._peer_array = (ctypes.c_uint64 * _lib.MAX_RANKS)(*buffer_ptrs)
        self.reset()

        T, K, H = self.num_max_tokens_per_rank, self.num_topk, self.hidden
        o = self._sym_off
        self.x = _view(self.buffer, o["x"], (T, H), torch.float8_e4m3fn)
        self.x_sf = _view(self.buffer, o["x_sf"], (T,), torch.float32)
        self.topk_idx = _view(self.buffer, o["topk_idx"], (T, K), torch.int64)
        self.topk_weights = _view(self.buffer, o["topk_weights"], (T, K), torch.float32)
        empty_fp8 = self.buffer[o["combine"]:o["combine"]].view(torch.float8_e4m3fn)
        empty_f32 = self.buffer[o["combine"]:o["combine"]].view(torch.float32)
        self.l1_acts, self.l1_acts_sf, self.l2_acts, self.l2_acts_sf = empty_fp8, empty_f32, empty_fp8, empty_f32
        self.cuda_graph_num_tokens = _view(self.buffer, o["runtime_num_tokens"], (1,), torch.int32)
        self.cuda_graph_num_tokens.fill_(self.cuda_graph_max_tokens_per_rank)
        torch.cuda.synchronize()
        if group is not None:
            import torch.distributed as dist
            dist.barrier(group)

    # -- maintenance ------------------------------------------------------------------------------
    def reset(self) -> None:
        """Zero the control regions and (re)write the peer table; collective across the group."""
        torch.cuda.synchronize()
        if self.group is not None:
            import torch.distributed as dist
            dist.barrier(self.group)
        _lib.check(_lib.lib().mm_init_buffers(self.buffer.data_ptr(), self.route_scratch.data_ptr(), self._peer_array,
                                              self.rank, *self._dims, _stream_ptr()))
        torch.cuda.synchronize()
        if self.group is not None:
            import torch.distributed as dist
            dist.barrier(self.group)
        if getattr(self, "cuda_graph_num_tokens", None) is not None:
            self.cuda_graph_num_tokens.fill_(self.cuda_graph_max_tokens_per_rank)

    def check_status(self) -> None:
        """Synchronise and raise if a bounded device-side wait expired during an earlier call."""
        out = (ctypes.c_int32 * 5)()
        _lib.check(_lib.lib().mm_read_status(self.route_scratch.data_ptr(), _stream_ptr(), out))
        if out[0] != 0:
            raise _lib.MegaMoeError(
                f"device status {out[0]} ({_lib.STATUS_NAMES.get(out[0], '?')}): phase={out[1]} rank/block={out[2]} "
                f"expected={out[3]} observed={out[4]}; call SymmBuffer.reset() on every rank before reuse")

    def scratch_view(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        """Typed view of a region of the local scratch buffer (for tests and inspection)."""
        return _view(self.route_scratch, self._scr_off[name], shape, dtype)

    def symm_view(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        return _view(self.buffer, self._sym_off[name], shape, dtype)

    @property
    def pool_rows(self) -> int:
        return int(self._sym_off["pool_rows"])

    def destroy(self):
        if self.handle is not None:
            torch.cuda.synchronize()
            lib = _lib.lib()
            for p in self._peer_mapped:
                _lib.check(lib.mm_ipc_close(p))
            self._peer_mapped = []
            if self.group is not None:
                import torch.distributed as dist
                dist.barrier(self.group)
            self.x = self.x_sf = self.topk_idx = self.topk_weights = None
            self.l1_acts = self.l1_acts_sf = self.l2_acts = self.l2_acts_sf = None
            self.cuda_graph_num_tokens = None
            self.buffer = None
            if self._owned_ptr is not None:
                _lib.check(lib.mm_ipc_free(self._owned_ptr))
                self._owned_ptr = None
        self.handle = None
        self.buffer = None
        self.group = None
        self.route_scratch = None


def get_symm_buffer_for_mega_moe(group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                                 intermediate_hidden: int, use_fp8_dispatch: bool = True,
                                 activation: str = "swiglu") -> SymmBuffer:
    """megamoe/__init__.py:252-277: capacity aligned up to 384 tokens, the request kept as the graph bucket size."""
    requested = int(num_max_tokens_per_rank)
    aligned = _align(requested, _lib.lib().mm_token_alignment())
    return SymmBuffer(group, num_experts, aligned, num_topk, hidden, intermediate_hidden, use_fp8_dispatch, activation,
                      cuda_graph_max_tokens_per_rank=requested)


# ------------------------------------------------------------------------------------------------ the layer
_packed_weight_cache = {}


def _tiled_weight(w: torch.Tensor, rows: int, k: int, which: str) -> torch.Tensor:
    """Accept the tiled layout [E_loc, n blocks, K/128, 256, 128] as is; plain [E_loc, rows, K] and the reference's
    Marlin shape [E_loc, rows/16, K*16] are re-packed once and cached (keyed by storage address and version)."""
    nb = rows // 256 if which == "l1" else (rows + 255) // 256
    if w.dim() == 5 and tuple(w.shape[1:]) == (nb, k // 128, 256, 128):
        return w if w.is_contiguous() else w.contiguous()
    if w.dim() != 3:
        raise RuntimeError("weights must be grouped 3D tensors (or tiled 5D tensors)")
    native = w.shape[1] == rows and w.shape[2] == k
    marlin = w.shape[1] == rows // 16 and w.shape[2] == k * 16
    if not (native or marlin):
        raise RuntimeError(f"invalid {which.upper()} weight shape {tuple(w.shape)}, expected [expert, {rows}, {k}], "
                           f"Marlin [expert, {rows // 16}, {k * 16}] or tiled [expert, {nb}, {k // 128}, 256, 128]")
    # Keyed by address, shape, version counter and packing kind, and valid only while the SAME tensor object is alive: the
    # allocator hands a freed address to the next tensor of that size, whose version counter also starts at 0.
    key = (w.data_ptr(), tuple(w.shape), w._version, which)
    hit = _packed_weight_cache.get(key)
    if hit is not None and hit[0]() is w:
        return hit[1]
    for stale in [k_ for k_, v in _packed_weight_cache.items() if v[0]() is None]:
        del _packed_weight_cache[stale]
    if len(_packed_weight_cache) > 16:
        _packed_weight_cache.clear()
    packed = pack_weights_tiled(w.contiguous() if native else _marlin_inverse(w, rows, k), which)
    _packed_weight_cache[key] = (weakref.ref(w), packed)
    return packed


def fp8_mega_moe(y: torch.Tensor, l1_weights, l2_weights, sym_buffer: SymmBuffer,
                 cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                 recipe=(1, 1, 32), activation: str = "swiglu",
                 activation_clamp: Optional[float] = None, fast_math: bool = True, big_fused_cuda_graph: bool = False,
                 stages_fused_cuda_graph: bool = False, dispatch_num_tokens: Optional[int] = None) -> None:
    """The W8A8 channelwise Mega MoE layer, in place into `y` (megamoe/__init__.py:328-449 and
    csrc/apis/mega_dcu.hpp:338-445 for the argument checks).  Inputs are read from the SymmBuffer views
    x / x_sf / topk_idx / topk_weights; the call is asynchronous on the current stream."""
    if big_fused_cuda_graph and stages_fused_cuda_graph:
        raise ValueError("choose only one of big_fused_cuda_graph or stages_fused_cuda_graph")
    graph_mode = big_fused_cuda_graph or stages_fused_cuda_graph
    sb = sym_buffer
    if graph_mode:
        graph_max_tokens = int(sb.cuda_graph_max_tokens_per_rank)
        if int(y.size(0)) < graph_max_tokens:
            raise ValueError(f"CUDA graph mode requires y to have at least {graph_max_tokens} rows; pass a fixed "
                             "graph-bucket output buffer and consume only the valid prefix")
        if cumulative_local_expert_recv_stats is not None:
            raise ValueError("CUDA graph mode does not support cumulative_local_expert_recv_stats")
        if stages_fused_cuda_graph and sb._large_opt_3stage_mode == "off":
            raise RuntimeError("stages_fused_cuda_graph=True requires MEGAMOE_DCU_USE_LARGE_OPT_3STAGE=auto or 1")
        staged = bool(stages_fused_cuda_graph)
        call_y = y[:graph_max_tokens]
        runtime_ptr = sb.cuda_graph_num_tokens.data_ptr()
        split_tokens = graph_max_tokens
    else:
        if _is_current_stream_capturing():
            raise RuntimeError(
                "DCU MegaMoE CUDA Graph capture requires an explicit graph mode: pass big_fused_cuda_graph=True for the "
                "persistent fused path or stages_fused_cuda_graph=True for the staged K1/K2/K3 path. "
                "Capturing the eager auto-dispatch path is not graph-bucket safe.")
        dispatch_tokens = int(y.size(0)) if dispatch_num_tokens is None else int(dispatch_num_tokens)
        if dispatch_tokens < 0 or dispatch_tokens > int(sb.num_max_tokens_per_rank):
            raise ValueError(f"dispatch_num_tokens must be in 0..{int(sb.num_max_tokens_per_rank)}")
        staged = _eager_variant_is_staged(sb._large_opt_3stage_mode, sb._large_opt_3stage_threshold, int(y.size(0)),
                                          dispatch_num_tokens)
        call_y = y
        runtime_ptr = None
        split_tokens = dispatch_tokens

    # argument checks of csrc/apis/mega_dcu.hpp:355-445
    ue8m0 = isinstance(recipe, str) and recipe == RECIPE_UE8M0_PER32
    if not ue8m0 and (isinstance(recipe, str) or tuple(recipe) != (1, 1, 32)):
        raise RuntimeError(f"DCU W8A8 MegaMoE expects recipe=(1,1,32) (or recipe={RECIPE_UE8M0_PER32!r} for per-32 UE8M0 "
                           "activation scales)")
    if ue8m0:
        if graph_mode and not stages_fused_cuda_graph:
            raise ValueError("the UE8M0 recipe runs as staged launches: use stages_fused_cuda_graph=True for graph capture")
        staged = True
    if activation != "swiglu":
        raise RuntimeError("DCU W8A8 MegaMoE supports swiglu only")
    if not fast_math:
        raise RuntimeError("fast_math=False is not supported")
    _require_cuda(call_y, "y")
    if call_y.dtype != torch.bfloat16 or call_y.dim() != 2 or not call_y.is_contiguous():
        raise RuntimeError("y must be a contiguous 2D BF16 tensor")
    l1_w, l1_sf = l1_weights
    l2_w, l2_sf = l2_weights
    if l1_w.dtype != torch.float8_e4m3fn or l2_w.dtype != torch.float8_e4m3fn:
        raise RuntimeError("DCU MegaMoE expects FP8 E4M3 L1/L2 weights")
    if l1_sf.dtype != torch.float32 or l2_sf.dtype != torch.float32:
        raise RuntimeError("DCU MegaMoE expects FP32 channelwise weight scales")
    if l1_w.dim() not in (3, 5) or l2_w.dim() not in (3, 5):
        raise RuntimeError("weights must be grouped 3D tensors (or tiled 5D tensors)")
    if l1_sf.dim() != 2 or l2_sf.dim() != 2:
        raise RuntimeError("weight scales must be [expert,row]")
    num_tokens, hidden = int(call_y.size(0)), int(call_y.size(1))
    if l1_sf.size(1) % 2 != 0:
        raise RuntimeError("invalid L1 scale shape")
    inter = int(l1_sf.size(1)) // 2
    e_loc = int(l1_w.size(0))
    if hidden != sb.hidden or inter != sb.intermediate_hidden:
        raise RuntimeError("weights / y do not match the SymmBuffer's hidden sizes")
    if sb.num_experts != e_loc * sb.num_ranks:
        raise RuntimeError("invalid expert count")
    if tuple(l1_sf.shape) != (e_loc, 2 * inter):
        raise RuntimeError("invalid L1 scale shape")
    if tuple(l2_sf.shape) != (e_loc, hidden) or int(l2_w.size(0)) != e_loc:
        raise RuntimeError("invalid L2 scale shape")
    if num_tokens > sb.num_max_tokens_per_rank:
        raise RuntimeError("too many tokens")
    w1 = _tiled_weight(l1_w, 2 * inter, hidden, "l1")
    w2 = _tiled_weight(l2_w, hidden, inter, "l2")
    stats_ptr = None
    if cumulative_local_expert_recv_stats is not None:
        st = cumulative_local_expert_recv_stats
        if st.dtype != torch.int32:
            raise RuntimeError("stats must be int32")
        if st.numel() != e_loc:
            raise RuntimeError("stats must have num_experts_per_rank elements")
        _require_cuda(st, "stats")
        stats_ptr = st.data_ptr()
    clamp = float("inf") if activation_clamp is None else float(activation_clamp)
    with torch.cuda.device(sb.device):
        _lib.check(_lib.lib().mm_fp8_w8a8_mega_moe(
            call_y.data_ptr(), w1.data_ptr(), l1_sf.contiguous().data_ptr(), w2.data_ptr(), l2_sf.contiguous().data_ptr(),
            stats_ptr, sb.buffer.data_ptr(), sb.route_scratch.data_ptr(), sb._peer_array, sb.rank, sb.num_ranks,
            sb.num_max_tokens_per_rank, e_loc, num_tokens, sb.num_topk, hidden, inter, clamp,
            _lib.MODE_STAGED_UE8M0 if ue8m0 else
            ((_lib.MODE_STAGED_SPLIT if _staged_as_split_launches(sb, split_tokens, e_loc) else _lib.MODE_STAGED)
             if staged else _lib.MODE_FUSED), runtime_ptr, _stream_ptr()))


fp8_w8a8_mega_moe = fp8_mega_moe


def fill_inputs_from_router(sym_buffer: SymmBuffer, x: torch.Tensor, router_logits: torch.Tensor) -> int:
    """Fill sym_buffer.x / x_sf / topk_idx / topk_weights from bf16 activations [T, H] and fp32 router logits [T, E] with
    one kernel: top-k (descending, ties to the lower index), softmax over the selected logits, per-token FP8 cast.
    The reference leaves this to the caller as torch.topk + softmax + cast_to_fp8_channelwise + four copies
    (tests/test_mega_moe_dcu.py:491-508).  Returns the number of tokens written."""
    sb = sym_buffer
    _require_cuda(x, "x")
    _require_cuda(router_logits, "router_logits")
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.size(1) != sb.hidden:
        raise ValueError("x must be bf16 [tokens, hidden]")
    if router_logits.dtype != torch.float32 or tuple(router_logits.shape) != (x.size(0), sb.num_experts):
        raise ValueError("router_logits must be fp32 [tokens, num_experts]")
    if x.size(0) > sb.num_max_tokens_per_rank:
        raise ValueError("too many tokens")
    x = x.contiguous()
    router_logits = router_logits.contiguous()
    with torch.cuda.device(sb.device):
        _lib.check(_lib.lib().mm_router_topk_quant(x.data_ptr(), router_logits.data_ptr(), x.size(0), sb.num_experts, sb.num_topk,
                                                  sb.hidden, sb.x.data_ptr(), sb.x_sf.data_ptr(), sb.topk_idx.data_ptr(),
                                                  sb.topk_weights.data_ptr(), _stream_ptr()))
    return int(x.size(0))


def deepep_deepgemm_preprocess_channelwise(recv_x: torch.Tensor, recv_x_scale: torch.Tensor, recv_topk_ids: torch.Tensor,
                                           recv_topk_weights: torch.Tensor, num_recv_tokens_per_expert: torch.Tensor,
                                           all_tokens: int):
    """Group DeepEP-received tokens by expert for a grouped GEMM (csrc/apis/mega_dcu.hpp:222-291): returns
    (grouped_x fp8 [rows,H], grouped_x_scale f32 [rows], route_weights f32 [rows], m_indices i32 [rows],
    output_index i32 [tokens, topk]) with rows = max(all_tokens, 1)."""
    for t in (recv_x, recv_x_scale, recv_topk_ids, recv_topk_weights, num_recv_tokens_per_expert):
        _require_cuda(t, "DeepEP preprocess tensors")
        if not t.is_contiguous():
            raise RuntimeError("DeepEP preprocess tensors must be contiguous")
    if recv_x.dtype != torch.float8_e4m3fn:
        raise RuntimeError("DeepEP preprocess expects FP8 E4M3 recv_x")
    if recv_x_scale.dtype != torch.float32 or recv_topk_weights.dtype != torch.float32:
        raise RuntimeError("DeepEP preprocess scales and weights must be FP32")
    if recv_topk_ids.dtype not in (torch.int64, torch.int32):
        raise RuntimeError("DeepEP preprocess topk ids must be int64 or int32")
    if num_recv_tokens_per_expert.dtype != torch.int32:
        raise RuntimeError("num_recv_tokens_per_expert must be int32")
    if recv_x.dim() != 2 or recv_topk_ids.dim() != 2 or recv_topk_ids.shape != recv_topk_weights.shape:
        raise RuntimeError("recv_x must be [tokens, hidden]; topk ids/weights must be [tokens, topk]")
    if recv_topk_ids.size(0) != recv_x.size(0) or recv_x_scale.numel() != recv_x.size(0):
        raise RuntimeError("topk rows and recv_x_scale must match recv_x")
    if all_tokens < 0:
        raise RuntimeError("all_tokens must be non-negative")
    rows = max(int(all_tokens), 1)
    recv_rows, hidden = recv_x.shape
    topk = recv_topk_ids.size(1)
    num_experts = num_recv_tokens_per_expert.numel()
    dev = recv_x.device
    grouped_x = torch.empty((rows, hidden), dtype=torch.float8_e4m3fn, device=dev)
    grouped_x_scale = torch.empty((rows,), dtype=torch.float32, device=dev)
    route_weights = torch.zeros((rows,), dtype=torch.float32, device=dev)
    m_indices = torch.full((rows,), -1, dtype=torch.int32, device=dev)
    output_index = torch.full((recv_rows, topk), -1, dtype=torch.int32, device=dev)
    expert_start_loc = torch.empty((num_experts,), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().mm_deepep_scatter_channelwise(
            grouped_x.data_ptr(), grouped_x_scale.data_ptr(), route_weights.data_ptr(), m_indices.data_ptr(), output_index.data_ptr(),
            expert_start_loc.data_ptr(), recv_x.data_ptr(), recv_x_scale.data_ptr(), recv_topk_ids.data_ptr(),
            recv_topk_weights.data_ptr(), num_recv_tokens_per_expert.data_ptr(), rows, recv_rows, topk, hidden, num_experts,
            1 if recv_topk_ids.dtype == torch.int64 else 0, _stream_ptr()))
    return grouped_x, grouped_x_scale, route_weights, m_indices, output_index


def deepep_deepgemm_postprocess_channelwise(recv_y: torch.Tensor, l2_out: torch.Tensor, recv_topk_ids: torch.Tensor,
                                            recv_topk_weights: torch.Tensor, output_index: torch.Tensor,
                                            apply_topk_weights: bool = False) -> None:
    """Sum the per-route grouped-GEMM outputs back per received token, in place into recv_y
    (csrc/apis/mega_dcu.hpp:293-336)."""
    for t in (recv_y, l2_out, recv_topk_ids, recv_topk_weights, output_index):
        _require_cuda(t, "DeepEP postprocess tensors")
        if not t.is_contiguous():
            raise RuntimeError("DeepEP postprocess tensors must be contiguous")
    if recv_y.dtype != torch.bfloat16 or l2_out.dtype != torch.bfloat16:
        raise RuntimeError("DeepEP postprocess expects BF16 tensors")
    if recv_topk_ids.dtype not in (torch.int64, torch.int32):
        raise RuntimeError("DeepEP postprocess topk ids must be int64 or int32")
    if recv_topk_weights.dtype != torch.float32 or output_index.dtype != torch.int32:
        raise RuntimeError("topk weights must be FP32 and output_index int32")
    if (recv_y.dim() != 2 or l2_out.dim() != 2 or recv_topk_ids.shape != recv_topk_weights.shape
            or recv_topk_ids.shape != output_index.shape or recv_y.size(0) != recv_topk_ids.size(0)
            or recv_y.size(1) != l2_out.size(1)):
        raise RuntimeError("DeepEP postprocess shape mismatch")
    with torch.cuda.device(recv_y.device):
        _lib.check(_lib.lib().mm_deepep_gather_channelwise(
            recv_y.data_ptr(), l2_out.data_ptr(), recv_topk_ids.data_ptr(), recv_topk_weights.data_ptr(), output_index.data_ptr(),
            recv_y.size(0), recv_topk_ids.size(1), recv_y.size(1), 1 if recv_topk_ids.dtype == torch.int64 else 0,
            1 if apply_topk_weights else 0, _stream_ptr()))


def m_grouped_fp8_gemm_nt_contiguous(a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor],
                                     d: torch.Tensor, m_indices: torch.Tensor, check: bool = False) -> torch.Tensor:
    """d[row] = bf16((a_fp8[row] . w[e]^T) * a_scale[row] * w_scale[e]) with e = m_indices[row]: the grouped GEMM of the
    reference test's split baseline (its external `deepgemm.m_grouped_fp8_gemm_nt_contiguous`,
    tests/test_mega_moe_dcu.py:245-250) with per-row and per-output-channel fp32 scales.  Rows are grouped by expert,
    groups padded to 128 rows, padding rows have m_indices -1 and are left untouched.  The weight may be plain
    [E, N, K] e4m3 (re-packed once and cached) or already tiled (pack_weights_tiled(w, "l2")).
    check=True synchronises and raises if a 128-row block mixed experts."""
    (a_q, a_s), (w, w_s) = a, b
    for t in (a_q, a_s, w, w_s, d, m_indices):
        _require_cuda(t, "m-grouped GEMM tensors")
    if a_q.dtype != torch.float8_e4m3fn or w.dtype != torch.float8_e4m3fn or d.dtype != torch.bfloat16:
        raise RuntimeError("m-grouped GEMM expects e4m3 operands and a bf16 output")
    if a_s.dtype != torch.float32 or w_s.dtype != torch.float32 or m_indices.dtype != torch.int32:
        raise RuntimeError("m-grouped GEMM expects fp32 scales and int32 m_indices")
    rows, k = a_q.shape
    e, n = w_s.shape
    if d.shape != (rows, n) or a_s.numel() != rows or m_indices.numel() != rows:
        raise RuntimeError("m-grouped GEMM shape mismatch")
    if not (a_q.is_contiguous() and a_s.is_contiguous() and w_s.is_contiguous() and d.is_contiguous() and m_indices.is_contiguous()):
        raise RuntimeError("m-grouped GEMM tensors must be contiguous")
    if w.size(0) != e:
        raise RuntimeError("m-grouped GEMM: weight and scale disagree on the number of experts")
    w_tiled = _tiled_weight(w, n, k, "l2")
    work = torch.empty((32 + 2 * (rows // _lib.BLOCK_M) + 2,), dtype=torch.int32, device=a_q.device)
    with torch.cuda.device(a_q.device):
        _lib.check(_lib.lib().mm_m_grouped_fp8_gemm_nt_contiguous(
            a_q.data_ptr(), a_s.data_ptr(), w_tiled.data_ptr(), w_s.data_ptr(), d.data_ptr(), m_indices.data_ptr(),
            rows, n, k, e, work.data_ptr(), _stream_ptr()))
        if check:
            out = (ctypes.c_int32 * 5)()
            _lib.check(_lib.lib().mm_read_status(work.data_ptr(), _stream_ptr(), out))
            if out[0] != 0:
                raise _lib.MegaMoeError(f"device status {out[0]} ({_lib.STATUS_NAMES.get(out[0], '?')}): block={out[2]} "
                                        f"expert={out[3]} valid rows={out[4]}")
    return d


def swiglu_quant_channelwise_out(x: torch.Tensor, topk_weights: Optional[torch.Tensor], out_fp8: torch.Tensor,
                                 out_scale: torch.Tensor, out_bf16: Optional[torch.Tensor], *, num_per_channels: int,
                                 use_col_major_scales: bool = False, round_scale: bool = False, ue8m0_scale: bool = False,
                                 output_bf16: bool = False, clamp_value: Optional[float] = 10.0,
                                 row_combine_ptrs: Optional[torch.Tensor] = None, verbose_build: bool = False):
    """SwiGLU x route weight + per-row FP8 quantisation of a [rows, 2*hidden] bf16 (gate | up) tensor: the K2 step of the
    reference's staged path and split baseline (megamoe/dcu_megamoe_large_opt/K2_fused/k2_fused.py:12-58)."""
    if x.dim() != 2:
        raise ValueError("x must be [rows, 2 * hidden]")
    hidden = x.shape[1] // 2
    if x.shape[1] != hidden * 2:
        raise ValueError("x hidden dimension must be even")
    if num_per_channels != hidden:
        raise ValueError("K2 fused currently implements channelwise one-scale-per-row quant only")
    if use_col_major_scales:
        raise ValueError("K2 fused currently supports use_col_major_scales=False only")
    if round_scale:
        raise ValueError("K2 fused currently supports round_scale=False only")
    if ue8m0_scale:
        raise ValueError("K2 fused currently supports ue8m0_scale=False only")
    _require_cuda(x, "x")
    if x.dtype != torch.bfloat16 or out_fp8.dtype != torch.float8_e4m3fn or out_scale.dtype != torch.float32:
        raise RuntimeError("swiglu_quant expects bf16 input, e4m3 output and fp32 scales")
    rows = x.shape[0]
    if tuple(out_fp8.shape) != (rows, hidden) or out_scale.numel() != rows or not out_fp8.is_contiguous() or not out_scale.is_contiguous():
        raise RuntimeError("swiglu_quant output shape mismatch")
    if output_bf16 and (out_bf16 is None or tuple(out_bf16.shape) != (rows, hidden) or out_bf16.dtype != torch.bfloat16
                        or not out_bf16.is_contiguous()):
        raise RuntimeError("output_bf16=True needs a contiguous bf16 [rows, hidden] out_bf16")
    x = x.contiguous()
    w = topk_weights.contiguous() if topk_weights is not None and topk_weights.numel() else None
    if w is not None and (w.dtype != torch.float32 or w.numel() != rows):
        raise RuntimeError("topk_weights must be fp32 [rows]")
    ptrs = row_combine_ptrs.contiguous() if row_combine_ptrs is not None else None
    if ptrs is not None and (ptrs.dtype != torch.int64 or ptrs.numel() != rows):
        raise RuntimeError("row_combine_ptrs must be int64 [rows]")
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mm_swiglu_quant_channelwise(
            x.data_ptr(), w.data_ptr() if w is not None else None, ptrs.data_ptr() if ptrs is not None else None,
            out_fp8.data_ptr(), out_scale.data_ptr(), out_bf16.data_ptr() if output_bf16 else None, rows, hidden,
            1 if clamp_value is not None else 0, float(clamp_value or 0.0), _stream_ptr()))
    out_scale_view = out_scale.view(1, rows)
    if output_bf16:
        return out_fp8, out_scale_view, out_bf16
    return out_fp8, out_scale_view


__all__ = [
    "SymmBuffer",
    "cast_to_fp8_channelwise",
    "cast_grouped_weight_to_fp8_channelwise",
    "weight8bit_nt_kpack2_marlin",
    "get_mega_moe_hip_build_config",
    "get_symm_buffer_for_mega_moe",
    "transform_fp8_weights_for_mega_moe",
    "pack_weights_tiled",
    "unpack_weights_tiled",
    "deepep_deepgemm_preprocess_channelwise",
    "deepep_deepgemm_postprocess_channelwise",
    "m_grouped_fp8_gemm_nt_contiguous",
    "swiglu_quant_channelwise_out",
    "fp8_mega_moe",
    "fp8_w8a8_mega_moe",
    "fill_inputs_from_router",
    "RECIPE_UE8M0_PER32",
]
