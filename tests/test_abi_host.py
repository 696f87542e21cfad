"""Host-side checks that need no GPU: the library loads, exports every declared symbol, and its layout arithmetic."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "megamoe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_lib):
    from deepgemm_b200 import _lib
    declared = _declared_symbols()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(built_lib, name), f"{name} declared in include/megamoe_b200.h but not exported"
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared


def test_token_alignment_and_build_config(built_lib):
    from deepgemm_b200 import _lib
    assert built_lib.mm_token_alignment() == 384
    cfg = _lib.build_config()
    assert cfg["operator"] == "fp8_w8a8_mega_moe" and cfg["arch"] == "sm_100a"
    assert cfg["weight_scale_mode"] == "channelwise_fp32"


def test_symm_layout_regions_are_disjoint_and_sized(built_lib):
    from deepgemm_b200 import _lib
    R, E, T, K, H, I = 8, 256, 8448, 6, 4096, 2048
    off, total = _lib.symm_buffer_layout(R, E, T, K, H, I)
    sizes = {"peer_ptrs": 8 * 16, "signals": 4 * 4 * 16, "runtime_num_tokens": 4, "count_matrix": 4 * R * E, "x": T * H,
             "x_sf": 4 * T, "topk_idx": 8 * T * K, "topk_weights": 4 * T * K, "pool_x": off["pool_rows"] * H,
             "pool_meta": 16 * off["pool_rows"], "combine": 2 * K * T * H}
    order = sorted(sizes, key=lambda k: off[k])
    for a, b in zip(order, order[1:]):
        assert off[a] + sizes[a] <= off[b], (a, b)
    assert off[order[-1]] + sizes[order[-1]] <= total
    for k in sizes:
        assert off[k] % 256 == 0
    # worst case: every route of every rank lands on this rank, plus per-expert padding to 128 rows
    assert off["pool_rows"] >= R * T * K + (E // R) * 127 and off["pool_rows"] % 128 == 0
    # the caller-visible part equals the reference's formula (csrc/apis/mega_dcu.hpp:104-116) up to alignment
    assert sizes["combine"] == K * T * H * 2


def test_scratch_layout_regions(built_lib):
    from deepgemm_b200 import _lib
    R, E, T, K, H, I = 2, 8, 384, 2, 512, 256
    off, total = _lib.scratch_layout(R, E, T, K, H, I)
    rows = _lib.symm_buffer_layout(R, E, T, K, H, I)[0]["pool_rows"]
    assert off["act_fp8"] + rows * I <= total
    assert off["act_bf16"] + rows * I * 2 <= off["act_fp8"]
    assert off["route_blocks"] == (T * K + 255) // 256


@pytest.mark.parametrize("args", [
    (0, 8, 384, 2, 512, 256), (3, 8, 384, 2, 512, 256), (1, 8, 384, 2, 500, 256), (1, 8, 384, 2, 512, 200),
    (1, 8, 384, 40, 512, 256), (1, 2048, 384, 2, 512, 256), (17, 34, 384, 2, 512, 256),
])
def test_bad_shapes_are_rejected_with_a_message(built_lib, args):
    from deepgemm_b200 import _lib
    with pytest.raises(_lib.MegaMoeError):
        _lib.symm_buffer_layout(*args)
    assert built_lib.mm_last_error()


def test_layer_entry_point_validates_before_touching_the_device(built_lib):
    """Argument errors are reported without any CUDA call (so this runs on a machine without a GPU)."""
    peers = (ctypes.c_uint64 * 16)(0x1000)
    rc = built_lib.mm_fp8_w8a8_mega_moe(0x10, 0x10, 0x10, 0x10, 0x10, None, 0x1000, 0x10, peers, 0, 1, 384, 8, 500, 2, 512, 256,
                                        float("inf"), 0, None, None)
    assert rc != 0 and b"too many tokens" in built_lib.mm_last_error()
    rc = built_lib.mm_fp8_w8a8_mega_moe(0x10, 0x10, 0x10, 0x10, 0x10, None, 0x2000, 0x10, peers, 0, 1, 384, 8, 10, 2, 512, 256,
                                        float("inf"), 0, None, None)
    assert rc != 0 and b"peer_ptrs" in built_lib.mm_last_error()
    rc = built_lib.mm_quant_per_token(0x10, 4, 12, 0x10, 0x10, None)
    assert rc != 0


def test_python_api_surface_and_selector():
    import megamoe
    import numpy as np
    for name in ["SymmBuffer", "cast_to_fp8_channelwise", "cast_grouped_weight_to_fp8_channelwise",
                 "weight8bit_nt_kpack2_marlin", "get_mega_moe_hip_build_config", "get_symm_buffer_for_mega_moe",
                 "transform_fp8_weights_for_mega_moe", "deepep_deepgemm_preprocess_channelwise",
                 "deepep_deepgemm_postprocess_channelwise", "fp8_mega_moe", "fp8_w8a8_mega_moe"]:
        assert hasattr(megamoe, name)
    assert megamoe.fp8_w8a8_mega_moe is megamoe.fp8_mega_moe
    gold = np.load(os.path.join(ROOT, "tests", "golden", "ref_quant.npz"))
    for mode, n, want in zip(gold["selector_modes"], gold["selector_tokens"], gold["selector_result"]):
        assert megamoe._large_opt_3stage_selected(int(n), str(mode), 128) == bool(want)


def test_variant_choice_follows_the_reference_rule():
    """Staged above the token threshold, decided on dispatch_num_tokens if given, else on the rows of y -- the rule of the
    reference (megamoe/__init__.py:398-404).  Ranks holding different token counts agree by passing one
    dispatch_num_tokens, as the reference asks of its callers."""
    from deepgemm_b200.megamoe import _eager_variant_is_staged as sel
    assert sel("auto", 128, 7, None) is False
    assert sel("auto", 128, 133, None) is True
    assert sel("auto", 128, 128, None) is False                      # at the threshold: still fused
    # an explicit dispatch_num_tokens (the same on every rank) wins over the rank's own count
    assert sel("auto", 128, 7, 133) is True and sel("auto", 128, 133, 64) is False
    assert sel("auto", 128, 133, 0) is False
    # forced modes ignore the counts; there is no route ceiling on the fused variant any more
    assert sel("force", 128, 1, None) is True and sel("off", 128, 100000, None) is False


def test_packed_weight_cache_is_bound_to_the_tensor_object():
    """A freed weight's address, shape and version counter can all recur in the next weight tensor; the cache of re-packed
    weights must then miss (it is valid only for the tensor object it was filled from)."""
    import weakref
    import torch
    from deepgemm_b200 import megamoe as mm
    g = torch.Generator().manual_seed(3)
    w_old = torch.randint(0, 120, (2, 512, 128), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
    w_new = torch.randint(0, 120, (2, 512, 128), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
    packed_old = mm._tiled_weight(w_old, 512, 128, "l2")
    assert mm._tiled_weight(w_old, 512, 128, "l2") is packed_old                      # same object: served from the cache
    # plant w_old's packing under the key w_new would look up, as an address-reusing allocator would
    mm._packed_weight_cache[(w_new.data_ptr(), tuple(w_new.shape), w_new._version, "l2")] = (weakref.ref(w_old), packed_old)
    packed_new = mm._tiled_weight(w_new, 512, 128, "l2")
    assert torch.equal(mm.unpack_weights_tiled(packed_new, "l2", 512).view(torch.uint8), w_new.view(torch.uint8))
    assert not torch.equal(packed_new.view(torch.uint8), packed_old.view(torch.uint8))
    # the two packings of one tensor are cached separately
    assert not torch.equal(mm._tiled_weight(w_new, 512, 128, "l1").view(torch.uint8), packed_new.view(torch.uint8))


def test_marlin_helper_matches_reference_fixture():
    import megamoe
    import numpy as np
    import torch
    gold = np.load(os.path.join(ROOT, "tests", "golden", "ref_quant.npz"))
    q = torch.from_numpy(gold["w1_q"].copy()).view(torch.float8_e4m3fn)
    m = megamoe.weight8bit_nt_kpack2_marlin(q)
    assert np.array_equal(m.view(torch.uint8).numpy(), gold["w1_marlin"])
    with pytest.raises(ValueError):
        megamoe.weight8bit_nt_kpack2_marlin(q, k_tile=8)


def test_cpu_tensors_are_refused():
    import megamoe
    import torch
    with pytest.raises(RuntimeError):
        megamoe.cast_to_fp8_channelwise(torch.zeros((2, 16), dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        megamoe.cast_to_fp8_channelwise(torch.zeros((16,), dtype=torch.bfloat16))


def _tile_order(lib, num_mblocks, wave_m, nb1, nb2, interleave):
    import numpy as np
    n = num_mblocks * (nb1 + nb2)
    out = np.zeros((max(n, 1), 3), dtype=np.int32)
    rc = lib.mm_tile_order(num_mblocks, wave_m, nb1, nb2, int(interleave), out.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)))
    assert rc == 0, lib.mm_last_error()
    return out[:n]


@pytest.mark.parametrize("interleave", [True, False])
def test_tile_order_is_a_permutation_with_backward_dependencies(built_lib, interleave):
    """The layer kernel's tile order, produced by the same code the device runs (mm_tile_order): every GEMM1 and GEMM2
    tile exactly once; every GEMM2 tile of an m-block after ALL GEMM1 tiles of that m-block (the kernel's waits then only
    ever point at earlier tiles, which is what rules out a cycle); GEMM1 m-blocks start in ascending order (the order the
    requantisation units are claimed in)."""
    import numpy as np
    rng = np.random.default_rng(0)
    shapes = [(0, 3, 16, 16), (1, 1, 1, 1), (1, 19, 16, 16), (2, 1, 3, 2), (32, 19, 16, 16), (192, 19, 16, 16), (257, 7, 2, 5),
              (40, 1 << 28, 16, 16), (5, 2, 1, 9), (64, 3, 9, 1)]
    shapes += [tuple(int(v) for v in (rng.integers(1, 300), rng.integers(1, 40), rng.integers(1, 20), rng.integers(1, 20))) for _ in range(40)]
    for num_mblocks, wave_m, nb1, nb2 in shapes:
        order = _tile_order(built_lib, num_mblocks, wave_m, nb1, nb2, interleave)
        assert order.shape[0] == num_mblocks * (nb1 + nb2)
        if num_mblocks == 0:
            continue
        kind, mb, nb = order[:, 0], order[:, 1], order[:, 2]
        assert set(np.unique(kind)) <= {0, 1}
        g1 = np.nonzero(kind == 0)[0]; g2 = np.nonzero(kind == 1)[0]
        key1 = mb[g1].astype(np.int64) * nb1 + nb[g1]
        key2 = mb[g2].astype(np.int64) * nb2 + nb[g2]
        assert np.array_equal(np.sort(key1), np.arange(num_mblocks * nb1)), (num_mblocks, wave_m, nb1, nb2)
        assert np.array_equal(np.sort(key2), np.arange(num_mblocks * nb2)), (num_mblocks, wave_m, nb1, nb2)
        assert (nb[g1] < nb1).all() and (nb[g2] < nb2).all() and (mb >= 0).all() and (mb < num_mblocks).all()
        last_g1 = np.full(num_mblocks, -1); first_g2 = np.full(num_mblocks, order.shape[0])
        np.maximum.at(last_g1, mb[g1], g1)
        np.minimum.at(first_g2, mb[g2], g2)
        assert (last_g1 < first_g2).all(), (num_mblocks, wave_m, nb1, nb2)
        first_g1 = np.full(num_mblocks, order.shape[0]); np.minimum.at(first_g1, mb[g1], g1)
        assert (np.diff(first_g1) > 0).all()


def test_tile_order_keeps_gemm2_three_waves_behind_gemm1(built_lib):
    """Default shape of the order (two rounds of GEMM1 tiles per wave, GEMM2 of wave k beside GEMM1 of wave k + 3): a
    GEMM2 tile of m-block b never comes before the first GEMM1 tile of m-block b + 3 * wave (its requantisation has three
    waves of GEMM1 work to finish behind), and inside a mixed group the two kinds alternate tile by tile."""
    import numpy as np
    num_mblocks, wave_m, nb1, nb2 = 192, 19, 16, 16
    order = _tile_order(built_lib, num_mblocks, wave_m, nb1, nb2, True)
    kind, mb = order[:, 0], order[:, 1]
    first_g1 = np.full(num_mblocks, order.shape[0]); np.minimum.at(first_g1, mb[kind == 0], np.nonzero(kind == 0)[0])
    for t in np.nonzero(kind == 1)[0]:
        ahead = mb[t] // wave_m * wave_m + 3 * wave_m
        if ahead < num_mblocks:
            assert first_g1[ahead] < t
    # the first three waves are GEMM1 only; then the kinds alternate
    assert (kind[:3 * wave_m * nb1] == 0).all()
    mixed = kind[3 * wave_m * nb1: 3 * wave_m * nb1 + 2 * wave_m * nb1]
    assert (mixed[0::2] == 0).all() and (mixed[1::2] == 1).all()
