"""Generate the golden fixtures under tests/golden/.

Run where a checkout of the reference project is available, giving its root directory:

    python tests/golden/make_golden.py <reference root>          # or MEGAMOE_REFERENCE_ROOT=<reference root>

    python tests/golden/make_golden.py <reference root> --only ue8m0     # just ref_ue8m0.npz

Three kinds of fixture are written:

* ``ref_quant.npz`` -- outputs of the REFERENCE'S OWN torch helpers (``megamoe/__init__.py``:
  ``cast_to_fp8_channelwise``, ``cast_grouped_weight_to_fp8_channelwise``, ``weight8bit_nt_kpack2_marlin``,
  ``transform_fp8_weights_for_mega_moe``, ``_large_opt_3stage_selected``) on seeded inputs.  The reference package
  imports a HIP extension ``megamoe._C`` at import time; a stub module with that name is installed first so the
  pure-torch helpers can be imported unmodified.  These vectors pin the oracle's quantisation stages.
* ``ref_ue8m0.npz`` -- outputs of the reference's torch helper ``per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=32)``
  (``deep_gemm/utils/math.py:13-37``, loaded from its file: the package itself imports a CUDA extension) on seeded
  inputs: e4m3 codes and power-of-two scales per (row, 32 columns).  Pins ``oracle.moe_oracle.ue8m0_block_quant``.
* ``layer_small.npz`` -- inputs and outputs of the CPU oracle (oracle/moe_oracle.py) for the small configuration
  (256 tokens, hidden 512, intermediate 256, 8 experts, top-2, seed 0) and a 2-rank variant.  The reference has no
  runnable implementation of the layer, so these are regression vectors of the restatement, not reference outputs.
"""
import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def import_reference_megamoe(ref_root: str):
    stub = types.ModuleType("megamoe._C")
    stub.init = lambda *a, **k: None
    stub.get_token_alignment_for_mega_moe = lambda: 384
    saved = {k: sys.modules.get(k) for k in ("megamoe", "megamoe._C")}
    sys.path.insert(0, ref_root)
    try:
        sys.modules.pop("megamoe", None)
        sys.modules["megamoe._C"] = stub
        mod = importlib.import_module("megamoe")
        assert os.path.realpath(mod.__file__).startswith(os.path.realpath(ref_root)), mod.__file__
        return mod
    finally:
        sys.path.remove(ref_root)
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def edge_values():
    """Every e4m3 code point, its neighbours' midpoints (exact ties), +-1 fp32 ulp around them, 0, +-448."""
    codes = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    codes = codes[torch.isfinite(codes)]
    pos = torch.unique(codes.abs())
    mids = (pos[:-1] + pos[1:]) / 2
    base = torch.cat([pos, mids])
    up = torch.nextafter(base, torch.full_like(base, 1e9))
    dn = torch.nextafter(base, torch.full_like(base, -1e9))
    allv = torch.cat([base, up, dn])
    allv = allv[allv <= 448.0]
    return torch.cat([allv, -allv]).contiguous()


def write_ue8m0(ref_root: str):
    import importlib.util
    spec = importlib.util.spec_from_file_location("_ref_dg_math", os.path.join(ref_root, "deep_gemm", "utils", "math.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    g = torch.Generator().manual_seed(7)
    x = torch.randn((48, 256), generator=g)
    x *= torch.exp2(torch.randint(-8, 9, (48, 1), generator=g).float())          # rows over 16 octaves
    # blocks whose amax sits on, just below and just above a scale boundary (448 * 2^e), and a block of small values
    for i, (e, f) in enumerate([(0, 1.0), (0, 1.0 - 2.0 ** -24), (0, 1.0 + 2.0 ** -23), (-3, 1.0), (5, 1.0 + 2.0 ** -23), (2, 0.75)]):
        x[i, :32] = torch.linspace(-0.9, 0.9, 32) * 448.0 * 2.0 ** e
        x[i, 7] = 448.0 * 2.0 ** e * f
    x[6, 32:64] = torch.linspace(-1, 1, 32) * 3e-4                                # above the helper's 1e-4 floor on amax
    q, sf = m.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=32)
    out = {"x": x.numpy(), "q": q.view(torch.uint8).numpy(), "sf": sf.numpy()}
    np.savez_compressed(os.path.join(HERE, "ref_ue8m0.npz"), **out)
    print("wrote ref_ue8m0.npz", {k: v.shape for k, v in out.items()})


def main():
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    ref_root = args[0] if args else os.environ.get("MEGAMOE_REFERENCE_ROOT")
    if not ref_root or not os.path.isdir(ref_root):
        raise SystemExit("usage: make_golden.py <root of the reference checkout> [--only ue8m0]")
    if "--only" in sys.argv:
        what = sys.argv[sys.argv.index("--only") + 1]
        if what != "ue8m0":
            raise SystemExit("--only knows: ue8m0")
        write_ue8m0(ref_root)
        return
    write_ue8m0(ref_root)
    ref = import_reference_megamoe(ref_root)
    out = {}
    g = torch.Generator().manual_seed(0)

    # (1) per-token cast: bf16 N(0,1), a tiny-amplitude row (1e-4 floor), an all-zero row, a large row
    x = torch.randn((24, 512), generator=g).to(torch.bfloat16)
    x[3] *= 1e-6
    x[5] = 0
    x[7] *= 300.0
    q, s = ref.cast_to_fp8_channelwise(x)
    out["x_bf16_bits"] = x.view(torch.int16).numpy()
    out["x_q"] = q.view(torch.uint8).numpy()
    out["x_scale"] = s.numpy()

    # (2) rounding edge cases: a row whose amax is exactly 448 so that scale == 1 and codes are direct casts
    ev = edge_values()
    pad = (-ev.numel()) % 16
    row = torch.cat([ev, torch.zeros(pad)])
    row[-1] = 448.0
    q2, s2 = ref.cast_to_fp8_channelwise(row.view(1, -1))
    out["edge_x"] = row.numpy()
    out["edge_q"] = q2.view(torch.uint8).numpy()
    out["edge_scale"] = s2.numpy()

    # (3) grouped weights + Marlin permutation + the full transform
    w1 = (torch.randn((3, 64, 128), generator=g) / 128 ** 0.5).to(torch.bfloat16)
    w2 = (torch.randn((3, 128, 32), generator=g) / 32 ** 0.5).to(torch.bfloat16)
    wq, ws = ref.cast_grouped_weight_to_fp8_channelwise(w1)
    out["w1_bf16_bits"] = w1.view(torch.int16).numpy()
    out["w2_bf16_bits"] = w2.view(torch.int16).numpy()
    out["w1_q"] = wq.view(torch.uint8).numpy()
    out["w1_scale"] = ws.numpy()
    out["w1_marlin"] = ref.weight8bit_nt_kpack2_marlin(wq).view(torch.uint8).numpy()
    (t1, t1s), (t2, t2s) = ref.transform_fp8_weights_for_mega_moe(w1, w2)
    out["t1"] = t1.view(torch.uint8).numpy(); out["t1s"] = t1s.numpy()
    out["t2"] = t2.view(torch.uint8).numpy(); out["t2s"] = t2s.numpy()

    # (4) the fused/staged selector
    sel = []
    for mode in ("force", "auto", "off"):
        for n in (0, 1, 127, 128, 129, 4096):
            sel.append((mode, n, 128, bool(ref._large_opt_3stage_selected(n, mode, 128))))
    out["selector_modes"] = np.array([m for m, *_ in sel])
    out["selector_tokens"] = np.array([n for _, n, *_ in sel], dtype=np.int64)
    out["selector_result"] = np.array([r for *_, r in sel], dtype=np.bool_)
    np.savez_compressed(os.path.join(HERE, "ref_quant.npz"), **out)
    print("wrote ref_quant.npz", {k: v.shape for k, v in out.items()})

    # ---- oracle regression vectors for the layer --------------------------------------------
    from oracle import moe_oracle as orc

    layer = {}
    for tag, R in (("r1", 1), ("r2", 2)):
        E, K, H, I, T = 8, 2, 512, 256, 256
        xs, sx, idx, wt, w1q, w1s, w2q, w2s = [], [], [], [], [], [], [], []
        for r in range(R):
            xb = orc.make_inputs(T // R, H, seed=0 + r)
            q_, s_ = orc.cast_to_fp8_channelwise(xb)
            i_, w_ = orc.make_routing(T // R, E, K, seed=100 + r)
            a, b = orc.make_weights(E // R, H, I, seed=200 + r)
            aq, as_ = orc.cast_grouped_weight_to_fp8_channelwise(a)
            bq, bs_ = orc.cast_grouped_weight_to_fp8_channelwise(b)
            xs.append(q_); sx.append(s_); idx.append(i_); wt.append(w_)
            w1q.append(aq); w1s.append(as_); w2q.append(bq); w2s.append(bs_)
        for variant in ("fused", "staged"):
            for clamp in (None, 10.0):
                ys, lay, _ = orc.moe_layer(xs, sx, idx, wt, w1q, w1s, w2q, w2s, E, clamp, variant)
                key = f"{tag}_{variant}_{'noclamp' if clamp is None else 'clamp10'}"
                # first 16 tokens of every rank (bf16 bit patterns); fp32 summation order may differ between
                # hosts, so the regression test compares these within a tolerance, not bit for bit
                layer[key + "_y_bits"] = np.stack([y[:16].view(torch.int16).numpy() for y in ys])
        layer[tag + "_counts"] = lay.counts
        layer[tag + "_pool_off"] = lay.pool_off
        layer[tag + "_dest_row"] = np.stack(lay.dest_row)
    np.savez_compressed(os.path.join(HERE, "layer_small.npz"), **layer)
    print("wrote layer_small.npz", {k: v.shape for k, v in layer.items()})


if __name__ == "__main__":
    main()
