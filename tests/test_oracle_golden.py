"""Pins the CPU oracle against fixtures generated from the reference itself
(tests/golden/make_golden.py): the reference's pure-torch fake-quant branches,
its EMA / qparam code, its CPU LUT-BGEMM operator and its LRE slope generator."""

import numpy as np
import pytest

from oracle import c_oracle, lut_oracle as lo


def test_fakequant_symmetric_matches_reference(golden):
    g = golden("fakequant")
    for tag in "abcd":
        x, s = g[f"sym_{tag}_x"], g[f"sym_{tag}_scale"]
        qmin, qmax = g[f"sym_{tag}_qrange"]
        q, mask = lo.fakequant_sym(x, s, qmin, qmax)
        np.testing.assert_array_equal(q, g[f"sym_{tag}_q"])
        gx = lo.fakequant_bwd(g[f"sym_{tag}_go"], mask, s)
        np.testing.assert_array_equal(gx, g[f"sym_{tag}_gx"])


def test_fakequant_asymmetric_matches_reference(golden):
    g = golden("fakequant")
    for tag in "ab":
        qmin, qmax = g[f"asym_{tag}_qrange"]
        q, mask = lo.fakequant_asym(g[f"asym_{tag}_x"], g[f"asym_{tag}_scale"],
                                    g[f"asym_{tag}_zero"], qmin, qmax)
        np.testing.assert_array_equal(q, g[f"asym_{tag}_q"])
        gx = lo.fakequant_bwd(g[f"asym_{tag}_go"], mask, g[f"asym_{tag}_scale"])
        np.testing.assert_array_equal(gx, g[f"asym_{tag}_gx"])


def test_fakequant_per_channel_matches_reference(golden):
    g = golden("fakequant")
    w = g["pc_w"]
    for bits in range(3, 9):
        qm = 2 ** (bits - 1) - 1
        sc = g[f"pc_{bits}_scale"]
        np.testing.assert_array_equal(lo.weight_absmax_scale(w, bits), sc)
        q, mask = lo.fakequant_sym(w, sc.reshape(-1, 1, 1, 1), -qm, qm)
        np.testing.assert_array_equal(q, g[f"pc_{bits}_q"])
        gx = lo.fakequant_bwd(g[f"pc_{bits}_go"], mask, sc.reshape(-1, 1, 1, 1))
        np.testing.assert_array_equal(gx, g[f"pc_{bits}_gx"])
    q, _ = lo.fakequant_asym(w, g["pca_scale"].reshape(-1, 1, 1, 1),
                             g["pca_zero"].reshape(-1, 1, 1, 1), 0, 255)
    np.testing.assert_array_equal(q, g["pca_q"])


def test_ema_and_qparams_match_reference(golden):
    g = golden("stats")
    for bits in (8, 5, 4, 3):
        w = g[f"i8_{bits}_w"].copy()
        sw = lo.weight_absmax_scale(w, bits)
        np.testing.assert_array_equal(sw, g[f"i8_{bits}_scale_w0"])
        sx = np.float32(1.0)
        for step in range(3):
            w = (w * np.float32(1.1)).astype(np.float32)
            sx = lo.ema_scale_x(np.abs(g[f"i8_{bits}_xs"][step]).max(), sx, 0.1)
            sw = lo.ema(lo.weight_absmax_scale(w, bits, old=sw), sw, 0.1)
            np.testing.assert_array_equal(sx, g[f"i8_{bits}_scale_x"][step])
            np.testing.assert_array_equal(sw, g[f"i8_{bits}_scale_w"][step])
    sc, zp = lo.uint8_qparams(g["qp_mn"], g["qp_mx"])
    np.testing.assert_array_equal(sc, g["qp_scale"])
    np.testing.assert_array_equal(zp, g["qp_zero"])
    # uint8 layer statistics: EMA on min/max, qparams recomputed after each step
    w = g["u8_w"]
    xmin, xmax = np.float32(0.0), np.float32(1.0)
    wmin = w.reshape(6, -1).min(axis=1)
    wmax = w.reshape(6, -1).max(axis=1)
    for step in range(3):
        x = g["u8_xs"][step]
        xmin = lo.ema(x.min(), xmin, 0.25)
        xmax = lo.ema(x.max(), xmax, 0.25)
        wmin = lo.ema(w.reshape(6, -1).min(axis=1), wmin, 0.25)
        wmax = lo.ema(w.reshape(6, -1).max(axis=1), wmax, 0.25)
        sx, zx = lo.uint8_qparams(xmin, xmax)
        sw, zw = lo.uint8_qparams(wmin, wmax)
        state = np.concatenate([[xmin], [xmax], [sx], [zx], wmin, wmax, sw, zw]).astype(np.float32)
        np.testing.assert_array_equal(state, g["u8_state"][step])


@pytest.mark.parametrize("name", ["affine", "noisy", "trunc4", "utrunc6"])
def test_bgemm_matches_reference_cpu_operator(golden, name):
    g = golden("bgemm_ref_cpu")
    lut = g[f"lut_{name}"]
    for si in range(4):
        x, w, y = g[f"{name}_{si}_x"], g[f"{name}_{si}_w"], g[f"{name}_{si}_y"]
        np.testing.assert_array_equal(lo.bgemm_exact(x, w, lut), y.astype(np.int64))
        np.testing.assert_array_equal(c_oracle.bgemm_u8(x, w, lut), y.astype(np.float64))
        np.testing.assert_array_equal(lo.bgemm_f32_ascending(x, w, lut), y.astype(np.float32))


def test_signed_offset_rule_matches_reference(golden):
    g = golden("bgemm_ref_cpu")
    x, w = g["int8_x"], g["int8_w"]
    y = lo.bgemm_exact(lo.index_of(x, True), lo.index_of(w, True), g["lut_affine"])
    np.testing.assert_array_equal(y, g["int8_y"].astype(np.int64))
    # fp32 integer-valued operands take the same route through the rounding prepass
    y2 = lo.bgemm_exact(lo.to_lut_index(x.astype(np.float32), 128),
                        lo.to_lut_index(w.astype(np.float32), 128), g["lut_affine"])
    np.testing.assert_array_equal(y2, y)


def test_conv_layer_matches_reference_pieces(golden):
    g = golden("conv_layer")
    x, w, lut = g["x"], g["w"], g["lut"]
    O = w.shape[0]
    for bits in (8, 4):
        qm = 2 ** (bits - 1) - 1
        sw = lo.weight_absmax_scale(w, bits)
        np.testing.assert_array_equal(sw, g[f"b{bits}_scale_w"])
        xq, _ = lo.fakequant_sym(x, g["scale_x"], -127, 127)
        wq, _ = lo.fakequant_sym(w, sw.reshape(-1, 1, 1, 1), -qm, qm)
        for s, p in ((1, 1), (2, 0)):
            cols = lo.im2col_index(lo.to_lut_index(xq, 128), 3, 3, s, s, p, p)
            yint = lo.bgemm_exact(cols, lo.to_lut_index(wq.reshape(O, -1), 128), lut)
            np.testing.assert_array_equal(yint, g[f"b{bits}_s{s}p{p}_yint"].astype(np.int64))
            OH = (x.shape[2] + 2 * p - 3) // s + 1
            y = lo.dequant(yint.reshape(x.shape[0], O, OH, OH), g["scale_x"], sw, g["bias"])
            np.testing.assert_allclose(y, g[f"b{bits}_s{s}p{p}_y"], rtol=1e-6, atol=1e-6)


def test_lre_slopes_match_reference(golden):
    g = golden("setup")
    dx, dw = lo.lre_slopes(g["lut"])
    np.testing.assert_allclose(dx, g["lre_grad_a"], rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(dw, g["lre_grad_b"], rtol=2e-5, atol=2e-5)


def test_known_answer_constructions():
    rng = np.random.default_rng(0)
    x = rng.integers(-128, 128, (2, 19, 23)).astype(np.int8)
    w = rng.integers(-128, 128, (7, 19)).astype(np.int8)
    xi, wi = lo.index_of(x, True), lo.index_of(w, True)
    # exact-product table == integer einsum
    y = lo.bgemm_exact(xi, wi, lo.lut_exact_signed())
    ref = np.einsum("nkl,ok->nol", x.astype(np.int64), w.astype(np.int64))
    np.testing.assert_array_equal(y, ref)
    # unsigned op on raw indices == signed op on (v - 128) with the same table
    y_aff = lo.bgemm_exact(xi, wi, lo.lut_affine_asymmetric())
    swapped = lo.bgemm_exact(xi, wi, lo.lut_affine_asymmetric().T)
    assert not np.array_equal(y_aff, swapped)
    assert lo.lut_class(lo.lut_exact_signed()) == "i16"
    assert lo.lut_class(lo.lut_exact_unsigned()) == "u16"
    assert lo.lut_class(lo.lut_exact_signed() * 0.5) == "f32"
    t = lo.lut_exact_signed().copy(); t[0, 0] = 32768
    assert lo.lut_class(t) == "f32"          # mixed sign beyond int16
    # gradients: exact-derivative custom tables reduce to the STE einsum pair
    go = rng.standard_normal((2, 7, 23))
    DX = np.broadcast_to(np.arange(-128, 128, dtype=np.float64)[None, :], (256, 256))
    DW = np.broadcast_to(np.arange(-128, 128, dtype=np.float64)[:, None], (256, 256))
    gx, gw = lo.custom_backward(go, xi, wi, DX, DW)
    sx, sw = lo.ste_backward(go, xi, wi)
    np.testing.assert_allclose(gx, sx, rtol=1e-12, atol=1e-9)
    np.testing.assert_allclose(gw, sw, rtol=1e-12, atol=1e-9)
    # fold == torch.nn.functional.fold
    import torch
    cols = rng.standard_normal((2, 27, 9))
    ours = lo.fold(cols, 3, 6, 5, 3, 3, 2, 1, 1, 0, 1, 1)
    ref = torch.nn.functional.fold(torch.from_numpy(cols), (6, 5), (3, 3), dilation=(1, 1),
                                   padding=(1, 0), stride=(2, 1)).numpy()
    np.testing.assert_allclose(ours, ref, rtol=1e-12, atol=1e-12)
