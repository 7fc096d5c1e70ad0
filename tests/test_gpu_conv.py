"""GPU parity of the approximate Conv2d path: im2col-free forward, fused dequantisation, STE / LRE /
custom backward, the uint8 layer and the depthwise operator, against the oracle and the fixture
composed from reference pieces.  Integer accumulators bit-exact; fp32 outputs / gradients rel 1e-5."""

import numpy as np
import pytest
import torch

from oracle import lut_oracle as lo

pytestmark = pytest.mark.gpu
RTOL = 1e-5


def _t(a, dev):
    a = np.asarray(a)
    return torch.from_numpy(np.ascontiguousarray(a).reshape(a.shape)).to(dev)


def _close(got, ref, rtol=RTOL):
    got = got.detach().cpu().numpy().astype(np.float64) if isinstance(got, torch.Tensor) else got
    scale = max(np.abs(ref).max(), 1e-30)
    assert np.abs(got - ref).max() <= rtol * scale, (np.abs(got - ref).max(), scale)


GEOMS = [  # (B, C, H, W, O, k, s, p, d)
    (2, 3, 8, 8, 4, 3, 1, 1, 1), (1, 16, 12, 10, 24, 3, 2, 1, 1), (2, 8, 9, 9, 5, 1, 1, 0, 1),
    (2, 8, 9, 9, 70, 1, 2, 0, 1), (1, 4, 11, 13, 6, (3, 2), (2, 1), (1, 2), (1, 2)), (3, 5, 7, 7, 9, 5, 1, 2, 1),
    (1, 2, 6, 6, 3, 3, 1, 0, 2), (8, 64, 8, 8, 64, 3, 1, 1, 1),
]


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


@pytest.mark.parametrize("geom", GEOMS)
def test_conv_forward_is_bit_exact(dev, geom):
    from approxtorch_b200.backend import ops
    B, C, H, W, O, k, s, p, d = geom
    (kh, kw), (sh, sw), (ph, pw), (dh, dw) = _pair(k), _pair(s), _pair(p), _pair(d)
    rng = np.random.default_rng(abs(hash(geom)) & 0xffff)
    x8 = rng.integers(-127, 128, (B, C, H, W)).astype(np.int8)
    widx = rng.integers(0, 256, (O, C * kh * kw), dtype=np.uint8)
    lut = lo.lut_signed_noisy(64, seed=5)
    cols = lo.im2col_index(lo.index_of(x8, True), kh, kw, sh, sw, ph, pw, dh, dw, 128)
    ref = lo.bgemm_exact(cols, widx, lut)
    img = ops.lut_image(_t(lut.reshape(-1), dev))
    g4 = ((kh, kw), (sh, sw), (ph, pw), (dh, dw))
    y = ops.lut_conv2d_launch(_t(x8, dev), _t(widx, dev), img, g4, 128)
    np.testing.assert_array_equal(y.flatten(2).cpu().numpy().astype(np.int64), ref)
    # uint8 index image input and a forced split-K give the same integers
    y2 = ops.lut_conv2d_launch(_t(lo.index_of(x8, True), dev), _t(widx, dev), img, g4, 128, cfg=(3 << 16) | 64)
    assert torch.equal(y, y2)
    # identical to the materialised route im2col_u8 -> LUT-BGEMM
    cols_gpu = ops.im2col_u8(_t(x8, dev), (kh, kw), (sh, sw), (ph, pw), (dh, dw))
    y3 = torch.empty_like(y.flatten(2))
    ops.lut_gemm_launch(cols_gpu, _t(widx, dev), img, y3, B, C * kh * kw, cols.shape[2], O)
    assert torch.equal(y.flatten(2), y3)


ROWS_GEOMS = [  # (B, C, H, W, O, k, s, p, d): few pixels, many channels - the shapes the channels-as-rows orientation serves
    (3, 64, 7, 7, 600, 1, 1, 0, 1), (2, 48, 7, 7, 520, 3, 1, 1, 1), (5, 32, 9, 8, 130, 3, 2, 1, 1), (1, 16, 5, 5, 64, 1, 1, 0, 1),
    (2, 20, 6, 7, 1100, (3, 2), 1, (1, 0), 1),
]


@pytest.mark.parametrize("geom", ROWS_GEOMS)
def test_channels_as_rows_orientation_is_bit_identical(dev, geom, monkeypatch):
    """The convolution with the output channels as tile rows (pixel matrix + transposed table) gives the same bits
    as the pixels-as-rows kernel and the int64 oracle: signed table without zero points, unsigned table with the
    zero-point correction, per-channel scale and shift."""
    from approxtorch_b200.backend import ops
    B, C, H, W, O, k, s, p, d = geom
    (kh, kw), (sh, sw), (ph, pw), (dh, dw) = _pair(k), _pair(s), _pair(p), _pair(d)
    g4 = ((kh, kw), (sh, sw), (ph, pw), (dh, dw))
    rng = np.random.default_rng(abs(hash(geom)) & 0xffff)
    K = C * kh * kw
    widx = rng.integers(0, 256, (O, K), dtype=np.uint8)
    alpha = _t(rng.uniform(0.5, 2.0, O).astype(np.float32), dev)
    beta = _t(rng.standard_normal(O).astype(np.float32), dev)

    def both(x8, image, pad, **kw_):
        monkeypatch.setattr(ops, "ROWS_ORIENTATION", False)
        a = ops.lut_conv2d_launch(x8, _t(widx, dev), image, g4, pad, **kw_)
        monkeypatch.setattr(ops, "ROWS_ORIENTATION", True)
        monkeypatch.setattr(ops, "_rows_orientation_wins", lambda R, K_, O_: True)
        calls = []
        real = ops._lut_conv2d_rows
        monkeypatch.setattr(ops, "_lut_conv2d_rows", lambda *a_, **k_: (calls.append(1), real(*a_, **k_))[1])
        b = ops.lut_conv2d_launch(x8, _t(widx, dev), image, g4, pad, **kw_)
        assert calls, "the channels-as-rows path was not taken"
        assert torch.equal(a, b)
        return b

    # signed table, int8 image, plain sums against the oracle
    x8 = rng.integers(-127, 128, (B, C, H, W)).astype(np.int8)
    lut = lo.lut_signed_noisy(64, seed=9)
    lut_dev = _t(lut.reshape(-1), dev)             # kept alive: the transposed image is built from the table tensor
    img = ops.lut_image(lut_dev)
    y = both(_t(x8, dev), img, 128)
    cols = lo.im2col_index(lo.index_of(x8, True), kh, kw, sh, sw, ph, pw, dh, dw, 128)
    np.testing.assert_array_equal(y.flatten(2).cpu().numpy().astype(np.int64), lo.bgemm_exact(cols, widx, lut))
    both(_t(x8, dev), img, 128, alpha=alpha, beta=beta)
    # a table rewritten in place (as a re-broadcast module buffer is): the transposed image follows it
    lut_dev.view(256, 256)[3:40, 100:180] += 2.0
    both(_t(x8, dev), ops.lut_image(lut_dev), 128)
    # unsigned table, uint8 image, zero points (the pad value is the activation zero point)
    xu = rng.integers(0, 256, (B, C, H, W), dtype=np.uint8)
    lutu = lo.lut_unsigned_truncated(6)
    lutu_dev = _t(lutu.reshape(-1), dev)
    imgu = ops.lut_image(lutu_dev)
    zx = torch.tensor(117.0, device=dev)
    zw = _t(rng.integers(0, 256, O).astype(np.float32), dev)
    ws = _t(widx.astype(np.int64).sum(axis=1).astype(np.int32), dev)
    yu = both(_t(xu, dev), imgu, -1, alpha=alpha, beta=beta, zero_x=zx, zero_w=zw, wsum=ws)
    colsu = lo.im2col_index(xu, kh, kw, sh, sw, ph, pw, dh, dw, 117)
    t = lo.uint8_zero_point_correction(lo.bgemm_exact(colsu, widx, lutu), colsu, widx, 117, zw.cpu().numpy().astype(np.int64))
    want = t.astype(np.float32) * alpha.cpu().numpy()[None, :, None] + beta.cpu().numpy()[None, :, None]
    np.testing.assert_allclose(yu.flatten(2).cpu().numpy(), want, rtol=1e-6, atol=1e-3)


def test_layer_matches_fixture_composed_from_reference_pieces(golden, dev):
    import approxtorch_b200 as at
    g = golden("conv_layer")
    x = _t(g["x"], dev)
    lut = _t(g["lut"], dev)
    for bits in (8, 4):
        for s, p in ((1, 1), (2, 0)):
            layer = at.nn.Conv2d_int8(16, 24, 3, lut, bias=True, stride=s, padding=p, weight_bits=bits,
                                      update_scale=False).to(dev)
            with torch.no_grad():
                layer.weight.copy_(_t(g["w"], dev))
                layer.bias.copy_(_t(g["bias"], dev))
                layer.scale_x.copy_(_t(g["scale_x"], dev))
                # the fixture's scales were formed on the CPU; a device division by a constant may differ in the last bit
                layer.scale_w.copy_(_t(g[f"b{bits}_scale_w"], dev))
            y = layer(x)
            ref = g[f"b{bits}_s{s}p{p}_y"]
            np.testing.assert_allclose(y.detach().cpu().numpy(), ref, rtol=1e-6, atol=1e-6 * np.abs(ref).max())
            # integer accumulator: undo the dequantisation through the raw operator chain
            xq = at.nn.quantization.static_quantize_int8(x, layer.scale_x, -127, 127)
            qm = 2 ** (bits - 1) - 1
            wq = at.nn.quantization.static_quantize_int8(layer.weight, layer.scale_w, -qm, qm, ch_axis=0)
            yint = at.nn.bgemm_int8.conv2d_int8_ste(xq, wq.view(24, -1), lut, ((3, 3), (s, s), (p, p), (1, 1), 1))
            np.testing.assert_array_equal(yint.detach().cpu().numpy().astype(np.int32), g[f"b{bits}_s{s}p{p}_yint"])


def _fp64_layer_truth(x, w, bias, lut, scale_x, scale_w, qmax_w, geom, go, mode, dx=None, dw=None):
    """float64 forward / backward of the whole signed layer from the oracle pieces."""
    (kh, kw), (sh, sw), (ph, pw), (dh, dw_) = geom
    B, C, H, W = x.shape
    O = w.shape[0]
    xq, xm = lo.fakequant_sym(x, scale_x, -127, 127)
    wq, wm = lo.fakequant_sym(w, scale_w.reshape(-1, 1, 1, 1), -qmax_w, qmax_w)
    cols = lo.im2col_index(lo.to_lut_index(xq, 128), kh, kw, sh, sw, ph, pw, dh, dw_, 128)
    widx = lo.to_lut_index(wq.reshape(O, -1), 128)
    yint = lo.bgemm_exact(cols, widx, lut).astype(np.float64)
    s = (np.float32(scale_x) * scale_w).astype(np.float64)
    y = yint * s[None, :, None] + (0 if bias is None else bias.astype(np.float64)[None, :, None])
    g = go.reshape(B, O, -1).astype(np.float64) * s[None, :, None]
    if mode == "ste":
        gcols, gw = lo.ste_backward(g, cols, widx)
    elif mode == "lre":
        gcols, gw = lo.lre_backward(g, cols, widx, dx, dw)
    else:
        gcols, gw = lo.custom_backward(g, cols, widx, dx, dw)
    gx = lo.fold(gcols, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw_)
    sx = max(np.float64(np.float32(scale_x)), 1e-12)
    gx = gx * xm / sx
    gw = gw.reshape(w.shape) * wm / np.maximum(scale_w.astype(np.float64), 1e-12).reshape(-1, 1, 1, 1)
    gb = go.astype(np.float64).sum(axis=(0, 2, 3))
    return y, gx, gw, gb


@pytest.mark.parametrize("mode", ["ste", "lre", "custom"])
@pytest.mark.parametrize("geom", [(2, 6, 9, 9, 10, 3, 1, 1, 1), (2, 4, 10, 8, 7, 3, 2, 1, 1), (3, 8, 6, 6, 12, 1, 1, 0, 1),
                                  (1, 3, 9, 11, 5, (3, 2), (2, 1), (1, 2), (1, 2))])
def test_layer_forward_backward_against_fp64_truth(dev, mode, geom):
    import approxtorch_b200 as at
    B, C, H, W, O, k, s, p, d = geom
    g4 = (_pair(k), _pair(s), _pair(p), _pair(d))
    rng = np.random.default_rng(7)
    torch.manual_seed(3)
    lut = lo.lut_signed_noisy(128, seed=4)
    if mode == "lre":
        dx, dw = lo.lre_slopes(lut)
        dw = dw.copy(); dw[128] = 3.25            # a non-zero slope at quantised zero exercises the padding rule
    elif mode == "custom":
        dx = (rng.standard_normal((256, 256)) * 10).astype(np.float32).reshape(-1)
        dw = (rng.standard_normal((256, 256)) * 10).astype(np.float32).reshape(-1)
    else:
        dx = dw = None
    for bits in (8, 4):
        layer = at.nn.Conv2d_int8(C, O, _pair(k), _t(lut.reshape(-1), dev), grad=mode,
                                  dx=None if dx is None else _t(dx, dev), dw=None if dw is None else _t(dw, dev),
                                  bias=True, stride=_pair(s), padding=_pair(p), dilation=_pair(d),
                                  weight_bits=bits, update_scale=False).to(dev)
        x = (rng.standard_normal((B, C, H, W)) * 1.5).astype(np.float32)
        with torch.no_grad():
            layer.scale_x.fill_(0.02)              # clips part of the activations: masks matter
        xt = _t(x, dev).requires_grad_(True)
        y = layer(xt)
        go = rng.standard_normal(tuple(y.shape)).astype(np.float32)
        y.backward(_t(go, dev))
        ry, rgx, rgw, rgb = _fp64_layer_truth(
            x, layer.weight.detach().cpu().numpy(), layer.bias.detach().cpu().numpy(), lut,
            np.float32(0.02), layer.scale_w.cpu().numpy(), 2 ** (bits - 1) - 1, g4, go, mode, dx, dw)
        _close(y.flatten(2), ry)
        _close(xt.grad, rgx)
        _close(layer.weight.grad, rgw)
        _close(layer.bias.grad, rgb)
        # eval / no-grad forward is bit-identical
        with torch.no_grad():
            assert torch.equal(layer.eval()(_t(x, dev)), y.detach())


def test_reference_signature_functions_agree_with_fused_layer(dev):
    """conv2d_int8_{ste,lre} driven exactly as the reference layer drives them give the fused layer's numbers."""
    import approxtorch_b200 as at
    rng = np.random.default_rng(11)
    lut = lo.lut_signed_truncated(4)
    dx, dw = lo.lre_slopes(lut)
    for mode in ("ste", "lre"):
        layer = at.nn.Conv2d_int8(6, 8, 3, _t(lut.reshape(-1), dev), grad=mode, dx=_t(dx, dev), dw=_t(dw, dev),
                                  bias=True, padding=1, update_scale=False).to(dev)
        with torch.no_grad():
            layer.scale_x.fill_(0.03)
        x = _t(rng.standard_normal((2, 6, 7, 7)).astype(np.float32), dev)
        xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        ya = layer(xa)
        q = at.nn.quantization
        xq = q.static_quantize_int8(xb, layer.scale_x, -127, 127)
        wq = q.static_quantize_int8(layer.weight, layer.scale_w, -127, 127, ch_axis=0)
        geom = ((3, 3), (1, 1), (1, 1), (1, 1), 1)
        if mode == "ste":
            yb = at.nn.bgemm_int8.conv2d_int8_ste(xq, wq.view(8, -1), layer.lut, geom)
        else:
            yb = at.nn.bgemm_int8.conv2d_int8_lre(xq, wq.view(8, -1), layer.lut, layer.dx, layer.dw, geom)
        yb = torch.addcmul(layer.bias.view(1, -1, 1, 1), yb.view(2, 8, 7, 7), (layer.scale_x * layer.scale_w).view(1, -1, 1, 1))
        torch.testing.assert_close(ya, yb, rtol=1e-6, atol=1e-6)
        go = torch.randn_like(ya)
        ga = torch.autograd.grad(ya, [xa, layer.weight], go)
        gb = torch.autograd.grad(yb, [xb, layer.weight], go)
        for a, b in zip(ga, gb):
            _close(a, b.cpu().numpy().astype(np.float64))


def test_gemm_level_functions(dev):
    import approxtorch_b200 as at
    rng = np.random.default_rng(13)
    N, K, L, O = 2, 19, 23, 7
    x = rng.integers(-128, 128, (N, K, L)).astype(np.float32)
    w = rng.integers(-128, 128, (O, K)).astype(np.float32)
    go = rng.standard_normal((N, O, L)).astype(np.float32)
    lut = lo.lut_signed_noisy(100, seed=9)
    lt = _t(lut.reshape(-1), dev)
    xi, wi = lo.to_lut_index(x, 128), lo.to_lut_index(w, 128)
    dx, dw = lo.lre_slopes(lut)
    DX = (rng.standard_normal(65536) * 5).astype(np.float32)
    DW = (rng.standard_normal(65536) * 5).astype(np.float32)
    cases = {
        "ste": (lambda a, b: at.nn.bgemm_int8.bgemm_int8_ste(a, b, lt), lo.ste_backward(go, xi, wi)),
        "lre": (lambda a, b: at.nn.bgemm_int8.bgemm_int8_lre(a, b, lt, _t(dx, dev), _t(dw, dev)),
                lo.lre_backward(go, xi, wi, dx, dw)),
        "custom": (lambda a, b: at.nn.bgemm_int8.bgemm_int8_custom(a, b, lt, _t(DX, dev), _t(DW, dev)),
                   lo.custom_backward(go, xi, wi, DX, DW)),
    }
    for name, (fn, (rgx, rgw)) in cases.items():
        xt, wt = _t(x, dev).requires_grad_(True), _t(w, dev).requires_grad_(True)
        y = fn(xt, wt)
        np.testing.assert_array_equal(y.detach().cpu().numpy().astype(np.int64), lo.bgemm_exact(xi, wi, lut))
        y.backward(_t(go, dev))
        _close(xt.grad, rgx)
        _close(wt.grad, rgw)
    # raw operators: [K,O] weight layout of the LRE op, every operand dtype, zero-size shapes, int8 custom twins
    from approxtorch_b200.backend import ops
    rgx, rgw = lo.lre_backward(go, xi, wi, dx, dw)
    for xa, wa in ((x, w), (x.astype(np.int8), w.astype(np.int8)), (xi, wi)):
        gx, gw = ops.bgemm_lre_backward_claude(_t(go, dev), _t(xa, dev), _t(np.ascontiguousarray(wa.T), dev),
                                               _t(dx, dev), _t(dw, dev))
        assert tuple(gw.shape) == (K, O)
        _close(gx, rgx)
        _close(gw, rgw.T)
    gx, gw = ops.bgemm_lre_backward_claude(torch.zeros(0, O, L, device=dev), torch.zeros(0, K, L, device=dev),
                                           _t(np.ascontiguousarray(w.T), dev), _t(dx, dev), _t(dw, dev))
    assert gx.shape == (0, K, L) and not gw.any()
    cgx, cgw = lo.custom_backward(go, xi, wi, DX, DW)
    _close(ops.bgemm_custom_grad_int8_dx(_t(x.astype(np.int8), dev), _t(w.astype(np.int8), dev), _t(go, dev), _t(DX, dev)), cgx)
    _close(ops.bgemm_custom_grad_int8_dw(_t(x.astype(np.int8), dev), _t(w.astype(np.int8), dev), _t(go, dev), _t(DW, dev)), cgw)
    with pytest.raises(RuntimeError):
        ops.bgemm_custom_grad_int8_dx(_t(xi, dev), _t(wi, dev), _t(go, dev), _t(DX, dev))     # wrong dtype


def test_lre_backward_im2col_operator(dev):
    from approxtorch_b200.backend import ops
    rng = np.random.default_rng(17)
    B, C, H, W, O = 2, 5, 8, 7, 6
    x8 = rng.integers(-128, 128, (B, C, H, W)).astype(np.int8)
    w = rng.integers(-128, 128, (O, C * 9)).astype(np.int8)
    table_x = rng.standard_normal(256).astype(np.float32)
    table_w = rng.standard_normal(256).astype(np.float32)
    table_w[128] = 1e4                            # adversarial slope at the padding index
    cols = lo.im2col_index(lo.index_of(x8, True), 3, 3, 2, 1, 1, 1)
    go = rng.standard_normal((B, O, cols.shape[2])).astype(np.float32)
    rgx, rgw = lo.lre_backward(go, cols, lo.index_of(w, True), table_x, table_w)
    gx, gw = ops.bgemm_lre_backward_claude_im2col(_t(go, dev), _t(x8, dev), _t(np.ascontiguousarray(w.T), dev),
                                                  _t(table_x, dev), _t(table_w, dev), 3, (2, 1), 1, 1)
    _close(gx, rgx)
    _close(gw, rgw.T)


@pytest.mark.parametrize("geom", [(4, 70, 20, 20, 150, 3, 1, 1, 1), (3, 40, 17, 19, 130, 3, 2, 1, 1), (2, 200, 9, 9, 260, 1, 1, 0, 1),
                                  (2, 33, 14, 14, 40, (3, 2), (2, 1), (1, 2), (1, 2)), (3, 20, 12, 17, 24, (3, 2), 1, (1, 0), 1)])
def test_tensor_core_backward_against_fp64_and_the_simt_kernels(dev, geom):
    """Image-space STE / LRE backward on the tensor cores (three-term bf16 split, fp32 accumulation): several output
    tiles, a reduction split over the grid, stride classes, ragged edges - against the fp64 oracle at rel 1e-5 and
    against the fp32 SIMT kernels of the same entry point."""
    from approxtorch_b200.backend import ops, _C
    import ctypes
    B, C, H, W, O, k, s, p, d = geom
    g4 = (_pair(k), _pair(s), _pair(p), _pair(d))
    (kh, kw), (sh, sw), (ph, pw), (dh, dw_) = g4
    rng = np.random.default_rng(97)
    x8 = rng.integers(-127, 128, (B, C, H, W)).astype(np.int8)
    widx = rng.integers(0, 256, (O, C * kh * kw), dtype=np.uint8)
    cols = lo.im2col_index(lo.index_of(x8, True), kh, kw, sh, sw, ph, pw, dh, dw_, 128)
    go = rng.standard_normal((B, O, cols.shape[2])).astype(np.float32)
    gs = rng.uniform(0.5, 2.0, O).astype(np.float32)
    OH, OW = lo.conv_out_hw(H, W, kh, kw, sh, sw, ph, pw, dh, dw_)
    slopes_x = (rng.standard_normal(256) * 3).astype(np.float32)
    slopes_w = (rng.standard_normal(256) * 3).astype(np.float32)
    slopes_w[128] = 777.0                                     # the padded taps' value
    dec = np.arange(256, dtype=np.float32) - 128
    for name, tx, tw, exact in (("ste", dec, dec, True), ("lre", slopes_x, slopes_w, False)):
        g64 = go.astype(np.float64) * gs.astype(np.float64)[None, :, None]
        rgcols, rgw = lo.lre_backward(g64, cols, widx, tx, tw)
        rgx = lo.fold(rgcols, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw_)
        outs = {}
        for tc in ("packed", "in-kernel", False):                      # tensor cores (operands packed ahead / built in the kernel), SIMT
            ops.TENSOR_CORE_BACKWARD = bool(tc)
            ops.PACKED_BACKWARD = tc == "packed"
            try:
                gx, gw = ops.lre_conv_backward(_t(go, dev).view(B, O, OH, OW), _t(x8, dev), _t(widx, dev), _t(tx, dev), _t(tw, dev),
                                               g4, 128, go_scale=_t(gs, dev), exact_tables=exact)
            finally:
                ops.TENSOR_CORE_BACKWARD = True
                ops.PACKED_BACKWARD = True
            _close(gx, rgx)
            _close(gw, rgw)
            outs[tc] = (gx, gw)
        for tc in ("packed", "in-kernel"):
            _close(outs[tc][0], outs[False][0].double().cpu().numpy())
            _close(outs[tc][1], outs[False][1].double().cpu().numpy())
    status = ctypes.c_int(-1)
    torch.cuda.synchronize()
    assert _C.lib.atb_tensor_core_status(ctypes.byref(status)) == 0 and status.value == 0


def test_packed_backward_grad_w_in_fixed_order_is_reproducible(dev):
    """With the fixed-order option the slices of grad_w's pixel axis are stored and added by a second pass: two runs
    give the same bits, and the result stays within rel 1e-5 of the fp64 oracle."""
    from approxtorch_b200.backend import ops
    rng = np.random.default_rng(77)
    B, C, H, W, O = 6, 40, 24, 24, 72
    g4 = ((3, 3), (1, 1), (1, 1), (1, 1))
    x8 = rng.integers(-127, 128, (B, C, H, W), dtype=np.int8)
    widx = rng.integers(0, 256, (O, C * 9), dtype=np.uint8)
    cols = lo.im2col_index(lo.index_of(x8, True), 3, 3, 1, 1, 1, 1, 1, 1, 128)
    go = rng.standard_normal((B, O, cols.shape[2])).astype(np.float32)
    tab = (rng.standard_normal(256) * 3).astype(np.float32)
    _, rgw = lo.lre_backward(go.astype(np.float64), cols, widx, tab, tab)
    ops.DETERMINISTIC_GRAD_W = True
    try:
        runs = [ops.lre_conv_backward(_t(go, dev).view(B, O, H, W), _t(x8, dev), _t(widx, dev), _t(tab, dev), _t(tab, dev),
                                      g4, 128, need_x=False)[1] for _ in range(3)]
    finally:
        ops.DETERMINISTIC_GRAD_W = False
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])
    _close(runs[0], rgw)


def _uint8_layer_truth(x, w, bias, lut, sx, zx, sw, zw, geom):
    (kh, kw), (sh, sw_), (ph, pw), (dh, dw_) = geom
    O = w.shape[0]
    xq, _ = lo.fakequant_asym(x, sx, zx, 0, 255)
    wq, _ = lo.fakequant_asym(w, sw.reshape(-1, 1, 1, 1), zw.reshape(-1, 1, 1, 1), 0, 255)
    cols = lo.im2col_index(xq.astype(np.uint8), kh, kw, sh, sw_, ph, pw, dh, dw_, int(zx))
    widx = wq.reshape(O, -1).astype(np.uint8)
    t = lo.uint8_zero_point_correction(lo.bgemm_exact(cols, widx, lut), cols, widx, zx, zw)
    s = (np.float32(sx) * sw).astype(np.float64)
    return t * s[None, :, None] + (0 if bias is None else bias.astype(np.float64)[None, :, None])


@pytest.mark.parametrize("geom", [(2, 6, 9, 9, 10, 3, 1, 1, 1), (2, 4, 10, 8, 7, 3, 2, 1, 1), (3, 8, 6, 6, 70, 1, 2, 0, 1)])
def test_uint8_layer_inference_and_training_routes(dev, geom):
    import approxtorch_b200 as at
    B, C, H, W, O, k, s, p, d = geom
    g4 = (_pair(k), _pair(s), _pair(p), _pair(d))
    rng = np.random.default_rng(19)
    torch.manual_seed(5)
    lut = lo.lut_unsigned_truncated(6)
    layer = at.nn.Conv2d_uint8(C, O, _pair(k), _t(lut.reshape(-1), dev), bias=True, stride=_pair(s),
                               padding=_pair(p), update_scale=False).to(dev)
    x = (rng.standard_normal((B, C, H, W)) * 1.2).astype(np.float32)
    with torch.no_grad():
        layer.x_min.fill_(-2.0)
        layer.x_max.fill_(2.5)
    layer._reset_qparams_from_stats()
    assert torch.equal(layer.zero_x, torch.round(layer.zero_x)) and torch.equal(layer.zero_w, torch.round(layer.zero_w))
    ref = _uint8_layer_truth(x, layer.weight.detach().cpu().numpy(), layer.bias.detach().cpu().numpy(), lut,
                             layer.scale_x.item(), layer.zero_x.item(), layer.scale_w.cpu().numpy(),
                             layer.zero_w.cpu().numpy(), g4)
    with torch.no_grad():
        y_inf = layer.eval()(_t(x, dev))
    _close(y_inf.flatten(2), ref)
    xt = _t(x, dev).requires_grad_(True)
    y_tr = layer.train()(xt)                       # update_scale is off: statistics stay frozen
    _close(y_tr.flatten(2), ref)
    # STE gradient == autograd through the exact centred convolution surrogate
    go = torch.randn_like(y_tr)
    y_tr.backward(go)
    q = at.nn.quantization
    xs = _t(x, dev).requires_grad_(True)
    ws = layer.weight.detach().clone().requires_grad_(True)
    xq = q.static_quantize_uint8(xs, layer.scale_x, layer.zero_x, 0, 255) - layer.zero_x
    wq = q.static_quantize_uint8(ws, layer.scale_w, layer.zero_w, 0, 255, ch_axis=0) - layer.zero_w.view(-1, 1, 1, 1)
    prev = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        ysur = torch.nn.functional.conv2d(xq.double(), wq.double(), None, _pair(s), _pair(p)) \
            * (layer.scale_x * layer.scale_w).double().view(1, -1, 1, 1)
        gxs, gws = torch.autograd.grad(ysur, [xs, ws], go.double())
    finally:
        torch.backends.cudnn.allow_tf32 = prev
    _close(xt.grad, gxs.cpu().numpy().astype(np.float64))
    _close(layer.weight.grad, gws.cpu().numpy().astype(np.float64))


@pytest.mark.parametrize("mode", ["ste", "lre"])
@pytest.mark.parametrize("geom", [(2, 6, 9, 9, 10, 3, 1, 1, 1), (2, 4, 10, 8, 7, 3, 2, 1, 1), (3, 8, 6, 6, 70, 1, 2, 0, 1),
                                  (2, 5, 7, 9, 6, (3, 2), (1, 2), (2, 1), 1)])
def test_uint8_fused_training_matches_decoupled_chain(dev, mode, geom):
    """The fused image-space training route against the reference's decoupled chain (fake-quant -> pad with z_x ->
    unfold -> LUT-BGEMM Function -> differentiable correction) on the same layer: outputs and all three
    gradients, including the padded taps' contribution to grad_w under LRE slopes."""
    import approxtorch_b200 as at
    B, C, H, W, O, k, s, p, d = geom
    rng = np.random.default_rng(23)
    torch.manual_seed(7)
    lut = lo.lut_unsigned_truncated(6)
    dx = _t(rng.uniform(20, 200, 256).astype(np.float32), dev) if mode == "lre" else None
    dw = _t(rng.uniform(20, 200, 256).astype(np.float32), dev) if mode == "lre" else None
    layer = at.nn.Conv2d_uint8(C, O, _pair(k), _t(lut.reshape(-1), dev), grad=mode, dx=dx, dw=dw, bias=True,
                               stride=_pair(s), padding=_pair(p), update_scale=False).to(dev).train()
    with torch.no_grad():
        layer.x_min.fill_(-1.5)            # narrower than the data: some activations clip, so masks matter
        layer.x_max.fill_(2.0)
    layer._reset_qparams_from_stats()
    x = (rng.standard_normal((B, C, H, W)) * 1.2).astype(np.float32)
    outs = {}
    for fused in (True, False):
        layer.fused_training = fused
        layer.zero_grad(set_to_none=True)
        xt = _t(x, dev).requires_grad_(True)
        y = layer(xt)
        torch.manual_seed(11)
        go = torch.randn_like(y)
        y.backward(go)
        outs[fused] = (y.detach(), xt.grad.clone(), layer.weight.grad.clone(), layer.bias.grad.clone())
    for got, ref in zip(outs[True], outs[False]):
        _close(got, ref.double().cpu().numpy())


def test_ema_statistics_on_device(dev):
    import approxtorch_b200 as at
    rng = np.random.default_rng(23)
    lut = _t(lo.lut_exact_signed().reshape(-1), dev)
    layer = at.nn.Conv2d_int8(3, 4, 3, lut, padding=1, scale_momentum=0.1).to(dev).train()
    sx, sw = np.float32(1.0), layer.scale_w.cpu().numpy().copy()
    for step in range(3):
        x = (rng.standard_normal((2, 3, 6, 6)) * (step + 1)).astype(np.float32)
        layer(_t(x, dev))
        sx = lo.ema_scale_x(np.abs(x).max(), sx, 0.1)
        sw = lo.ema(lo.weight_absmax_scale(layer.weight.detach().cpu().numpy(), 8, old=sw), sw, 0.1)
        assert layer.scale_x.item() == sx
        np.testing.assert_array_equal(layer.scale_w.cpu().numpy(), sw)
    layer.freeze_scale()
    before = layer.scale_x.clone()
    layer(_t(x * 10, dev))
    assert torch.equal(before, layer.scale_x)
    layer.unfreeze_scale()
    layer.eval()(_t(x * 10, dev))                  # eval never updates
    assert torch.equal(before, layer.scale_x)


def test_depthwise_layer(dev):
    import approxtorch_b200 as at
    from approxtorch_b200.backend import ops
    rng = np.random.default_rng(29)
    B, C, H, W = 2, 6, 9, 8
    lut = lo.lut_signed_noisy(64, seed=6)
    x8 = rng.integers(-127, 128, (B, C, H, W)).astype(np.int8)
    w = rng.integers(-127, 128, (C, 9)).astype(np.float32)
    y, wq = ops.dwconv_fake_int8_claude(_t(x8, dev), _t(w, dev), _t(lut.reshape(-1), dev), 3, 2, 1, 1)
    cols = lo.im2col_index(lo.index_of(x8, True), 3, 3, 2, 2, 1, 1)            # [B, C*9, L]
    L = cols.shape[2]
    ref = np.stack([lo.bgemm_exact(cols[:, c * 9:(c + 1) * 9], lo.to_lut_index(w[c:c + 1], 128), lut)[:, 0]
                    for c in range(C)], axis=1)
    np.testing.assert_array_equal(y.flatten(2).cpu().numpy().astype(np.int64), ref)
    # the layer: forward and STE / LRE gradients against the per-channel fp64 chain (stride 2, and a 5x5 window with
    # dilation), including the padded taps' slope dw[128] and clipped activations
    for mode in ("ste", "lre"):
        for (k, s, p, d) in ((3, 2, 1, 1), (3, 1, 1, 1), (5, 1, 4, 2)):
            dx, dw = lo.lre_slopes(lut)
            dw = dw.copy(); dw[128] = 2.5
            torch.manual_seed(5)
            layer = at.nn.Conv2d_int8(C, C, k, _t(lut.reshape(-1), dev), grad=mode, dx=_t(dx, dev), dw=_t(dw, dev), bias=True,
                                      stride=s, padding=p, dilation=d, groups=C, update_scale=False).to(dev)
            with torch.no_grad():
                layer.scale_x.fill_(0.02)
            xin = (rng.standard_normal((B, C, H, W)) * 1.5).astype(np.float32)
            xt = _t(xin, dev).requires_grad_(True)
            out = layer(xt)
            go = rng.standard_normal(tuple(out.shape)).astype(np.float32)
            out.backward(_t(go, dev))
            sw = layer.scale_w.cpu().numpy()
            wnp = layer.weight.detach().cpu().numpy()                       # [C, 1, k, k]
            xq, xm = lo.fakequant_sym(xin, np.float32(0.02), -127, 127)
            wq, wm = lo.fakequant_sym(wnp, sw.reshape(-1, 1, 1, 1), -127, 127)
            sc = (np.float32(0.02) * sw).astype(np.float64)
            OH, OW = out.shape[2], out.shape[3]
            ry = np.zeros((B, C, OH * OW)); rgx = np.zeros((B, C, H, W)); rgw = np.zeros((C, k * k))
            for c in range(C):
                colsc = lo.im2col_index(lo.to_lut_index(xq[:, c:c + 1], 128), k, k, s, s, p, p, d, d, 128)
                wc = lo.to_lut_index(wq[c].reshape(1, -1), 128)
                ry[:, c] = lo.bgemm_exact(colsc, wc, lut)[:, 0] * sc[c] + layer.bias.detach().cpu().numpy()[c]
                gch = go.reshape(B, C, -1)[:, c:c + 1].astype(np.float64) * sc[c]
                if mode == "ste":
                    gcols, gwc = lo.ste_backward(gch, colsc, wc)
                else:
                    gcols, gwc = lo.lre_backward(gch, colsc, wc, dx, dw)
                rgx[:, c] = lo.fold(gcols, 1, H, W, k, k, s, s, p, p, d, d)[:, 0]
                rgw[c] = gwc[0]
            rgx = rgx * xm / 0.02
            rgw = rgw.reshape(wnp.shape) * wm / np.maximum(sw.astype(np.float64), 1e-12).reshape(-1, 1, 1, 1)
            _close(out.flatten(2), ry)
            _close(xt.grad, rgx)
            _close(layer.weight.grad, rgw)
            _close(layer.bias.grad, go.astype(np.float64).sum(axis=(0, 2, 3)))


@pytest.mark.parametrize("in_f", [70, 64])        # byte-wise rows; rows read 16 bytes at a time (in_f % 16 == 0)
def test_linear_layer_on_the_lut_gemm(dev, in_f):
    """Fully connected layer: forward equals the exact integer product of the quantised operands under an exact
    table (bit for bit before the fp32 scale), STE gradients equal autograd through the exact surrogate."""
    import approxtorch_b200 as at
    rng = np.random.default_rng(31)
    torch.manual_seed(3)
    lut = lo.lut_exact_signed()
    layer = at.nn.Linear_int8(in_f, 33, _t(lut.reshape(-1), dev), bias=True, update_scale=False).to(dev)
    x = (rng.standard_normal((4, 6, in_f)) * 1.5).astype(np.float32)          # leading dims are flattened
    with torch.no_grad():
        layer.conv.scale_x.fill_(float(np.abs(x).max() / 127))
    xt = _t(x, dev).requires_grad_(True)
    y = layer.train()(xt)
    assert tuple(y.shape) == (4, 6, 33)
    q = at.nn.quantization
    xs = _t(x, dev).requires_grad_(True)
    ws = layer.weight.detach().clone().requires_grad_(True)
    xq = q.static_quantize_int8(xs, layer.conv.scale_x, -127, 127)
    wq = q.static_quantize_int8(ws, layer.conv.scale_w, -127, 127, ch_axis=0)
    ysur = (xq.double().reshape(-1, in_f) @ wq.double().t()) * (layer.conv.scale_x * layer.conv.scale_w).double() \
        + layer.bias.double()
    _close(y.reshape(-1, 33), ysur.detach().cpu().numpy())
    go = torch.randn_like(y)
    y.backward(go)
    gxs, gws = torch.autograd.grad(ysur, [xs, ws], go.double().reshape(-1, 33))
    _close(xt.grad, gxs.cpu().numpy().astype(np.float64))
    _close(layer.conv.weight.grad.view(33, in_f), gws.cpu().numpy().astype(np.float64))
    with torch.no_grad():
        assert torch.equal(layer.eval()(_t(x, dev)), y.detach())
