"""GPU parity of the fake-quantisation / statistics / map kernels: bit-exact against the reference
fixtures and the oracle."""

import numpy as np
import pytest
import torch

from oracle import lut_oracle as lo

pytestmark = pytest.mark.gpu


def _t(a, dev):
    a = np.asarray(a)
    return torch.from_numpy(np.ascontiguousarray(a).reshape(a.shape)).to(dev)


def test_per_tensor_fakequant_matches_reference_fixture(golden, dev):
    import approxtorch_b200 as at
    q = at.nn.quantization
    g = golden("fakequant")
    for tag in "abcd":
        x = _t(g[f"sym_{tag}_x"], dev).requires_grad_(True)
        qmin, qmax = (int(v) for v in g[f"sym_{tag}_qrange"])
        out = q.static_quantize_int8(x, _t(g[f"sym_{tag}_scale"], dev), qmin, qmax)
        np.testing.assert_array_equal(out.detach().cpu().numpy(), g[f"sym_{tag}_q"])
        out.backward(_t(g[f"sym_{tag}_go"], dev))
        np.testing.assert_array_equal(x.grad.cpu().numpy(), g[f"sym_{tag}_gx"])
    for tag in "ab":
        x = _t(g[f"asym_{tag}_x"], dev).requires_grad_(True)
        qmin, qmax = (int(v) for v in g[f"asym_{tag}_qrange"])
        out = q.static_quantize_uint8(x, _t(g[f"asym_{tag}_scale"], dev), _t(g[f"asym_{tag}_zero"], dev), qmin, qmax)
        np.testing.assert_array_equal(out.detach().cpu().numpy(), g[f"asym_{tag}_q"])
        out.backward(_t(g[f"asym_{tag}_go"], dev))
        np.testing.assert_array_equal(x.grad.cpu().numpy(), g[f"asym_{tag}_gx"])


def test_per_channel_fakequant_matches_reference_fixture(golden, dev):
    import approxtorch_b200 as at
    q = at.nn.quantization
    g = golden("fakequant")
    for bits in range(3, 9):
        qm = 2 ** (bits - 1) - 1
        w = _t(g["pc_w"], dev).requires_grad_(True)
        out = q.static_quantize_int8(w, _t(g[f"pc_{bits}_scale"], dev), -qm, qm, ch_axis=0)
        np.testing.assert_array_equal(out.detach().cpu().numpy(), g[f"pc_{bits}_q"])
        out.backward(_t(g[f"pc_{bits}_go"], dev))
        np.testing.assert_array_equal(w.grad.cpu().numpy(), g[f"pc_{bits}_gx"])
    out = q.static_quantize_uint8(_t(g["pc_w"], dev), _t(g["pca_scale"], dev), _t(g["pca_zero"], dev), 0, 255, ch_axis=0)
    np.testing.assert_array_equal(out.cpu().numpy(), g["pca_q"])
    # channel axis other than 0
    w = g["pc_w"]
    sc = np.abs(w).max(axis=(0, 2, 3)) / 127
    out = q.static_quantize_int8(_t(w, dev), _t(sc.astype(np.float32), dev), -127, 127, ch_axis=1)
    ref, _ = lo.fakequant_sym(w, sc.astype(np.float32).reshape(1, -1, 1, 1), -127, 127)
    np.testing.assert_array_equal(out.cpu().numpy(), ref)


def test_fused_image_and_weight_quantisation(dev):
    from approxtorch_b200.backend import ops
    rng = np.random.default_rng(1)
    for n in (1, 3, 4097, 8 * 64 * 32 * 32):
        x = (rng.standard_normal(n) * 2).astype(np.float32)
        s = np.float32(np.abs(x).max() / 127)
        q8, mask = ops.quantize_image(_t(x, dev), _t(np.array(s), dev), None, -127, 127)
        rq, rm = lo.fakequant_sym(x, s, -127, 127)
        assert q8.dtype == torch.int8
        np.testing.assert_array_equal(q8.cpu().numpy(), rq.astype(np.int8))
        np.testing.assert_array_equal(mask.cpu().numpy(), rm)
        zs, zz = np.float32(0.037), np.float32(91.0)
        u8, mask = ops.quantize_image(_t(x, dev), _t(np.array(zs), dev), _t(np.array(zz), dev), 0, 255)
        rq, rm = lo.fakequant_asym(x, zs, zz, 0, 255)
        assert u8.dtype == torch.uint8
        np.testing.assert_array_equal(u8.cpu().numpy(), rq.astype(np.uint8))
        np.testing.assert_array_equal(mask.cpu().numpy(), rm)
    w = (rng.standard_normal((37, 5, 3, 3)) * 0.1).astype(np.float32)
    w[4] = 0
    for bits in (8, 4, 3):
        qm = 2 ** (bits - 1) - 1
        sc = lo.weight_absmax_scale(w, bits)
        widx, mask, q, wsum = ops.quantize_weight(_t(w, dev), _t(sc, dev), None, -qm, qm, 128,
                                                  want_mask=True, want_q=True, want_sum=True)
        rq, rm = lo.fakequant_sym(w, sc.reshape(-1, 1, 1, 1), -qm, qm)
        np.testing.assert_array_equal(q.cpu().numpy(), rq)
        np.testing.assert_array_equal(mask.cpu().numpy(), rm)
        np.testing.assert_array_equal(widx.cpu().numpy(), (rq.reshape(37, -1) + 128).astype(np.uint8))
        np.testing.assert_array_equal(wsum.cpu().numpy(), (rq.reshape(37, -1) + 128).sum(axis=1).astype(np.int32))


def test_statistics_kernel(dev):
    from approxtorch_b200.backend import ops
    rng = np.random.default_rng(2)
    for n in (1, 5, 1000, 1 << 20, (1 << 20) + 3):
        x = (rng.standard_normal(n) * 3 - 0.2).astype(np.float32)
        st = ops.absmax(_t(x, dev), want_minmax=True).cpu().numpy()
        assert st[0] == np.abs(x).max() and st[1] == x.min() and st[2] == x.max()
        st = ops.absmax(_t(np.abs(x) + 1, dev), want_minmax=True).cpu().numpy()       # all positive
        assert st[1] == (np.abs(x) + 1).min()
        st = ops.absmax(_t(-np.abs(x) - 1, dev), want_minmax=True).cpu().numpy()      # all negative
        assert st[2] == (-np.abs(x) - 1).max() and st[0] == (np.abs(x) + 1).max()
    big = torch.zeros(1001, device=dev)[1:]                                             # misaligned
    big[17] = -7.5
    assert ops.absmax(big)[0].item() == 7.5
    assert ops.absmax(torch.zeros(0, device=dev))[0].item() == 0.0


def test_im2col_and_table_maps(dev):
    from approxtorch_b200.backend import ops
    rng = np.random.default_rng(3)
    x8 = rng.integers(-128, 128, (2, 5, 9, 11)).astype(np.int8)
    for (k, s, p, d) in ((3, 1, 1, 1), (3, 2, 0, 1), (1, 1, 0, 1), (1, 2, 0, 1), ((3, 2), (2, 1), (1, 2), (1, 2)), (5, 1, 2, 1)):
        kh, kw = (k, k) if isinstance(k, int) else k
        sh, sw = (s, s) if isinstance(s, int) else s
        ph, pw = (p, p) if isinstance(p, int) else p
        dh, dw = (d, d) if isinstance(d, int) else d
        ref = lo.im2col_index(lo.index_of(x8, True), kh, kw, sh, sw, ph, pw, dh, dw, 128)
        for src in (x8, lo.index_of(x8, True), x8.astype(np.float32)):
            got = ops.im2col_u8(_t(src, dev), (kh, kw), (sh, sw), (ph, pw), (dh, dw))
            if src.dtype == np.uint8:
                # uint8 input = already indices; padding still maps to 128
                np.testing.assert_array_equal(got.cpu().numpy(), ref)
            else:
                np.testing.assert_array_equal(got.cpu().numpy(), ref)
        # == unfold + 128, the identity the reference's tests pin
        unf = torch.nn.functional.unfold(torch.from_numpy(x8.astype(np.float32)), (kh, kw), dilation=(dh, dw),
                                         padding=(ph, pw), stride=(sh, sw)) + 128
        np.testing.assert_array_equal(ref, unf.numpy().astype(np.uint8))
    table = rng.standard_normal(256).astype(np.float32)
    for src in (x8, lo.index_of(x8, True), (x8.astype(np.float32) * 1.0)):
        got = ops.lut_map(_t(src, dev), _t(table, dev))
        np.testing.assert_array_equal(got.cpu().numpy(), lo.lut_map(src, table))
        got = ops.lut_map_pad(_t(src, dev), _t(table, dev), (2, 1))
        np.testing.assert_array_equal(got.cpu().numpy(), lo.lut_map_pad(src, table, 2, 1))
