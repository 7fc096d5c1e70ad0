"""GPU parity at the shapes the benchmark configurations state (not scaled-down stand-ins), and in the
large-reduction regime that ResNet-50's last stage reaches:

* the single-layer configuration exactly: x [8,64,32,32], kaiming-normal w [64,64,3,3], stride 1 pad 1,
  truncated-product table, scale_x = max|x|/127 — integer accumulator bit-exact, STE gradients rel 1e-5;
* K = 4608 / O = 512 / L = 49 unsigned conv with zero points (sums above 2^24) against the int64 oracle, through the
  whole-tile and cut-tile plans, with the reference CUDA operator's own deviation printed beside ours;
* K = 65536 with every table entry 65535 and every operand 255 (the bound of the modulo-2^32 accumulators);
* three layers of the converted ResNet-50 against the oracle on the activations they actually received;
* the unsigned layer with the custom (pair-wise) estimator against fp64;
* the calibration tool on CUDA tensors.
"""

import ctypes

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
    got = got.detach().cpu().numpy().astype(np.float64) if isinstance(got, torch.Tensor) else np.asarray(got, np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    scale = max(np.abs(ref).max(), 1e-30)
    err = np.abs(got - ref).max()
    assert err <= rtol * scale, (err, scale)
    return err / scale


# ------------------------------------------------------------------------------------------- configuration 0
def test_single_layer_configuration_at_its_stated_shape(dev):
    import approxtorch_b200 as at
    torch.manual_seed(0)
    x = torch.randn(8, 64, 32, 32)
    w = torch.nn.init.kaiming_normal_(torch.empty(64, 64, 3, 3))
    lutn = lo.lut_signed_truncated(4)
    lut = _t(lutn.reshape(-1), dev)
    layer = at.nn.Conv2d_int8(64, 64, 3, lut, grad="ste", bias=False, stride=1, padding=1, update_scale=False)
    with torch.no_grad():
        layer.weight.copy_(w)
        layer.scale_x.fill_(float(x.abs().max()) / 127)
    layer._reset_scale_w_from_weight()
    layer = layer.to(dev)
    sx = np.float32(layer.scale_x.item())
    sw = layer.scale_w.cpu().numpy()

    # integer accumulator, before dequantisation: the conv-level Function on the fake-quantised operands
    q = at.nn.quantization
    xq = q.static_quantize_int8(x.to(dev), layer.scale_x, -127, 127)
    wq = q.static_quantize_int8(layer.weight, layer.scale_w, -127, 127, ch_axis=0)
    yint = at.nn.bgemm_int8.conv2d_int8_ste(xq, wq.view(64, -1), lut, ((3, 3), (1, 1), (1, 1), (1, 1), 1))
    xq_o, xm = lo.fakequant_sym(x.numpy(), sx, -127, 127)
    wq_o, wm = lo.fakequant_sym(w.numpy(), sw.reshape(-1, 1, 1, 1), -127, 127)
    np.testing.assert_array_equal(xq.cpu().numpy(), xq_o)                      # quantised tensors bit-exact
    np.testing.assert_array_equal(wq.detach().cpu().numpy(), wq_o)
    cols = lo.im2col_index(lo.to_lut_index(xq_o, 128), 3, 3, 1, 1, 1, 1)
    widx = lo.to_lut_index(wq_o.reshape(64, -1), 128)
    ref_int = lo.bgemm_exact(cols, widx, lutn)                                 # [8, 64, 1024] int64
    assert np.abs(ref_int).max() < 2 ** 24                                     # the bit-exact bar applies
    np.testing.assert_array_equal(yint.detach().cpu().numpy().astype(np.int64), ref_int)

    # the layer itself: dequantised output and STE gradients against the fp64 chain
    xt = x.to(dev).requires_grad_(True)
    y = layer(xt)
    torch.manual_seed(1)
    go = torch.randn(8, 64, 32, 32)
    y.backward(go.to(dev))
    s = (sx * sw).astype(np.float64)
    _close(y.flatten(2), ref_int.astype(np.float64) * s[None, :, None])
    g = go.numpy().reshape(8, 64, -1).astype(np.float64) * s[None, :, None]
    gcols, gw = lo.ste_backward(g, cols, widx)
    gx = lo.fold(gcols, 64, 32, 32, 3, 3, 1, 1, 1, 1) * xm / max(np.float64(sx), 1e-12)
    gw = gw.reshape(64, 64, 3, 3) * wm / np.maximum(sw.astype(np.float64), 1e-12).reshape(-1, 1, 1, 1)
    _close(xt.grad, gx)
    _close(layer.weight.grad, gw)


# ------------------------------------------------------------------------------------------- large reductions
def _plan(_C, R, K, O, cfg):
    plan = _C.GemmPlan()
    assert _C.lib.atb_lut_gemm_plan(R, K, O, 0, cfg, ctypes.byref(plan)) == 0
    return plan


def test_resnet50_last_stage_shape_against_int64_oracle(dev, capsys):
    """K = 512*3*3 = 4608, O = 512, L = 7*7: table entries up to 65024, sums up to 3e8 (beyond fp32's exact
    integers), zero points on both operands.  Every plan must give the correctly rounded exact result."""
    from approxtorch_b200.backend import ops, _C
    rng = np.random.default_rng(4608)
    B, C, H, W, O = 4, 512, 7, 7, 512
    lut = lo.lut_unsigned_truncated(6)
    img = ops.lut_image(_t(lut.reshape(-1), dev))
    # operands skewed high so that the sums really are large
    x8 = rng.integers(96, 256, (B, C, H, W), dtype=np.uint8)
    widx = rng.integers(64, 256, (O, C * 9), dtype=np.uint8)
    zx, zw = 117.0, rng.integers(90, 160, O).astype(np.float32)
    cols = lo.im2col_index(x8, 3, 3, 1, 1, 1, 1, 1, 1, int(zx))
    lutsum = lo.bgemm_exact(cols, widx, lut)
    assert lutsum.max() > 2 ** 26
    exact = lo.uint8_zero_point_correction(lutsum, cols, widx, zx, zw)         # float64, integer-valued, exact
    want = exact.astype(np.float32)                                            # one rounding
    g4 = ((3, 3), (1, 1), (1, 1), (1, 1))
    wsum = _t(widx.astype(np.int64).sum(axis=1).astype(np.int32), dev)
    zx_t, zw_t = torch.tensor(zx, device=dev), _t(zw, dev)
    R, K = B * H * W, C * 9
    plans = {"automatic": -1, "whole tiles": (1 << 16) | 256, "every tile in six segments": (6 << 16) | 128,
             "every tile in nineteen segments, short tiles": (19 << 16) | 96}
    seen = set()
    for name, cfg in plans.items():
        p = _plan(_C, R, K, O, cfg)
        seen.add("cut" if p.cut_tiles else "whole")
        y = ops.lut_conv2d_launch(_t(x8, dev), _t(widx, dev), img, g4, -1, zero_x=zx_t, zero_w=zw_t, wsum=wsum, cfg=cfg)
        np.testing.assert_array_equal(y.flatten(2).cpu().numpy(), want, err_msg=name)
    assert seen == {"cut", "whole"}
    ours = np.abs(want.astype(np.float64) - exact).max() / np.abs(exact).max()

    # Raw sums of an exact unsigned product table (odd entries, so fp32 running sums above 2^24 must round): the
    # reference's own CUDA operator and this package, each against the int64 oracle
    from test_gpu_reference_kernels import _have_ref, run_ref
    plut = lo.lut_exact_unsigned()
    psum = lo.bgemm_exact(cols, widx, plut)
    wf = widx.astype(np.float32)
    mine = ops.bgemm_fake_uint8_claude(_t(cols, dev), _t(wf, dev), _t(plut.reshape(-1), dev))
    my_dev = np.abs(mine.cpu().numpy().astype(np.float64) - psum).max() / psum.max()
    assert my_dev <= 2.0 ** -24                                                # one rounding of the exact sum
    np.testing.assert_array_equal(mine.cpu().numpy(), psum.astype(np.float32))
    msg = f"this package {my_dev:.3e} (raw sums), {ours:.3e} (zero-point corrected output)"
    if _have_ref():
        (ry,) = run_ref("bgemm_fake_uint8_forward_cuda_claude", cols, wf, plut.reshape(-1))
        ref_dev = np.abs(ry.astype(np.float64) - psum).max() / psum.max()
        msg = f"reference CUDA operator {ref_dev:.3e}, " + msg
        assert ref_dev <= 1e-4
    with capsys.disabled():
        print(f"\n[K=4608, sums up to {psum.max():.3g}] max deviation from the int64 oracle, relative to the largest sum: {msg}")


def test_accumulator_bound_and_reductions_longer_than_it(dev):
    """K = 65536 with all-65535 entries and all-255 operands is the largest sum the modulo-2^32 accumulators keep
    exact (65536 * 65535 < 2^32), whole tiles or cut; anything longer is refused."""
    from approxtorch_b200.backend import ops, _C
    lut = np.full((256, 256), 65535.0, dtype=np.float32)
    img = ops.lut_image(_t(lut.reshape(-1), dev))
    rng = np.random.default_rng(5)
    for K, cfgs in ((32768, (-1, (1 << 16) | 64, (5 << 16) | 64)), (40000, (-1, (1 << 16) | 64)),
                    (65536, (-1, (1 << 16) | 160, (3 << 16) | 64))):
        R, O = 150, 70
        x = np.full((1, K, R), 255, dtype=np.uint8)
        w = np.full((O, K), 255, dtype=np.uint8)
        for cfg in cfgs:
            y = torch.empty((1, O, R), dtype=torch.float32, device=dev)
            ops.lut_gemm_launch(_t(x, dev), _t(w, dev), img, y, 1, K, R, O, cfg=cfg)
            assert torch.all(y == float(np.float32(65535 * K))), (K, cfg)
    with pytest.raises(RuntimeError):
        ops.lut_gemm_launch(torch.zeros(1, 65537, 8, dtype=torch.uint8, device=dev), torch.zeros(4, 65537, dtype=torch.uint8, device=dev),
                            img, torch.empty(1, 4, 8, device=dev), 1, 65537, 8, 4)
    # a signed table at the bound, random operands, L == 1 layout, against the int64 oracle
    slut = np.where(rng.random((256, 256)) < 0.5, -32767.0, 32767.0).astype(np.float32)
    simg = ops.lut_image(_t(slut.reshape(-1), dev))
    K, R, O = 36000, 70, 33
    x = rng.integers(0, 256, (R, K, 1), dtype=np.uint8)
    w = rng.integers(0, 256, (O, K), dtype=np.uint8)
    y = torch.empty((R, O, 1), dtype=torch.float32, device=dev)
    ops.lut_gemm_launch(_t(x, dev), _t(w, dev), simg, y, R, K, 1, O)
    ref = lo.bgemm_exact(x, w, slut)
    np.testing.assert_array_equal(y.cpu().numpy(), ref.astype(np.float32))


# ------------------------------------------------------------------------------------------- ResNet-50 layers
def test_resnet50_layers_against_the_oracle_on_their_real_inputs(dev):
    import torchvision
    import approxtorch_b200 as at
    from test_gpu_conv import _uint8_layer_truth
    torch.manual_seed(0)
    lutn = lo.lut_unsigned_truncated(6)
    model = torchvision.models.resnet50()
    at.convert_model(model, _t(lutn.reshape(-1), dev), qtype="uint8", scale_momentum=1.0)
    model = model.to(dev).train()
    x = torch.randn(4, 3, 64, 64, device=dev)
    with torch.no_grad():
        model(x)                                                   # calibration pass (momentum 1)
    model.eval()
    picked = {"first 3x3": model.layer1[0].conv2, "stride-2 1x1 downsample": model.layer2[0].downsample[0],
              "last 3x3 (K = 4608)": model.layer4[2].conv2}
    assert picked["last 3x3 (K = 4608)"].in_channels * 9 == 4608
    feats, hooks = {}, []
    for name, layer in picked.items():
        hooks.append(layer.register_forward_hook(
            lambda m, i, o, name=name: feats.__setitem__(name, (i[0].detach().cpu().numpy(), o.detach().cpu().numpy()))))
    with torch.no_grad():
        model(x)
    for h in hooks:
        h.remove()
    for name, layer in picked.items():
        xin, yout = feats[name]
        g4 = (tuple(layer.kernel_size), tuple(layer.stride), tuple(layer.padding), tuple(layer.dilation))
        ref = _uint8_layer_truth(xin, layer.weight.detach().cpu().numpy(), None, lutn, layer.scale_x.item(),
                                 layer.zero_x.item(), layer.scale_w.cpu().numpy(), layer.zero_w.cpu().numpy(), g4)
        _close(yout.reshape(ref.shape), ref)


# ------------------------------------------------------------------------------------------- uint8 custom estimator
@pytest.mark.parametrize("geom", [(2, 5, 8, 8, 6, 3, 1, 1), (2, 4, 9, 7, 7, 3, 2, 1), (2, 6, 5, 5, 9, 1, 1, 0)])
def test_uint8_layer_custom_gradients_against_fp64(dev, geom):
    """Conv2d_uint8(grad='custom'): d out / d q_x = sum_o g s (DX[q_x][q_w] - z_w), d out / d q_w = sum g s (DW[q_x][q_w] - z_x)
    (the -z terms come from the differentiable zero-point correction), padded taps carry q_x = z_x and pass no
    gradient to the image."""
    import approxtorch_b200 as at
    B, C, H, W, O, k, s, p = geom
    rng = np.random.default_rng(41)
    torch.manual_seed(9)
    lut = lo.lut_unsigned_truncated(6)
    DX = (rng.standard_normal(65536) * 30).astype(np.float32)
    DW = (rng.standard_normal(65536) * 30).astype(np.float32)
    layer = at.nn.Conv2d_uint8(C, O, k, _t(lut.reshape(-1), dev), grad="custom", dx=_t(DX, dev), dw=_t(DW, dev),
                               bias=True, stride=s, padding=p, update_scale=False).to(dev).train()
    with torch.no_grad():
        layer.x_min.fill_(-1.5)
        layer.x_max.fill_(2.0)
    layer._reset_qparams_from_stats()
    x = (rng.standard_normal((B, C, H, W)) * 1.2).astype(np.float32)
    xt = _t(x, dev).requires_grad_(True)
    y = layer(xt)
    go = rng.standard_normal(tuple(y.shape)).astype(np.float32)
    y.backward(_t(go, dev))

    sx, zx = layer.scale_x.item(), layer.zero_x.item()
    sw, zw = layer.scale_w.cpu().numpy(), layer.zero_w.cpu().numpy()
    wnp = layer.weight.detach().cpu().numpy()
    xq, xm = lo.fakequant_asym(x, sx, zx, 0, 255)
    wq, wm = lo.fakequant_asym(wnp, sw.reshape(-1, 1, 1, 1), zw.reshape(-1, 1, 1, 1), 0, 255)
    cols = lo.im2col_index(xq.astype(np.uint8), k, k, s, s, p, p, 1, 1, int(zx))
    widx = wq.reshape(O, -1).astype(np.uint8)
    sc = (np.float32(sx) * sw).astype(np.float64)
    t = lo.uint8_zero_point_correction(lo.bgemm_exact(cols, widx, lut), cols, widx, zx, zw)
    _close(y.flatten(2), t * sc[None, :, None] + layer.bias.detach().cpu().numpy().astype(np.float64)[None, :, None])
    g = go.reshape(B, O, -1).astype(np.float64) * sc[None, :, None]
    gcols, gw = lo.custom_backward(g, cols, widx, DX, DW)
    gcols = gcols - np.einsum("nol,o->nl", g, zw.astype(np.float64))[:, None, :]
    gw = gw - zx * g.sum(axis=(0, 2))[:, None]
    gx = lo.fold(gcols, C, H, W, k, k, s, s, p, p) * xm / max(np.float64(np.float32(sx)), 1e-12)
    gw = gw.reshape(wnp.shape) * wm / np.maximum(sw.astype(np.float64), 1e-12).reshape(-1, 1, 1, 1)
    _close(xt.grad, gx)
    _close(layer.weight.grad, gw)
    _close(layer.bias.grad, go.astype(np.float64).sum(axis=(0, 2, 3)))


# ------------------------------------------------------------------------------------------- statistics / calibration
def test_statistics_kernel_signed_zero_and_nan(dev):
    from approxtorch_b200.backend import ops
    # -0.0 mixed into negative data must not displace the true minimum; an all -0.0 tensor has max -0.0, not -inf
    x = -torch.rand(1 << 16, device=dev) - 0.5
    x[::7] = -0.0
    st = ops.absmax(x, want_minmax=True).cpu()
    assert st[1].item() == x.min().item() and st[2].item() == 0.0 and st[0].item() == x.abs().max().item()
    z = torch.full((4099,), -0.0, device=dev)
    st = ops.absmax(z, want_minmax=True).cpu()
    assert st[0].item() == 0.0 and st[1].item() == 0.0 and st[2].item() == 0.0
    for n in (5, 4096, 100003):
        y = torch.randn(n, device=dev)
        st = ops.absmax(y, want_minmax=True).cpu()
        assert st[0].item() == y.abs().max().item() and st[1].item() == y.min().item() and st[2].item() == y.max().item()
        y[n // 2] = float("nan")
        assert torch.isnan(ops.absmax(y, want_minmax=True)).all()
        assert torch.isnan(ops.absmax(y)[0])


def test_calibration_on_cuda_tensors(golden, dev, tmp_path):
    """The hooks' CUDA branch (one fused abs-max / min / max pass per activation) gives torch's statistics bit for
    bit on the same tensor, and a calibration run on the GPU reproduces the CPU fixture recorded from the
    reference's tool: weight ranges exactly, scales to 1e-6 (torch divides by a constant as a multiplication by its
    reciprocal on the GPU), activation statistics to rel 1e-5 (the float model's own convolutions run through a
    different library on the GPU)."""
    import torch.nn as nn
    import approxtorch_b200 as at
    from approxtorch_b200 import calib
    a = torch.randn(3, 5, 17, 19, device=dev) * 3
    am, mn, mx = calib._batch_stats(a)
    assert am.item() == a.abs().max().item() and mn.item() == a.amin().item() and mx.item() == a.amax().item()
    g = golden("calib")

    def model():
        torch.manual_seed(0)
        return nn.Sequential(nn.Conv2d(3, 4, 3, padding=1), nn.ReLU(), nn.Conv2d(4, 6, 3, padding=1),
                             nn.BatchNorm2d(6), nn.Conv2d(6, 5, 1, bias=False))
    data = [torch.from_numpy(d) for d in g["data"]]
    prev = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        sd = at.calib.calibrate_int8(model().to(dev), [(x, 0) for x in data], 10, str(tmp_path / "c.pt"), weight_bits=8)
        sdu = at.calib.calibrate_uint8(model().to(dev), data, None)
    finally:
        torch.backends.cudnn.allow_tf32 = prev
    assert list(sd.keys()) == list(g["i8_8_keys"]) and list(sdu.keys()) == list(g["u8_all_keys"])
    for k, v in sd.items():
        if k.endswith("scale_w"):
            np.testing.assert_allclose(v.cpu().numpy(), g[f"i8_8_{k}"], rtol=1e-6)
        elif k.endswith("scale_x"):
            np.testing.assert_allclose(v.cpu().numpy(), g[f"i8_8_{k}"], rtol=1e-5)
    for k, v in sdu.items():
        field = k.rsplit(".", 1)[-1]
        if field in ("w_min", "w_max"):
            np.testing.assert_array_equal(v.cpu().numpy(), g[f"u8_all_{k}"])
        elif field in ("x_min", "x_max", "scale_x", "scale_w"):
            np.testing.assert_allclose(v.cpu().numpy(), g[f"u8_all_{k}"], rtol=1e-5, atol=1e-7)
        elif field in ("zero_x", "zero_w"):
            assert np.abs(v.cpu().numpy() - g[f"u8_all_{k}"]).max() <= 1.0
