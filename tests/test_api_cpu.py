"""CPU-side checks: the public Python surface (the cases of the reference's own
tests/test_convert_model.py, restated), host-side statistics against the golden fixtures, the LUT
text loaders / slope generator, and that the C-ABI library exports what include/*.h declares."""

import inspect
import os
import re

import numpy as np
import pytest
import torch
import torch.nn as nn

import approxtorch_b200 as at
from approxtorch_b200.convert_model import convert_model
from approxtorch_b200.nn import Conv2d_int8, Conv2d_uint8
from approxtorch_b200.nn.Conv2d_uint8 import uint8_qparams

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture
def lut():
    return torch.zeros(256, 256, dtype=torch.float32)


def test_public_api_has_only_the_unified_entry():
    params = inspect.signature(convert_model).parameters
    assert list(params) == ["model", "lut", "qtype", "grad", "dx", "dw", "ignore_first_conv",
                            "scale_momentum", "update_scale", "weight_bits"]
    assert "x_quantizer" not in params and "w_quantizer" not in params
    assert not hasattr(at, "to_qat_int8")
    assert "x_quantizer" not in inspect.signature(Conv2d_int8).parameters


def test_int8_conversion_preserves_state_and_skips_first_conv(lut):
    model = nn.Sequential(nn.Conv2d(3, 4, 3, padding=1), nn.Sequential(nn.ReLU(), nn.Conv2d(4, 5, 1)))
    src = model[1][1]
    src.weight.requires_grad_(False)
    w0, b0 = src.weight.detach().clone(), src.bias.detach().clone()
    model.eval()
    out = convert_model(model, lut, qtype="int8", weight_bits=5)
    assert out is model
    assert isinstance(model[0], nn.Conv2d) and isinstance(model[1][1], Conv2d_int8)
    conv = model[1][1]
    torch.testing.assert_close(conv.weight, w0)
    torch.testing.assert_close(conv.bias, b0)
    assert not conv.weight.requires_grad and not conv.training and conv.weight_bits == 5
    torch.testing.assert_close(conv.scale_w, w0.abs().amax(dim=(1, 2, 3)) / 15)


def test_uint8_conversion_initialises_weight_qparams(lut):
    model = nn.Sequential(nn.Conv2d(2, 3, 3, bias=False))
    w0 = model[0].weight.detach().clone()
    convert_model(model, lut, qtype="uint8", ignore_first_conv=False, update_scale=False)
    conv = model[0]
    assert isinstance(conv, Conv2d_uint8) and conv.bias is None and not conv.update_scale
    torch.testing.assert_close(conv.weight, w0)
    mn, mx = w0.amin(dim=(1, 2, 3)), w0.amax(dim=(1, 2, 3))
    sc, zp = uint8_qparams(mn, mx)
    torch.testing.assert_close(conv.w_min, mn)
    torch.testing.assert_close(conv.w_max, mx)
    torch.testing.assert_close(conv.scale_w, sc)
    torch.testing.assert_close(conv.zero_w, zp)


def test_root_conv_is_returned_as_replacement(lut):
    src = nn.Conv2d(3, 4, 1)
    w0 = src.weight.detach().clone()
    conv = convert_model(src, lut, qtype="int8", ignore_first_conv=False)
    assert isinstance(conv, Conv2d_int8)
    torch.testing.assert_close(conv.weight, w0)


def test_unsupported_uint8_group_does_not_partially_convert(lut):
    model = nn.Sequential(nn.Conv2d(4, 4, 1), nn.Conv2d(4, 4, 3, padding=1, groups=2))
    with pytest.raises(NotImplementedError):
        convert_model(model, lut, qtype="uint8", ignore_first_conv=False)
    assert isinstance(model[0], nn.Conv2d) and isinstance(model[1], nn.Conv2d)


def test_invalid_arguments_fail_early(lut):
    model = nn.Sequential(nn.Conv2d(1, 1, 1))
    with pytest.raises(ValueError, match="qtype"):
        convert_model(model, lut, qtype="int4")
    with pytest.raises(ValueError, match="65536"):
        convert_model(model, torch.zeros(10))
    with pytest.raises(ValueError, match="weight_bits"):
        convert_model(model, lut, weight_bits=2)
    with pytest.raises(ValueError, match="fixed"):
        convert_model(model, lut, qtype="uint8", weight_bits=4)
    with pytest.raises(TypeError):
        convert_model(model, lut, weight_bits=True)
    with pytest.raises(ValueError, match="dx and dw"):
        Conv2d_int8(1, 1, 1, lut, grad="lre")
    with pytest.raises(NotImplementedError):
        Conv2d_int8(4, 8, 3, lut, groups=2)
    with pytest.raises(NotImplementedError):
        convert_model(nn.Sequential(nn.Conv2d(2, 2, 3, padding="same")), lut, ignore_first_conv=False)


def test_convert_model_matches_reference_fixture(golden):
    g = golden("setup")
    model = nn.Sequential(nn.Conv2d(3, 4, 3, padding=1), nn.ReLU(), nn.Conv2d(4, 5, 3, padding=1, bias=False),
                          nn.Conv2d(5, 5, 1))
    with torch.no_grad():
        model[2].weight.copy_(torch.from_numpy(g["cm_w1"]))
        model[3].weight.copy_(torch.from_numpy(g["cm_w2"]))
        model[3].bias.copy_(torch.from_numpy(g["cm_b2"]))
    convert_model(model, torch.from_numpy(g["lut"]), qtype="int8", weight_bits=6)
    assert [type(m).__name__ for m in model] == list(g["cm_types"])
    np.testing.assert_array_equal(model[2].scale_w.numpy(), g["cm_scale_w1"])
    np.testing.assert_array_equal(model[3].scale_w.numpy(), g["cm_scale_w2"])


def test_layer_statistics_match_reference_fixture(golden):
    """EMA host logic of both layers on CPU tensors against values recorded from the reference."""
    g = golden("stats")
    lut = torch.zeros(65536)
    for bits in (8, 5, 4, 3):
        layer = Conv2d_int8(4, 6, 3, lut, weight_bits=bits, scale_momentum=0.1, padding=1)
        with torch.no_grad():
            layer.weight.copy_(torch.from_numpy(g[f"i8_{bits}_w"]))
        layer._reset_scale_w_from_weight()
        np.testing.assert_array_equal(layer.scale_w.numpy(), g[f"i8_{bits}_scale_w0"])
        for step in range(3):
            with torch.no_grad():
                layer.weight.mul_(1.1)
            layer._update_scale(torch.from_numpy(g[f"i8_{bits}_xs"][step]))
            layer._update_scale_w()
            np.testing.assert_array_equal(layer.scale_x.numpy(), g[f"i8_{bits}_scale_x"][step])
            np.testing.assert_array_equal(layer.scale_w.numpy(), g[f"i8_{bits}_scale_w"][step])
    layer = Conv2d_uint8(4, 6, 3, lut, scale_momentum=0.25, padding=1)
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(g["u8_w"]))
        layer.w_min.copy_(layer.weight.amin(dim=(1, 2, 3)))
        layer.w_max.copy_(layer.weight.amax(dim=(1, 2, 3)))
    layer._reset_qparams_from_stats()
    for step in range(3):
        layer._update_scale(torch.from_numpy(g["u8_xs"][step]))
        layer._update_scale_w()
        state = torch.cat([layer.x_min.view(1), layer.x_max.view(1), layer.scale_x.view(1), layer.zero_x.view(1),
                           layer.w_min, layer.w_max, layer.scale_w, layer.zero_w]).numpy()
        np.testing.assert_array_equal(state, g["u8_state"][step])
    sc, zp = uint8_qparams(torch.from_numpy(g["qp_mn"]), torch.from_numpy(g["qp_mx"]))
    np.testing.assert_array_equal(sc.numpy(), g["qp_scale"])
    np.testing.assert_array_equal(zp.numpy(), g["qp_zero"])


def test_uint8_state_dict_compatibility():
    lut = torch.zeros(65536)
    a = Conv2d_uint8(2, 3, 3, lut)
    sd = a.state_dict()
    assert {"lut", "x_min", "x_max", "w_min", "w_max", "scale_x", "zero_x", "scale_w", "zero_w", "weight"} <= set(sd)
    legacy = {k: v for k, v in sd.items() if k not in ("scale_x", "zero_x", "scale_w", "zero_w")}
    legacy["x_min"] = torch.tensor(-1.0)
    legacy["x_max"] = torch.tensor(3.0)
    b = Conv2d_uint8(2, 3, 3, lut)
    b.load_state_dict(legacy)                      # min/max-only checkpoint: qparams are re-derived
    sx, zx = uint8_qparams(torch.tensor(-1.0), torch.tensor(3.0))
    torch.testing.assert_close(b.scale_x, sx)
    torch.testing.assert_close(b.zero_x, zx)
    bad = dict(sd)
    bad["zero_x"] = torch.tensor(3.5)
    with pytest.raises(RuntimeError, match="integer-valued"):
        Conv2d_uint8(2, 3, 3, lut).load_state_dict(bad)
    i8 = Conv2d_int8(2, 3, 3, lut, grad="lre", dx=torch.zeros(256), dw=torch.zeros(256))
    assert {"lut", "scale_x", "scale_w", "dx", "dw", "weight"} <= set(i8.state_dict())


def test_lut_loaders_and_slopes_match_reference_fixture(golden, tmp_path):
    g = golden("setup")
    path = tmp_path / "lut.txt"
    np.savetxt(path, g["lut"].reshape(256, 256).astype(np.int64), fmt="%d")
    loaded = at.load_lut.load_lut(str(path))
    assert loaded.dtype == torch.int32 and loaded.shape == (65536,)
    np.testing.assert_array_equal(loaded.numpy(), g["loaded_lut"])
    ga, gb = at.grad_lut.lre(str(path), "int8", str(tmp_path / "m"))
    np.testing.assert_allclose(ga, g["lre_grad_a"], rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(gb, g["lre_grad_b"], rtol=2e-6, atol=2e-6)
    la, lb = at.load_lut.load_lre_grad_lut(str(tmp_path / "m_lre_grad_a.txt"), str(tmp_path / "m_lre_grad_b.txt"))
    np.testing.assert_array_equal(la.numpy(), g["loaded_a"])
    np.testing.assert_array_equal(lb.numpy(), g["loaded_b"])
    da, db = at.grad_lut.DATE(g["lut"].reshape(256, 256), half_ws=8)
    assert da.shape == db.shape == (256, 256) and da.dtype == np.float32


def test_library_exports_every_declared_symbol():
    from approxtorch_b200.backend import _C
    header = open(os.path.join(REPO, "include", "approxtorch_b200.h")).read()
    declared = set(re.findall(r"\b(atb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_C.EXPORTED), declared ^ set(_C.EXPORTED)
    for name in declared:
        assert hasattr(_C.lib, name), name
    assert _C.lib.atb_version() >= 100
    plan = _C.GemmPlan()
    assert _C.lib.atb_lut_gemm_plan(65536, 576, 256, 4096, -1, plan) == 0
    # 16 x 8 row tiles x 4 column tiles of 36 k-chunks on 148 SMs: equal runs of 125 units, which end inside tiles
    assert (plan.block_rows, plan.chunks_per_tile, plan.blocks, plan.units_per_block, plan.cut_tiles) == (512, 36, 148, 125, 1)
    assert plan.scratch_bytes == 2048 + 2 * 148 * 133120
    assert _C.lib.atb_lut_gemm_plan(65536, 576, 256, 4096, 1 << 16, plan) == 0          # whole tiles only
    assert (plan.units_per_block, plan.blocks, plan.cut_tiles, plan.scratch_bytes) == (4 * 36, 128, 0, 0)
    # 3136 rows (a ResNet-50 stage-3 layer at batch 16): seven 512-row tiles x 16 column tiles x 16 chunks in equal runs
    assert _C.lib.atb_lut_gemm_plan(3136, 256, 1024, 0, -1, plan) == 0
    assert (plan.block_rows, plan.chunks_per_tile) == (512, 16) and plan.blocks <= 148
    assert plan.blocks * plan.units_per_block >= 7 * 16 * 16 > (plan.blocks - 1) * plan.units_per_block
    # fewer than 512 rows: one shorter tile (a multiple of the 32 rows a warp holds)
    assert _C.lib.atb_lut_gemm_plan(200, 64, 64, 0, -1, plan) == 0 and plan.block_rows == 224
    # every tile cut in three: more blocks than SMs is fine (nobody waits for anybody)
    assert _C.lib.atb_lut_gemm_plan(3136, 256, 1024, 0, (3 << 16) | 64, plan) == 0
    assert (plan.block_rows, plan.units_per_block, plan.blocks, plan.cut_tiles) == (64, 6, 49 * 16 * 16 // 6 + 1, 1)
    assert _C.lib.atb_lut_gemm_plan(100, 70000, 8, 0, -1, plan) != 0 and "65536" in _C.last_error()


def test_operators_are_registered_and_refuse_cpu_tensors():
    from approxtorch_b200.backend import ops
    for name in ops.OPERATOR_NAMES:
        assert hasattr(torch.ops.approxtorch, name), name
    with pytest.raises((RuntimeError, NotImplementedError)):
        ops.bgemm_fake_int8_claude(torch.zeros(1, 2, 3), torch.zeros(4, 2), torch.zeros(65536))
    with pytest.raises(RuntimeError, match="CUDA"):
        at.nn.quantization.static_quantize_int8(torch.zeros(4), torch.tensor(1.0))
    layer = Conv2d_int8(2, 3, 3, torch.zeros(65536), padding=1).eval()
    with pytest.raises((RuntimeError, NotImplementedError)):
        layer(torch.zeros(1, 2, 5, 5))


def test_install_as_approxtorch_alias():
    import sys
    saved = {k: v for k, v in sys.modules.items() if k == "approxtorch" or k.startswith("approxtorch.")}
    for k in saved:
        del sys.modules[k]
    try:
        at.install_as_approxtorch()
        import approxtorch
        assert approxtorch.convert_model is at.convert_model
        from approxtorch.nn import Conv2d_int8 as C
        assert C is Conv2d_int8
    finally:
        for k in [k for k in sys.modules if k == "approxtorch" or k.startswith("approxtorch.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_calibration_matches_reference_fixture(golden, tmp_path):
    """calibrate_int8 / calibrate_uint8 on a small float model against the checkpoints the reference's own
    calibration tool produced for the same model and batches (key order included)."""
    g = golden("calib")

    def model():
        torch.manual_seed(0)
        return nn.Sequential(nn.Conv2d(3, 4, 3, padding=1), nn.ReLU(), nn.Conv2d(4, 6, 3, padding=1),
                             nn.BatchNorm2d(6), nn.Conv2d(6, 5, 1, bias=False))
    data = [torch.from_numpy(d) for d in g["data"]]
    for bits in (8, 4):
        sd = at.calib.calibrate_int8(model(), [(x, 0) for x in data], 10, str(tmp_path / "c.pt"), weight_bits=bits)
        assert list(sd.keys()) == list(g[f"i8_{bits}_keys"])
        for k, v in sd.items():
            if k.endswith(("scale_x", "scale_w")):
                np.testing.assert_array_equal(v.numpy(), g[f"i8_{bits}_{k}"])
        assert torch.load(tmp_path / "c.pt").keys() == sd.keys()
    for n, tag in ((None, "all"), (7, "7")):
        m = model().train()
        sd = at.calib.calibrate_uint8(m, data, n)
        assert m.training                                    # train / eval flags are restored
        assert list(sd.keys()) == list(g[f"u8_{tag}_keys"])
        for k, v in sd.items():
            if k.rsplit(".", 1)[-1] in ("x_min", "x_max", "w_min", "w_max", "scale_x", "zero_x", "scale_w", "zero_w"):
                np.testing.assert_array_equal(v.numpy(), g[f"u8_{tag}_{k}"])
    # the uint8 checkpoint loads straight into a converted model
    lut = torch.zeros(65536)
    conv = convert_model(model(), lut, qtype="uint8")
    res = conv.load_state_dict(at.calib.calibrate_uint8(model(), data, None), strict=False)
    assert not res.unexpected_keys and all(k.endswith("lut") for k in res.missing_keys)
    with pytest.raises(ValueError):
        at.calib.calibrate_uint8(nn.Sequential(nn.Conv2d(1, 1, 1)), data, None)
    with pytest.raises(TypeError):
        at.calib.calibrate_uint8(model(), data, True)


def test_linear_layer_state_dict_uses_flat_names():
    import approxtorch_b200 as at
    from oracle import lut_oracle as lo
    lut = torch.from_numpy(lo.lut_exact_signed().reshape(-1)).float()
    a = at.nn.Linear_int8(12, 5, lut, bias=True)
    sd = a.state_dict()
    assert set(sd) == {"weight", "bias", "lut", "scale_x", "scale_w"} and tuple(sd["weight"].shape) == (5, 12)
    b = at.nn.Linear_int8(12, 5, lut, bias=True)
    b.load_state_dict(sd)
    assert torch.equal(a.weight, b.weight) and torch.equal(a.bias, b.bias)
    with pytest.raises(RuntimeError):
        a(torch.zeros(3, 11))
