"""Generate the golden fixtures in this folder FROM THE REFERENCE ITSELF.

Run where the reference checkout is available (its path is the optional argument):

    python tests/golden/make_golden.py [reference_root]

It imports the reference's Python modules (with the compiled extension stubbed
out: only its pure-torch CPU branches are exercised) and runs the reference's
own CPU LUT-BGEMM operator compiled by ``oracle/build_ref.py``.  Inputs are
stored next to outputs so the fixtures do not depend on any RNG implementation.
The fixtures pin the oracle (``tests/test_oracle_golden.py``) and, through the
same inputs, the CUDA path (``tests/test_gpu_bgemm.py``, ``tests/test_gpu_quant.py``, ``tests/test_gpu_conv.py``).
"""

from __future__ import annotations

import os
import sys
import tempfile
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
from oracle.build_ref import reference_root        # noqa: E402

REF = sys.argv[1] if len(sys.argv) > 1 else reference_root()
if not REF:
    sys.exit("usage: make_golden.py <reference checkout>  (or set APPROXTORCH_REF)")
sys.path.insert(0, REF)
sys.modules["approxtorch.backend._C"] = types.ModuleType("approxtorch.backend._C")

import approxtorch as ref_at                       # noqa: E402  (the reference)
from approxtorch.nn import quantization as ref_q   # noqa: E402
from approxtorch.nn.Conv2d_uint8 import uint8_qparams as ref_qparams  # noqa: E402
from oracle import build_ref, lut_oracle as lo     # noqa: E402


def save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}.npz  {os.path.getsize(path) / 1024:.1f} KiB")


def t2n(t):
    return t.detach().cpu().numpy().copy()


# ---------------------------------------------------------------- fake-quant
def golden_fakequant():
    g = torch.Generator().manual_seed(11)
    out = {}
    # per-tensor symmetric, with exact .5 ties, clip boundaries and odd length
    s = torch.tensor(0.0625)
    ties = (torch.arange(-300, 301, dtype=torch.float32) * 0.5) * s
    x = torch.cat([torch.randn(1001, generator=g) * 3.0, ties,
                   torch.tensor([127.0, 127.5, 127.49, -127.0, -127.5, -128.0, 0.0, -0.0]) * s])
    for tag, scale, qmin, qmax in (("a", s, -127, 127), ("b", torch.tensor(0.3), -7, 7),
                                   ("c", torch.tensor(0.0), -127, 127),
                                   ("d", torch.tensor(1e-3), -3, 3)):
        xi = x.clone().requires_grad_(True)
        q = ref_q.static_quantize_int8(xi, scale, qmin, qmax)
        go = torch.randn(x.shape, generator=g)
        q.backward(go)
        out.update({f"sym_{tag}_x": t2n(x), f"sym_{tag}_scale": t2n(scale),
                    f"sym_{tag}_qrange": np.array([qmin, qmax]),
                    f"sym_{tag}_q": t2n(q), f"sym_{tag}_go": t2n(go),
                    f"sym_{tag}_gx": t2n(xi.grad)})
    # per-tensor asymmetric
    for tag, scale, zero, qmin, qmax in (("a", torch.tensor(0.021), torch.tensor(117.0), 0, 255),
                                         ("b", torch.tensor(0.4), torch.tensor(3.0), 0, 15)):
        xa = torch.cat([torch.randn(777, generator=g) * 2.0,
                        (torch.arange(-40, 41, dtype=torch.float32) * 0.5) * scale])
        xi = xa.clone().requires_grad_(True)
        q = ref_q.static_quantize_uint8(xi, scale, zero, qmin, qmax)
        go = torch.randn(xa.shape, generator=g)
        q.backward(go)
        out.update({f"asym_{tag}_x": t2n(xa), f"asym_{tag}_scale": t2n(scale),
                    f"asym_{tag}_zero": t2n(zero), f"asym_{tag}_qrange": np.array([qmin, qmax]),
                    f"asym_{tag}_q": t2n(q), f"asym_{tag}_go": t2n(go),
                    f"asym_{tag}_gx": t2n(xi.grad)})
    # per-channel symmetric weights at 3..8 bits
    w = torch.randn(6, 5, 3, 3, generator=g) * 0.2
    w[2] = 0.0
    for bits in range(3, 9):
        qm = 2 ** (bits - 1) - 1
        am = w.abs().amax(dim=(1, 2, 3))
        sc = torch.where(am > 0, am / qm, torch.ones_like(am))
        wi = w.clone().requires_grad_(True)
        q = ref_q.static_quantize_int8(wi, sc, -qm, qm, ch_axis=0)
        go = torch.randn(w.shape, generator=g)
        q.backward(go)
        out.update({f"pc_{bits}_scale": t2n(sc), f"pc_{bits}_q": t2n(q),
                    f"pc_{bits}_go": t2n(go), f"pc_{bits}_gx": t2n(wi.grad)})
    out["pc_w"] = t2n(w)
    # per-channel asymmetric
    mn = w.amin(dim=(1, 2, 3))
    mx = w.amax(dim=(1, 2, 3))
    sc, zp = ref_qparams(mn, mx, 255)
    q = ref_q.static_quantize_uint8(w, sc, zp, 0, 255, ch_axis=0)
    out.update({"pca_scale": t2n(sc), "pca_zero": t2n(zp), "pca_q": t2n(q)})
    save("fakequant", **out)


# ---------------------------------------------------------------- EMA / qparams
def golden_stats():
    g = torch.Generator().manual_seed(5)
    lut = torch.zeros(65536)
    out = {}
    for bits in (8, 5, 4, 3):
        layer = ref_at.nn.Conv2d_int8(4, 6, 3, lut, weight_bits=bits, scale_momentum=0.1,
                                      padding=1)
        with torch.no_grad():
            layer.weight.copy_(torch.randn(layer.weight.shape, generator=g) * 0.3)
            layer.weight[1].zero_()
        layer._reset_scale_w_from_weight()
        out[f"i8_{bits}_w"] = t2n(layer.weight)
        out[f"i8_{bits}_scale_w0"] = t2n(layer.scale_w)
        xs, sx, sw = [], [], []
        for step in range(3):
            x = torch.randn(2, 4, 5, 5, generator=g) * (1.0 + step)
            with torch.no_grad():
                layer.weight.mul_(1.1)
            layer._update_scale(x)
            layer._update_scale_w()
            xs.append(t2n(x)); sx.append(t2n(layer.scale_x).copy()); sw.append(t2n(layer.scale_w).copy())
        out[f"i8_{bits}_xs"] = np.stack(xs)
        out[f"i8_{bits}_scale_x"] = np.stack(sx)
        out[f"i8_{bits}_scale_w"] = np.stack(sw)
    layer = ref_at.nn.Conv2d_uint8(4, 6, 3, lut, scale_momentum=0.25, padding=1)
    with torch.no_grad():
        layer.weight.copy_(torch.randn(layer.weight.shape, generator=g) * 0.3)
        layer.weight[3].abs_()
        layer.w_min.copy_(layer.weight.amin(dim=(1, 2, 3)))
        layer.w_max.copy_(layer.weight.amax(dim=(1, 2, 3)))
    layer._reset_qparams_from_stats()
    out["u8_w"] = t2n(layer.weight)
    xs, st = [], []
    for step in range(3):
        x = torch.randn(2, 4, 5, 5, generator=g) + 0.5 * step
        layer._update_scale(x)
        layer._update_scale_w()
        xs.append(t2n(x))
        st.append(np.concatenate([t2n(layer.x_min).reshape(1), t2n(layer.x_max).reshape(1),
                                  t2n(layer.scale_x).reshape(1), t2n(layer.zero_x).reshape(1),
                                  t2n(layer.w_min), t2n(layer.w_max), t2n(layer.scale_w),
                                  t2n(layer.zero_w)]))
    out["u8_xs"] = np.stack(xs)
    out["u8_state"] = np.stack(st)
    mn = torch.tensor([-1.0, 0.2, -3.0, 0.0, -1e-20, -0.7])
    mx = torch.tensor([2.0, 0.9, -1.0, 0.0, 1e-20, 0.7])
    sc, zp = ref_qparams(mn, mx, 255)
    out.update({"qp_mn": t2n(mn), "qp_mx": t2n(mx), "qp_scale": t2n(sc), "qp_zero": t2n(zp)})
    save("stats", **out)


# ---------------------------------------------------------------- LUT-BGEMM by the reference CPU op
def golden_bgemm():
    assert build_ref.build(REF), "reference CPU operator did not build"
    rng = np.random.default_rng(3)
    tables = {
        "affine": lo.lut_affine_asymmetric(),
        "noisy": lo.lut_signed_noisy(64, seed=1),
        "trunc4": lo.lut_signed_truncated(4),
        "utrunc6": lo.lut_unsigned_truncated(6),
    }
    out = {}
    shapes = [(2, 37, 50, 11), (1, 576, 96, 64), (3, 9, 7, 130), (4, 64, 1, 33)]
    for name, tab in tables.items():
        out[f"lut_{name}"] = tab.reshape(-1)
        for si, (N, K, L, O) in enumerate(shapes):
            x = rng.integers(0, 256, (N, K, L), dtype=np.uint8)
            w = rng.integers(0, 256, (O, K), dtype=np.uint8)
            y = build_ref.bgemm_lut_xw(x, w, tab).numpy()
            out[f"{name}_{si}_x"] = x
            out[f"{name}_{si}_w"] = w
            out[f"{name}_{si}_y"] = y.astype(np.int32)
    # the reference's signed entry point on int8 dtypes (checks the +128 offset rule)
    x8 = rng.integers(-128, 128, (2, 21, 13), dtype=np.int8)
    w8 = rng.integers(-128, 128, (5, 21), dtype=np.int8)
    tT = torch.from_numpy(tables["affine"]).reshape(256, 256).t().contiguous().reshape(-1).to(torch.int32)
    y8 = torch.ops.approxtorch.bgemm_int8(torch.from_numpy(x8), torch.from_numpy(w8), tT).numpy()
    out.update({"int8_x": x8, "int8_w": w8, "int8_y": y8.astype(np.int32)})
    save("bgemm_ref_cpu", **out)


# ---------------------------------------------------------------- whole layer, composed from reference pieces
def golden_conv_layer():
    """Conv2d_int8 forward restated with the reference's own pieces on CPU:
    its fake-quant Functions, torch unfold (+128), its CPU LUT-BGEMM, its dequant
    expression.  Config-0 shaped but spatially smaller so the file stays small."""
    assert build_ref.build(REF)
    torch.manual_seed(0)
    B, C, H, W, O = 2, 16, 12, 12, 24
    x = torch.randn(B, C, H, W)
    w = torch.nn.init.kaiming_normal_(torch.empty(O, C, 3, 3))
    bias = torch.randn(O) * 0.1
    lut = lo.lut_signed_truncated(4)
    scale_x = x.abs().max() / 127
    am = w.abs().amax(dim=(1, 2, 3))
    out = {"x": t2n(x), "w": t2n(w), "bias": t2n(bias), "lut": lut.reshape(-1),
           "scale_x": t2n(scale_x)}
    for bits in (8, 4):
        qm = 2 ** (bits - 1) - 1
        scale_w = am / qm
        for (s, p) in ((1, 1), (2, 0)):
            xq = ref_q.static_quantize_int8(x, scale_x, -127, 127)
            wq = ref_q.static_quantize_int8(w, scale_w, -qm, qm, ch_axis=0)
            xu = torch.nn.functional.unfold(xq, 3, padding=p, stride=s) + 128
            y = build_ref.bgemm_lut_xw(xu.to(torch.uint8), (wq.view(O, -1) + 128).to(torch.uint8), lut)
            OH = (H + 2 * p - 3) // s + 1
            yf = y.to(torch.float32).view(B, O, OH, OH)
            sc = (scale_x * scale_w).view(1, -1, 1, 1)
            out[f"b{bits}_s{s}p{p}_yint"] = y.numpy().astype(np.int32)
            out[f"b{bits}_s{s}p{p}_y"] = t2n(torch.addcmul(bias.view(1, -1, 1, 1), yf, sc))
            out[f"b{bits}_scale_w"] = t2n(scale_w)
    save("conv_layer", **out)


# ---------------------------------------------------------------- LRE slopes, LUT file loader, convert_model
def golden_setup():
    out = {}
    lut = lo.lut_signed_noisy(128, seed=4)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "lut.txt")
        np.savetxt(path, lut.reshape(256, 256).astype(np.int64), fmt="%d")
        ga, gb = ref_at.grad_lut.lre(path, "int8", None)
        loaded = ref_at.load_lut.load_lut(path)
        np.savetxt(os.path.join(d, "a.txt"), ga, fmt="%.4f")
        np.savetxt(os.path.join(d, "b.txt"), gb, fmt="%.4f")
        la, lb = ref_at.load_lut.load_lre_grad_lut(os.path.join(d, "a.txt"), os.path.join(d, "b.txt"))
    out.update({"lut": lut.reshape(-1), "lre_grad_a": ga, "lre_grad_b": gb,
                "loaded_lut": t2n(loaded), "loaded_a": t2n(la), "loaded_b": t2n(lb)})
    torch.manual_seed(2)
    model = torch.nn.Sequential(torch.nn.Conv2d(3, 4, 3, padding=1), torch.nn.ReLU(),
                                torch.nn.Conv2d(4, 5, 3, padding=1, bias=False),
                                torch.nn.Conv2d(5, 5, 1))
    out["cm_w1"] = t2n(model[2].weight); out["cm_w2"] = t2n(model[3].weight)
    out["cm_b2"] = t2n(model[3].bias)
    ref_at.convert_model(model, torch.from_numpy(lut), qtype="int8", weight_bits=6)
    out["cm_scale_w1"] = t2n(model[2].scale_w); out["cm_scale_w2"] = t2n(model[3].scale_w)
    out["cm_types"] = np.array([type(m).__name__ for m in model])
    save("setup", **out)


# ---------------------------------------------------------------- calibration tool
def calib_model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Conv2d(3, 4, 3, padding=1), torch.nn.ReLU(), torch.nn.Conv2d(4, 6, 3, padding=1),
                               torch.nn.BatchNorm2d(6), torch.nn.Conv2d(6, 5, 1, bias=False))


def golden_calib():
    import contextlib
    import io
    g = torch.Generator().manual_seed(1)
    data = [torch.randn(4, 3, 8, 8, generator=g) for _ in range(3)]
    out = {"data": np.stack([t2n(d) for d in data])}
    with tempfile.TemporaryDirectory() as d, contextlib.redirect_stdout(io.StringIO()):
        for bits in (8, 4):
            sd = ref_at.calib.calibrate_int8(calib_model(), [(x, 0) for x in data], 10, os.path.join(d, "c.pt"), weight_bits=bits)
            out[f"i8_{bits}_keys"] = np.array(list(sd.keys()))
            for k, v in sd.items():
                if k.endswith(("scale_x", "scale_w")):
                    out[f"i8_{bits}_{k}"] = t2n(v)
        for n in (None, 7):
            sd = ref_at.calib.calibrate_uint8(calib_model(), data, n)
            tag = "all" if n is None else str(n)
            out[f"u8_{tag}_keys"] = np.array(list(sd.keys()))
            for k, v in sd.items():
                if k.rsplit(".", 1)[-1] in ("x_min", "x_max", "w_min", "w_max", "scale_x", "zero_x", "scale_w", "zero_w"):
                    out[f"u8_{tag}_{k}"] = t2n(v)
    save("calib", **out)


if __name__ == "__main__":
    golden_calib()
    golden_fakequant()
    golden_stats()
    golden_bgemm()
    golden_conv_layer()
    golden_setup()
