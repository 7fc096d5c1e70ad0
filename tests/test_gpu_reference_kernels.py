"""This package's operators against the REFERENCE'S OWN maintained CUDA operators, rebuilt for sm_100a from the
reference checkout by ``oracle/build_ref_gpu.py`` and run in a process of their own
(``oracle/ref_gpu_worker.py``: both libraries register the same ``torch.ops.approxtorch`` schemas).
Same inputs to both sides: integer accumulators and 8-bit tensors must be bit-identical, fp32 gradients within
rel 1e-5.  Skipped when the reference library was not built."""

import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from oracle import lut_oracle as lo

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _have_ref():
    from oracle import build_ref_gpu
    return build_ref_gpu.built_library() is not None


def run_ref(op, *args):
    with tempfile.TemporaryDirectory() as d:
        req, rep = os.path.join(d, "req.npz"), os.path.join(d, "rep.npz")
        np.savez(req, op=np.array(op), **{f"arg{i}": np.asarray(a) for i, a in enumerate(args)})
        proc = subprocess.run([sys.executable, os.path.join(REPO, "oracle", "ref_gpu_worker.py"), req, rep],
                              capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        out = np.load(rep, allow_pickle=False)
        assert "error" not in out, str(out["error"])
        return [out[f"out{j}"] for j in range(len(out.files))]


def _t(a, dev):
    a = np.asarray(a)
    return torch.from_numpy(np.ascontiguousarray(a).reshape(a.shape)).to(dev)


def _close(got, ref, rtol=1e-5):
    got = got.detach().cpu().numpy().astype(np.float64)
    ref = ref.astype(np.float64)
    assert np.abs(got - ref).max() <= rtol * max(np.abs(ref).max(), 1e-30)


@pytest.fixture(scope="module")
def ref_ready():
    if not _have_ref():
        pytest.skip("reference CUDA operators not built (oracle/_ref/gpu)")


@pytest.mark.parametrize("shape", [(2, 37, 50, 11), (1, 576, 1024, 64), (3, 9, 7, 130), (64, 512, 1, 100), (1, 147, 600, 64)])
def test_forward_operators_bit_identical(dev, ref_ready, shape):
    from approxtorch_b200.backend import ops
    N, K, L, O = shape
    rng = np.random.default_rng(sum(shape))
    x = (rng.integers(-260, 260, (N, K, L)) * 0.5).astype(np.float32)        # ties, out-of-range values
    w = rng.integers(-128, 128, (O, K)).astype(np.float32)
    lut = np.round(rng.standard_normal(65536) * 100).astype(np.float32)       # the reference bench's table family
    ry, rxq, rwq = run_ref("bgemm_fake_int8_forward_cuda_claude_save", x, w, lut)
    y, xq, wq = ops.bgemm_fake_int8_claude_save(_t(x, dev), _t(w, dev), _t(lut, dev))
    np.testing.assert_array_equal(xq.cpu().numpy(), rxq)
    np.testing.assert_array_equal(wq.cpu().numpy(), rwq)
    np.testing.assert_array_equal(y.cpu().numpy(), ry)
    xu = rng.integers(0, 256, (N, K, L), dtype=np.uint8)
    wu = rng.integers(0, 256, (O, K)).astype(np.float32)
    ulut = lo.lut_unsigned_truncated(6).reshape(-1)
    (ry,) = run_ref("bgemm_fake_uint8_forward_cuda_claude", xu, wu, ulut)
    np.testing.assert_array_equal(ops.bgemm_fake_uint8_claude(_t(xu, dev), _t(wu, dev), _t(ulut, dev)).cpu().numpy(), ry)


def test_gemm_fakequant_and_map_operators(dev, ref_ready):
    from approxtorch_b200.backend import ops
    rng = np.random.default_rng(5)
    A = rng.integers(-128, 128, (70, 45)).astype(np.float32)
    B = rng.integers(-128, 128, (45, 130)).astype(np.float32)
    lut = lo.lut_affine_asymmetric().reshape(-1)
    ry, raq, rbq = run_ref("gemm_fake_int8_forward_cuda_claude_save", A, B, lut)
    y, aq, bq = ops.gemm_fake_int8_claude_save(_t(A, dev), _t(B, dev), _t(lut, dev))
    np.testing.assert_array_equal(y.cpu().numpy(), ry)
    np.testing.assert_array_equal(aq.cpu().numpy(), raq)
    np.testing.assert_array_equal(bq.cpu().numpy(), rbq)
    x = (rng.standard_normal(10007) * 3).astype(np.float32)
    s = np.array(0.0371, dtype=np.float32)
    rq, rm = run_ref("fakequant_per_tensor_claude", x, s, np.array(-127), np.array(127))
    q, m = torch.ops.approxtorch.fakequant_per_tensor_claude(_t(x, dev), _t(s, dev), -127, 127)
    np.testing.assert_array_equal(q.cpu().numpy(), rq)
    np.testing.assert_array_equal(m.cpu().numpy(), rm)
    go = rng.standard_normal(10007).astype(np.float32)
    (rg,) = run_ref("fakequant_per_tensor_backward_claude", go, rm, s)
    g = torch.ops.approxtorch.fakequant_per_tensor_backward_claude(_t(go, dev), m, _t(s, dev))
    np.testing.assert_array_equal(g.cpu().numpy(), rg)
    z = np.array(97.0, dtype=np.float32)
    rq, rm = run_ref("fakequant_per_tensor_asymmetric_claude", x, s, z, np.array(0), np.array(255))
    q, m = torch.ops.approxtorch.fakequant_per_tensor_asymmetric_claude(_t(x, dev), _t(s, dev), _t(z, dev), 0, 255)
    np.testing.assert_array_equal(q.cpu().numpy(), rq)
    np.testing.assert_array_equal(m.cpu().numpy(), rm)
    img = rng.integers(-128, 128, (2, 5, 9, 11)).astype(np.int8)
    (rc,) = run_ref("im2col_u8", img, *[np.array(v) for v in (3, 3, 2, 1, 1, 2, 1, 1)])
    np.testing.assert_array_equal(ops.im2col_u8(_t(img, dev), 3, (2, 1), (1, 2), 1).cpu().numpy(), rc)
    table = rng.standard_normal(256).astype(np.float32)
    (rmapped,) = run_ref("lut_map", img, table)
    np.testing.assert_array_equal(ops.lut_map(_t(img, dev), _t(table, dev)).cpu().numpy(), rmapped)
    (rpad,) = run_ref("lut_map_pad", img, table, np.array(2), np.array(1))
    np.testing.assert_array_equal(ops.lut_map_pad(_t(img, dev), _t(table, dev), (2, 1)).cpu().numpy(), rpad)


def test_backward_operators(dev, ref_ready):
    from approxtorch_b200.backend import ops
    rng = np.random.default_rng(9)
    N, K, L, O = 3, 40, 70, 24
    go = rng.standard_normal((N, O, L)).astype(np.float32)
    xq = rng.integers(0, 256, (N, K, L), dtype=np.uint8)
    wq_ko = rng.integers(0, 256, (K, O), dtype=np.uint8)
    dx = rng.standard_normal(256).astype(np.float32)
    dw = rng.standard_normal(256).astype(np.float32)
    rgx, rgw = run_ref("bgemm_lre_backward_claude", go, xq, wq_ko, dx, dw)
    gx, gw = ops.bgemm_lre_backward_claude(_t(go, dev), _t(xq, dev), _t(wq_ko, dev), _t(dx, dev), _t(dw, dev))
    _close(gx, rgx)
    _close(gw, rgw)
    DX = (rng.standard_normal(65536) * 5).astype(np.float32)
    wq_ok = np.ascontiguousarray(wq_ko.T)
    (rcx,) = run_ref("bgemm_custom_grad_uint8_dx", xq, wq_ok, go, DX)
    (rcw,) = run_ref("bgemm_custom_grad_uint8_dw", xq, wq_ok, go, DX)
    _close(ops.bgemm_custom_grad_uint8_dx(_t(xq, dev), _t(wq_ok, dev), _t(go, dev), _t(DX, dev)), rcx, 2e-5)
    _close(ops.bgemm_custom_grad_uint8_dw(_t(xq, dev), _t(wq_ok, dev), _t(go, dev), _t(DX, dev)), rcw, 2e-5)
    img = rng.integers(-128, 128, (2, 5, 8, 7)).astype(np.int8)
    w8 = rng.integers(-128, 128, (45, 6)).astype(np.int8)
    go2 = rng.standard_normal((2, 6, 4 * 7)).astype(np.float32)
    rgx, rgw = run_ref("bgemm_lre_backward_claude_im2col", go2, img, w8, dx, dw,
                       *[np.array(v) for v in (3, 3, 2, 1, 1, 1, 1, 1)])
    gx, gw = ops.bgemm_lre_backward_claude_im2col(_t(go2, dev), _t(img, dev), _t(w8, dev), _t(dx, dev), _t(dw, dev),
                                                  3, (2, 1), 1, 1)
    _close(gx, rgx)
    _close(gw, rgw)
