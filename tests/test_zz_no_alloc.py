"""The allocation-free LUT-GEMM entry point (parked partial sums in the library's built-in scratch area)
must give exactly what the ordinary entry point gives with a caller-supplied scratch buffer.

It serves hosts that cannot allocate device memory at call time (graph capture, closed memory pools,
foreign-runtime bindings).  The scratch holds the partial sums that blocks park when a tile is cut between them.  Checked through the C ABI on two calls in a row with different data, so that
whatever the first call left in the shared area cannot leak into the second.  This file sorts last so a
run that stops at the first failure has already exercised everything else."""

import ctypes

import numpy as np
import pytest
import torch

from oracle import lut_oracle as lo

pytestmark = pytest.mark.gpu


def _call_both(ops, _C, x, w, image, N, K, L, O, cfg, epilogue=(None, None, None, None, None)):
    lib = _C.lib
    plan = _C.GemmPlan()
    assert lib.atb_lut_gemm_plan(N * L, K, O, 0, cfg, ctypes.byref(plan)) == 0
    assert plan.cut_tiles and 0 < plan.scratch_bytes <= lib.atb_static_scratch_bytes()
    stream = ops._stream(x)
    ep = [ops._ptr(t) for t in epilogue]                      # alpha, beta, zero_x, zero_w, wsum
    y_ref = torch.empty((N, O, L), dtype=torch.float32, device=x.device)
    scratch = torch.empty(plan.scratch_bytes, dtype=torch.uint8, device=x.device)
    _C.check(lib.atb_lut_bgemm_fwd(ops._ptr(x), ops._ptr(w), ops._ptr(image), ops._ptr(y_ref), N, K, L, O, 0, 0,
                                   *ep, cfg, ops._ptr(scratch), plan.scratch_bytes, stream),
             "atb_lut_bgemm_fwd")
    y_new = torch.full((N, O, L), float("nan"), dtype=torch.float32, device=x.device)
    _C.check(lib.atb_lut_bgemm_fwd_noalloc(ops._ptr(x), ops._ptr(w), ops._ptr(image), ops._ptr(y_new), N, K, L, O,
                                           0, 0, *ep, cfg, stream),
             "atb_lut_bgemm_fwd_noalloc")
    return y_ref, y_new


def test_noalloc_entry_matches_caller_scratch_entry(dev):
    from approxtorch_b200.backend import ops, _C
    rng = np.random.default_rng(77)
    lut = lo.lut_signed_noisy(64, seed=8)
    image = ops.lut_image(torch.from_numpy(lut.reshape(-1)).to(dev))
    cfg = (4 << 16) | 128                           # 128-row tiles, each cut into four k-segments: needs scratch
    for call, (N, K, L, O) in enumerate([(2, 200, 300, 70), (3, 160, 129, 33)]):
        x = torch.from_numpy(rng.integers(0, 256, (N, K, L), dtype=np.uint8)).to(dev)
        w = torch.from_numpy(rng.integers(0, 256, (O, K), dtype=np.uint8)).to(dev)
        y_ref, y_new = _call_both(ops, _C, x, w, image, N, K, L, O, cfg)
        torch.cuda.synchronize()
        assert torch.equal(y_ref, y_new), f"call {call}: outputs differ"
        oracle = lo.bgemm_exact(x.cpu().numpy(), w.cpu().numpy(), lut)
        np.testing.assert_array_equal(y_new.cpu().numpy().astype(np.int64), oracle)


def test_noalloc_entry_with_zero_points_and_stream_k(dev):
    """The row-sum part of the parking slots (zero-point epilogue), with every tile cut into segments and under the
    automatic plan, through both entry points: bit-identical, and equal to the exactly corrected oracle sum."""
    from approxtorch_b200.backend import ops, _C
    assert _C.lib.atb_static_scratch_bytes() == 32 << 20        # this call also performs the address lookup
    rng = np.random.default_rng(78)
    lut = lo.lut_unsigned_truncated(6)
    image = ops.lut_image(torch.from_numpy(lut.reshape(-1)).to(dev))
    N, K, L, O = 2, 200, 300, 70
    zx, zw = 113.0, rng.integers(100, 150, O).astype(np.float32)
    for call, cfg in enumerate(((4 << 16) | 128, (7 << 16) | 96, -1)):
        x = torch.from_numpy(rng.integers(0, 256, (N, K, L), dtype=np.uint8)).to(dev)
        w = torch.from_numpy(rng.integers(0, 256, (O, K), dtype=np.uint8)).to(dev)
        wsum = w.sum(dim=1, dtype=torch.int32)
        ep = (None, None, torch.tensor(zx, device=dev), torch.from_numpy(zw).to(dev), wsum)
        y_ref, y_new = _call_both(ops, _C, x, w, image, N, K, L, O, cfg, ep)
        torch.cuda.synchronize()
        assert torch.equal(y_ref, y_new), f"call {call}: outputs differ"
        xs, wn = x.cpu().numpy(), w.cpu().numpy()
        exact = lo.uint8_zero_point_correction(lo.bgemm_exact(xs, wn, lut), xs, wn, zx, zw)
        np.testing.assert_array_equal(y_new.cpu().numpy(), exact.astype(np.float32))


def test_noalloc_entry_refuses_oversized_shapes(dev):
    from approxtorch_b200.backend import ops, _C
    lib = _C.lib
    limit = lib.atb_static_scratch_bytes()
    N, K, L, O = 1, 64, 1 << 20, 64                 # 2048 tiles cut in four: two parking slots for each of 8192 blocks
    plan = _C.GemmPlan()
    cfg = (4 << 16) | 512
    assert lib.atb_lut_gemm_plan(N * L, K, O, 0, cfg, ctypes.byref(plan)) == 0 and plan.scratch_bytes > limit
    dummy = torch.zeros(16, dtype=torch.uint8, device=dev)
    rc = lib.atb_lut_bgemm_fwd_noalloc(ops._ptr(dummy), ops._ptr(dummy), ops._ptr(dummy), ops._ptr(dummy), N, K, L, O,
                                       0, 0, None, None, None, None, None, cfg, ops._stream(dummy))
    assert rc == 3 and "built-in area" in _C.last_error()
