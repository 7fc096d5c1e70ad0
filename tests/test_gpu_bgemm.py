"""GPU parity of the LUT-BGEMM / GEMM forward operators (through the C ABI) against the CPU oracle and
the fixtures recorded from the reference's CPU operator.  Integer tables: bit-exact."""

import numpy as np
import pytest
import torch

from oracle import c_oracle, lut_oracle as lo

pytestmark = pytest.mark.gpu


def _ops():
    from approxtorch_b200.backend import ops
    return ops


def _t(a, dev):
    a = np.asarray(a)
    return torch.from_numpy(np.ascontiguousarray(a).reshape(a.shape)).to(dev)


@pytest.mark.parametrize("name", ["affine", "noisy", "trunc4", "utrunc6"])
def test_matches_reference_cpu_operator_fixture(golden, dev, name):
    ops = _ops()
    g = golden("bgemm_ref_cpu")
    lut = _t(g[f"lut_{name}"], dev)
    for si in range(4):
        x, w, y = g[f"{name}_{si}_x"], g[f"{name}_{si}_w"], g[f"{name}_{si}_y"]
        # uint8 operator on raw indices (fp32 weights, uint8-dtype x = indices)
        out = ops.bgemm_fake_uint8_claude(_t(x, dev), _t(w.astype(np.float32), dev), lut)
        np.testing.assert_array_equal(out.cpu().numpy(), y.astype(np.float32))
        # fp32 x takes the rounding prepass and must agree bit for bit
        out2 = ops.bgemm_fake_uint8_claude(_t(x.astype(np.float32), dev), _t(w.astype(np.float32), dev), lut)
        assert torch.equal(out, out2)
        # int8 operator on shifted values: uint8_op(x, w) == int8_op(x - 128, w - 128)
        out3 = ops.bgemm_fake_int8_claude(_t(x.astype(np.float32) - 128, dev), _t(w.astype(np.float32) - 128, dev), lut)
        assert torch.equal(out, out3)


# (N, K, L, O): tails in every dimension, K below/above one operand chunk, L == 1, tiny and wide O
SHAPES = [(1, 1, 1, 1), (2, 17, 33, 5), (3, 64, 100, 64), (1, 130, 513, 65), (4, 48, 1, 200),
          (2, 576, 96, 64), (1, 31, 700, 129), (5, 16, 7, 3), (64, 512, 1, 100)]


@pytest.mark.parametrize("shape", SHAPES)
def test_shape_sweep_against_oracle(dev, shape):
    ops = _ops()
    N, K, L, O = shape
    rng = np.random.default_rng(hash(shape) & 0xffff)
    x = rng.integers(0, 256, (N, K, L), dtype=np.uint8)
    w = rng.integers(-128, 128, (O, K)).astype(np.float32)
    lut = lo.lut_signed_noisy(64, seed=2)
    ref = c_oracle.bgemm_u8(x, lo.to_lut_index(w, 128), lut)
    y, xq, wq = ops.bgemm_fake_int8_claude_save(_t(x, dev), _t(w, dev), _t(lut.reshape(-1), dev))
    np.testing.assert_array_equal(y.cpu().numpy().astype(np.float64), ref)
    assert xq.dtype == torch.uint8 and wq.dtype == torch.uint8 and tuple(wq.shape) == (O, K)
    np.testing.assert_array_equal(wq.cpu().numpy(), lo.to_lut_index(w, 128))


@pytest.mark.parametrize("cfg", [-1, 0, 7, 100, 32, 64, 96, 128, 256, 320, 512, (3 << 16) | 128, (2 << 16) | 512, (5 << 16),
                                 (1 << 16) | 448, (13 << 16) | 160, (1 << 24) | 256, (1 << 24) | (2 << 16) | 64])
def test_forced_tilings_and_split_k_are_bit_identical(dev, cfg):
    ops = _ops()
    rng = np.random.default_rng(5)
    N, K, L, O = 2, 200, 300, 70
    x = rng.integers(0, 256, (N, K, L), dtype=np.uint8)
    w = rng.integers(-128, 128, (O, K)).astype(np.float32)
    lut = lo.lut_affine_asymmetric()
    ref = c_oracle.bgemm_u8(x, lo.to_lut_index(w, 128), lut)
    y = torch.ops.approxtorch.bgemm_fake_int8_forward_cuda_claude_cfg(_t(x, dev), _t(w, dev), _t(lut.reshape(-1), dev), cfg)
    np.testing.assert_array_equal(y.cpu().numpy().astype(np.float64), ref)


def test_rounding_prepass_and_save_contract(dev):
    ops = _ops()
    rng = np.random.default_rng(9)
    x = (rng.integers(-300, 300, (2, 23, 40)) * 0.5).astype(np.float32)      # ties and out-of-range values
    w = (rng.integers(-300, 300, (6, 23)) * 0.5).astype(np.float32)
    lut = lo.lut_signed_noisy(64, seed=3)
    y, xq, wq = ops.bgemm_fake_int8_claude_save(_t(x, dev), _t(w, dev), _t(lut.reshape(-1), dev))
    np.testing.assert_array_equal(xq.cpu().numpy(), lo.to_lut_index(x, 128))
    np.testing.assert_array_equal(wq.cpu().numpy(), lo.to_lut_index(w, 128))
    ref = lo.bgemm_exact(lo.to_lut_index(x, 128), lo.to_lut_index(w, 128), lut)
    np.testing.assert_array_equal(y.cpu().numpy().astype(np.int64), ref)
    # uint8-dtype x: the returned index image aliases the input
    xi = _t(lo.to_lut_index(x, 128), dev)
    y2, xq2, _ = ops.bgemm_fake_int8_claude_save(xi, _t(w, dev), _t(lut.reshape(-1), dev))
    assert xq2.data_ptr() == xi.data_ptr() and torch.equal(y, y2)
    # misaligned storage offsets take the scalar paths
    big = torch.zeros(x.size + 3, dtype=torch.float32, device=dev)
    big[3:] = _t(x, dev).flatten()
    y3 = ops.bgemm_fake_int8_claude(big[3:].view(x.shape), _t(w, dev), _t(lut.reshape(-1), dev))
    assert torch.equal(y, y3)


def test_lut_classes(dev):
    """int16-exact, uint16-exact (incl. 0 / 32768 / 65535), beyond-int16 mixed sign and non-integer
    tables: 16-bit classes are bit-exact; fp32-class tables follow the ascending-k fp32 sum."""
    ops = _ops()
    rng = np.random.default_rng(21)
    N, K, L, O = 2, 75, 50, 40
    x = rng.integers(0, 256, (N, K, L), dtype=np.uint8)
    w = rng.integers(0, 256, (O, K)).astype(np.float32)
    wi = w.astype(np.uint8)
    edge16 = rng.integers(-32767, 32768, (256, 256)).astype(np.float32)
    edge16[0, 0], edge16[1, 1] = 32767, -32767
    u16 = rng.integers(0, 65536, (256, 256)).astype(np.float32)
    u16[0, 0], u16[0, 1], u16[0, 2] = 0, 65535, 32768
    for tab in (edge16, u16, lo.lut_exact_unsigned()):
        assert lo.lut_class(tab) in ("i16", "u16")
        y = ops.bgemm_fake_uint8_claude(_t(x, dev), _t(w, dev), _t(tab.reshape(-1), dev))
        np.testing.assert_array_equal(y.cpu().numpy().astype(np.float64), c_oracle.bgemm_u8(x, wi, tab))
    mixed = edge16.copy(); mixed[5, 5] = 40000.0; mixed[6, 6] = -40000.0
    half = (rng.integers(-2000, 2000, (256, 256)) * 0.5).astype(np.float32)
    for tab in (mixed, half):
        assert lo.lut_class(tab) == "f32"
        y = ops.bgemm_fake_uint8_claude(_t(x, dev), _t(w, dev), _t(tab.reshape(-1), dev))
        np.testing.assert_array_equal(y.cpu().numpy(), lo.bgemm_f32_ascending(x, wi, tab))
    # exact product table == integer einsum
    y = ops.bgemm_fake_uint8_claude(_t(x, dev), _t(w, dev), _t(lo.lut_exact_unsigned().reshape(-1), dev))
    ref = np.einsum("nkl,ok->nol", x.astype(np.int64), wi.astype(np.int64))
    np.testing.assert_array_equal(y.cpu().numpy().astype(np.int64), ref)


def test_fp32_class_table_on_chip_equals_the_global_gather(dev):
    """Tables that are not 16-bit exact: the kernel that keeps the fp32 table in a two-block cluster's shared memory,
    the same kernel staging from global memory, and the generic kernel's gather from global memory all sum in fp32
    in ascending k, so they agree bit for bit with each other and with the ascending-k oracle - column operand,
    row-major operand, image operand, with the zero-point epilogue, odd sizes."""
    ops = _ops()
    rng = np.random.default_rng(61)
    tab = (rng.integers(-3000, 3000, (256, 256)) * 0.25).astype(np.float32)          # sums round in fp32
    assert lo.lut_class(tab) == "f32"
    lt = _t(tab.reshape(-1), dev)
    img = ops.lut_image(lt)
    assert ops._class_flag(img) == 1 << 24
    N, K, L, O = 3, 150, 700, 70
    x = rng.integers(0, 256, (N, K, L), dtype=np.uint8)
    w = rng.integers(0, 256, (O, K), dtype=np.uint8)
    ref = lo.bgemm_f32_ascending(x, w, tab)
    outs = []
    for cfg in (-1, 1 << 25):                                 # cluster shared memory / staging from global memory
        y = torch.empty((N, O, L), dtype=torch.float32, device=dev)
        ops.lut_gemm_launch(_t(x, dev), _t(w, dev), img, y, N, K, L, O, cfg=cfg)
        outs.append(y)
    ops.FP32_TABLE_ON_CHIP = False
    try:
        y = torch.empty((N, O, L), dtype=torch.float32, device=dev)
        ops.lut_gemm_launch(_t(x, dev), _t(w, dev), img, y, N, K, L, O, cfg=1 << 16)          # generic kernel, whole tiles
        outs.append(y)
    finally:
        ops.FP32_TABLE_ON_CHIP = True
    for y in outs:
        np.testing.assert_array_equal(y.cpu().numpy(), ref)
    # row-major operand (L == 1) with scale, shift and zero points
    xr = np.ascontiguousarray(x.transpose(0, 2, 1).reshape(N * L, K))
    alpha = _t(rng.uniform(0.5, 2.0, O).astype(np.float32), dev)
    beta = _t(rng.uniform(-1, 1, O).astype(np.float32), dev)
    zx = _t(np.array([91.0], dtype=np.float32), dev)
    zw = _t(rng.integers(0, 256, O).astype(np.float32), dev)
    wsum = _t(w.astype(np.int64).sum(axis=1).astype(np.int32), dev)
    ya = torch.empty((N * L, O), dtype=torch.float32, device=dev)
    yb = torch.empty_like(ya)
    kw = dict(alpha=alpha, beta=beta, zero_x=zx, zero_w=zw, wsum=wsum)
    ops.lut_gemm_launch(_t(xr, dev), _t(w, dev), img, ya, N * L, K, 1, O, **kw)
    ops.FP32_TABLE_ON_CHIP = False
    try:
        ops.lut_gemm_launch(_t(xr, dev), _t(w, dev), img, yb, N * L, K, 1, O, cfg=1 << 16, **kw)
    finally:
        ops.FP32_TABLE_ON_CHIP = True
    assert torch.equal(ya, yb)
    # image operand: strided, padded conv with the pad value taken from the zero point
    B, C, H, W, Oc = 3, 10, 13, 11, 40
    x8 = rng.integers(0, 256, (B, C, H, W), dtype=np.uint8)
    wi = rng.integers(0, 256, (Oc, C * 9), dtype=np.uint8)
    g4 = ((3, 3), (2, 1), (1, 2), (1, 1))
    ws2 = _t(wi.astype(np.int64).sum(axis=1).astype(np.int32), dev)
    zw2 = _t(rng.integers(0, 256, Oc).astype(np.float32), dev)
    ya = ops.lut_conv2d_launch(_t(x8, dev), _t(wi, dev), img, g4, -1, zero_x=zx, zero_w=zw2, wsum=ws2)
    ops.FP32_TABLE_ON_CHIP = False
    try:
        yb = ops.lut_conv2d_launch(_t(x8, dev), _t(wi, dev), img, g4, -1, zero_x=zx, zero_w=zw2, wsum=ws2, cfg=1 << 16)
    finally:
        ops.FP32_TABLE_ON_CHIP = True
    assert torch.equal(ya, yb)
    cols = lo.im2col_index(x8, 3, 3, 2, 1, 1, 2, 1, 1, 91)
    raw = lo.bgemm_f32_ascending(cols, wi, tab).astype(np.float64)
    t = lo.uint8_zero_point_correction(raw, cols, wi, 91.0, zw2.cpu().numpy())
    np.testing.assert_allclose(ya.flatten(2).cpu().numpy(), t, rtol=1e-6, atol=1e-6 * np.abs(t).max())


def test_lut_image_cache_follows_in_place_updates(dev):
    ops = _ops()
    rng = np.random.default_rng(2)
    x = rng.integers(0, 256, (1, 9, 10), dtype=np.uint8)
    w = rng.integers(0, 256, (3, 9)).astype(np.float32)
    lut = _t(lo.lut_exact_unsigned().reshape(-1), dev)
    y1 = ops.bgemm_fake_uint8_claude(_t(x, dev), _t(w, dev), lut)
    lut.mul_(2.0)                                   # version bump must invalidate the cached image
    y2 = ops.bgemm_fake_uint8_claude(_t(x, dev), _t(w, dev), lut)
    assert torch.equal(y2, 2.0 * y1)


def test_gemm_operators(dev):
    ops = _ops()
    rng = np.random.default_rng(33)
    M, K, Nc = 70, 45, 130
    A = rng.integers(-128, 128, (M, K)).astype(np.float32)
    B = rng.integers(-128, 128, (K, Nc)).astype(np.float32)
    lut = lo.lut_affine_asymmetric()
    ref = lo.gemm_exact(lo.to_lut_index(A, 128), lo.to_lut_index(B, 128), lut)
    lt = _t(lut.reshape(-1), dev)
    y, aq, bq = ops.gemm_fake_int8_claude_save(_t(A, dev), _t(B, dev), lt)
    np.testing.assert_array_equal(y.cpu().numpy().astype(np.int64), ref)
    assert tuple(aq.shape) == (M, K) and tuple(bq.shape) == (Nc, K)      # bq is transposed
    np.testing.assert_array_equal(bq.cpu().numpy(), lo.to_lut_index(B, 128).T)
    # transposed-view B costs nothing extra and gives the same numbers
    Wt = _t(np.ascontiguousarray(B.T), dev)
    assert torch.equal(ops.gemm_fake_int8_claude(_t(A, dev), Wt.t(), lt), y)
    # orientation matters: A and B swapped through an asymmetric table differ
    yu = ops.gemm_fake_uint8_claude(_t(lo.to_lut_index(A, 128), dev), _t(lo.to_lut_index(B, 128), dev), lt)
    assert torch.equal(yu, y)
    # degenerate shapes
    assert ops.gemm_fake_int8_claude(torch.zeros(0, K, device=dev), _t(B, dev), lt).shape == (0, Nc)
    assert ops.gemm_fake_int8_claude(_t(A, dev), torch.zeros(K, 0, device=dev), lt).shape == (M, 0)
    z = ops.gemm_fake_int8_claude(torch.zeros(M, 0, device=dev), torch.zeros(0, Nc, device=dev), lt)
    assert z.shape == (M, Nc) and not z.any()
    with pytest.raises(RuntimeError):
        ops.gemm_fake_int8_claude(_t(A, dev), _t(B[:-1], dev), lt)
    with pytest.raises(RuntimeError):
        ops.gemm_fake_int8_claude(_t(A, dev), _t(B, dev), lt[:100])
    with pytest.raises(RuntimeError):
        ops.bgemm_fake_int8_claude(_t(A, dev), _t(B, dev), lt)              # wrong rank


def test_per_batch_weights_match_oracle(dev):
    """The benchmark's raw LUT-BGEMM shape family: one weight matrix per batch item, A k-contiguous."""
    ops = _ops()
    rng = np.random.default_rng(44)
    Bt, M, K, Nc = 3, 640, 96, 128
    A = rng.integers(0, 256, (Bt, M, K), dtype=np.uint8)
    Bm = rng.integers(0, 256, (Bt, Nc, K), dtype=np.uint8)                   # already [N,K] per batch
    lut = lo.lut_signed_noisy(64, seed=0)
    y = torch.empty((Bt, M, Nc), dtype=torch.float32, device=dev)
    ops.lut_gemm_launch(_t(A, dev), _t(Bm, dev), ops.lut_image(_t(lut.reshape(-1), dev)), y,
                        Bt * M, K, 1, Nc, wb_rows=M, w_batch_stride=Nc * K)
    for b in range(Bt):
        ref = lo.gemm_exact(A[b], Bm[b].T, lut)
        np.testing.assert_array_equal(y[b].cpu().numpy().astype(np.int64), ref)


def test_benchmark_size_rows_against_oracle(dev):
    """Full benchmark size (16 x [4096 x 576] . [576 x 256]): a random sample of output rows is checked
    bit-exactly against the C oracle, and the whole output against a column checksum identity:
    sum over rows of y[:, o] equals sum_k sum_a count_k[a] * lut[a][w[o,k]]."""
    ops = _ops()
    rng = np.random.default_rng(0)
    Bt, M, K, Nc = 16, 4096, 576, 256
    A = rng.integers(0, 256, (Bt, M, K), dtype=np.uint8)
    Bm = rng.integers(0, 256, (Bt, Nc, K), dtype=np.uint8)
    lut = lo.lut_signed_noisy(64, seed=0)
    y = torch.empty((Bt, M, Nc), dtype=torch.float32, device=dev)
    ops.lut_gemm_launch(_t(A, dev), _t(Bm, dev), ops.lut_image(_t(lut.reshape(-1), dev)), y,
                        Bt * M, K, 1, Nc, wb_rows=M, w_batch_stride=Nc * K)
    yh = y.cpu().numpy().astype(np.int64)
    rows = rng.integers(0, M, 24)
    for b in (0, 7, 13, 15):
        ref = lo.gemm_exact(A[b][rows], Bm[b].T, lut)
        np.testing.assert_array_equal(yh[b][rows], ref)
    tab = lut.reshape(256, 256).astype(np.int64)
    for b in (3, 12, 13, 15):
        counts = np.stack([np.bincount(A[b][:, k], minlength=256) for k in range(K)])      # [K, 256]
        expect = np.array([(counts * tab[:, Bm[b][o]].T).sum() for o in range(Nc)])
        np.testing.assert_array_equal(yh[b].sum(axis=0), expect)


def _plan(ops, R, K, O, wb_rows=0, cfg=-1):
    import ctypes
    from approxtorch_b200.backend import _C
    plan = _C.GemmPlan()
    assert _C.lib.atb_lut_gemm_plan(R, K, O, wb_rows, cfg, ctypes.byref(plan)) == 0
    return plan


NO_TAIL = 1 << 16            # cfg bits 16-23 = 1: runs of whole tiles only (no tile is cut between blocks)


def test_ragged_last_wave_is_split_along_k_column_operand(dev):
    """More tiles than one wave of blocks, not a multiple of the SM count: the equal runs end inside tiles, which are
    finished by the last block to arrive.  Same integers as the oracle and as the whole-tile plan, with and without
    the zero-point terms."""
    ops = _ops()
    rng = np.random.default_rng(77)
    N, K, L, O = 1, 80, 20000, 256
    plan = _plan(ops, N * L, K, O)
    assert plan.cut_tiles and plan.scratch_bytes > 0
    whole = _plan(ops, N * L, K, O, cfg=NO_TAIL)
    assert not whole.cut_tiles and whole.scratch_bytes == 0 and whole.units_per_block % whole.chunks_per_tile == 0
    x = rng.integers(0, 256, (N, K, L), dtype=np.uint8)
    w = rng.integers(0, 256, (O, K), dtype=np.uint8)
    lut = lo.lut_signed_noisy(64, seed=4)
    ref = c_oracle.bgemm_u8(x, w, lut)
    img = ops.lut_image(_t(lut.reshape(-1), dev))
    y = torch.empty((N, O, L), dtype=torch.float32, device=dev)
    ops.lut_gemm_launch(_t(x, dev), _t(w, dev), img, y, N, K, L, O)
    np.testing.assert_array_equal(y.cpu().numpy().astype(np.float64), ref)
    # asymmetric epilogue: row sums of the tail rows travel through scratch too
    alpha = _t(rng.uniform(0.5, 2.0, O).astype(np.float32), dev)
    beta = _t(rng.uniform(-1, 1, O).astype(np.float32), dev)
    zx = _t(np.array([37.0], dtype=np.float32), dev)
    zw = _t(rng.integers(0, 256, O).astype(np.float32), dev)
    wsum = _t(w.astype(np.int64).sum(axis=1).astype(np.int32), dev)
    ya, yb = torch.empty_like(y), torch.empty_like(y)
    ops.lut_gemm_launch(_t(x, dev), _t(w, dev), img, ya, N, K, L, O, alpha=alpha, beta=beta, zero_x=zx, zero_w=zw, wsum=wsum)
    ops.lut_gemm_launch(_t(x, dev), _t(w, dev), img, yb, N, K, L, O, alpha=alpha, beta=beta, zero_x=zx, zero_w=zw, wsum=wsum,
                        cfg=NO_TAIL)
    assert torch.equal(ya, yb)
    t = (ref - zw.cpu().numpy().astype(np.float64)[None, :, None] * x.astype(np.int64).sum(axis=1)[:, None, :]
         - 37.0 * wsum.cpu().numpy().astype(np.float64)[None, :, None] + K * 37.0 * zw.cpu().numpy().astype(np.float64)[None, :, None])
    expect = (t.astype(np.float32) * alpha.cpu().numpy()[None, :, None]) + beta.cpu().numpy()[None, :, None]
    np.testing.assert_array_equal(ya.cpu().numpy(), expect.astype(np.float32))


def test_ragged_last_wave_per_batch_weights_and_image_operand(dev):
    ops = _ops()
    rng = np.random.default_rng(78)
    lut = lo.lut_affine_asymmetric()
    img = ops.lut_image(_t(lut.reshape(-1), dev))
    # one weight matrix per batch item, batch rows not a multiple of the block rows
    Bt, M, K, Nc = 5, 4600, 96, 256
    assert _plan(ops, Bt * M, K, Nc, wb_rows=M).cut_tiles
    A = rng.integers(0, 256, (Bt, M, K), dtype=np.uint8)
    Bm = rng.integers(0, 256, (Bt, Nc, K), dtype=np.uint8)
    y = torch.empty((Bt, M, Nc), dtype=torch.float32, device=dev)
    ops.lut_gemm_launch(_t(A, dev), _t(Bm, dev), img, y, Bt * M, K, 1, Nc, wb_rows=M, w_batch_stride=Nc * K)
    for b in range(Bt):
        np.testing.assert_array_equal(y[b].cpu().numpy().astype(np.int64), lo.gemm_exact(A[b], Bm[b].T, lut))
    # image operand (im2col in the tile loader)
    B, C, H, W, O = 8, 8, 80, 80, 128
    assert _plan(ops, B * H * W, C * 9, O).cut_tiles
    x8 = rng.integers(-127, 128, (B, C, H, W)).astype(np.int8)
    widx = rng.integers(0, 256, (O, C * 9), dtype=np.uint8)
    cols = lo.im2col_index(lo.index_of(x8, True), 3, 3, 1, 1, 1, 1, 1, 1, 128)
    ref = c_oracle.bgemm_u8(cols, widx, lut)
    g4 = ((3, 3), (1, 1), (1, 1), (1, 1))
    yc = ops.lut_conv2d_launch(_t(x8, dev), _t(widx, dev), img, g4, 128)
    np.testing.assert_array_equal(yc.flatten(2).cpu().numpy().astype(np.float64), ref)
    assert torch.equal(yc, ops.lut_conv2d_launch(_t(x8, dev), _t(widx, dev), img, g4, 128, cfg=NO_TAIL))


STREAM_K = 3 << 16           # cfg bits 16-23 = 3: every tile is cut into three k-segments, one block each


@pytest.mark.parametrize("shape", [(1, 256, 3136, 200), (3, 100, 500, 70), (2, 37, 1300, 64), (1, 600, 70, 130),
                                   (1, 48, 4000, 1), (7, 40, 9, 5)])
def test_stream_k_is_bit_identical(dev, shape):
    """Blocks that work through runs of (tile, k-chunk) units: same integers as the oracle and as whole-tile
    blocks, with the zero-point epilogue, for L > 1 and L == 1 outputs."""
    ops = _ops()
    N, K, L, O = shape
    rng = np.random.default_rng(sum(shape))
    x = rng.integers(0, 256, (N, K, L), dtype=np.uint8)
    w = rng.integers(0, 256, (O, K), dtype=np.uint8)
    lut = lo.lut_signed_noisy(64, seed=6)
    img = ops.lut_image(_t(lut.reshape(-1), dev))
    assert _plan(ops, N * L, K, O, cfg=STREAM_K).cut_tiles == (1 if K > 16 else 0)
    ref = c_oracle.bgemm_u8(x, w, lut)
    y = torch.empty((N, O, L), dtype=torch.float32, device=dev)
    ops.lut_gemm_launch(_t(x, dev), _t(w, dev), img, y, N, K, L, O, cfg=STREAM_K)
    np.testing.assert_array_equal(y.cpu().numpy().astype(np.float64), ref)
    # row-major operand (L == 1) and the asymmetric epilogue
    xr = np.ascontiguousarray(x.transpose(0, 2, 1).reshape(N * L, K))
    alpha = _t(rng.uniform(0.5, 2.0, O).astype(np.float32), dev)
    zx = _t(np.array([91.0], dtype=np.float32), dev)
    zw = _t(rng.integers(0, 256, O).astype(np.float32), dev)
    wsum = _t(w.astype(np.int64).sum(axis=1).astype(np.int32), dev)
    ya = torch.empty((N * L, O), dtype=torch.float32, device=dev)
    yb = torch.empty_like(ya)
    for out, cfg in ((ya, STREAM_K), (yb, NO_TAIL)):
        ops.lut_gemm_launch(_t(xr, dev), _t(w, dev), img, out, N * L, K, 1, O, alpha=alpha, zero_x=zx, zero_w=zw,
                            wsum=wsum, cfg=cfg)
    assert torch.equal(ya, yb)


def test_stream_k_image_operand_and_fp32_table(dev):
    ops = _ops()
    rng = np.random.default_rng(90)
    B, C, H, W, O = 4, 24, 20, 20, 96
    x8 = rng.integers(-127, 128, (B, C, H, W)).astype(np.int8)
    widx = rng.integers(0, 256, (O, C * 9), dtype=np.uint8)
    g4 = ((3, 3), (2, 2), (1, 1), (1, 1))
    for lut in (lo.lut_affine_asymmetric(), lo.lut_signed_noisy(64, seed=1) + 0.25):     # integer table, fp32-class table
        img = ops.lut_image(_t(np.asarray(lut, dtype=np.float32).reshape(-1), dev))
        ya = ops.lut_conv2d_launch(_t(x8, dev), _t(widx, dev), img, g4, 128, cfg=STREAM_K)
        yb = ops.lut_conv2d_launch(_t(x8, dev), _t(widx, dev), img, g4, 128, cfg=NO_TAIL)
        if float(np.asarray(lut).reshape(-1)[0]) == int(np.asarray(lut).reshape(-1)[0]):
            assert torch.equal(ya, yb)
        else:                                   # fp32 sums: the partial sums are added in another order
            assert (ya - yb).abs().max().item() <= 1e-5 * yb.abs().max().item()
