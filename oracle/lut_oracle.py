"""numpy restatement of the reference's LUT-GEMM / fake-quant / gradient semantics.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Every function cites the
reference file:line it restates; paths are relative to the reference project
root (``approxtorch/...``).  Shape letters follow the reference: N batch,
K = C*kh*kw reduction, L = OH*OW output pixels, O output channels.

Index rule (approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:278-281,
approxtorch/backend/csrc/naive_cuda/bgemm_naive.cu:16-58): the activation is
the ROW of the 256x256 table, the weight the COLUMN:
``flat = idx(x) * 256 + idx(w)`` with ``idx_int8(v) = v + 128`` and
``idx_uint8(v) = v``.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------
# operand -> LUT index
# --------------------------------------------------------------------------

def to_lut_index(values, offset: int) -> np.ndarray:
    """fp32 integer-valued operand -> uint8 LUT index.

    ``clamp(__float2int_rn(v) + offset, 0, 255)``: round half to even, NaN -> 0
    before the offset, saturating clamp, never wraps
    (approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:62-67).
    ``offset`` is 128 for signed int8 operands and 0 for unsigned ones.
    """
    v = np.asarray(values, dtype=F32)
    r = np.rint(v.astype(np.float64))
    r = np.where(np.isnan(r), 0.0, r)
    r = np.clip(r, -2147483648.0, 2147483647.0)
    q = r.astype(np.int64) + int(offset)
    return np.clip(q, 0, 255).astype(np.uint8)


def index_of(values, signed: bool) -> np.ndarray:
    """LUT index of an already-quantised tensor by dtype
    (approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:69-80):
    int8 -> v + 128, uint8 -> v, float -> round/clamp to [-128,127] + 128
    (signed) or round/clamp to [0,255] (unsigned forward prepass)."""
    a = np.asarray(values)
    if a.dtype == np.int8:
        return (a.astype(np.int16) + 128).astype(np.uint8)
    if a.dtype == np.uint8:
        return a
    return to_lut_index(a, 128 if signed else 0)


def lut_class(lut) -> str:
    """Which in-kernel table image a LUT is eligible for
    (approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:116-142, 344-359):
    'i16' iff every entry is an integer with |v| <= 32767; else 'u16' iff every
    entry is an integer in [0, 65535]; else 'f32'."""
    t = np.asarray(lut, dtype=F32).reshape(-1)
    assert t.size == 65536
    is_int = t == np.rint(t)
    if bool(np.all(is_int & (np.abs(t) <= 32767.0))):
        return "i16"
    if bool(np.all(is_int & (t >= 0.0) & (t <= 65535.0))):
        return "u16"
    return "f32"


# --------------------------------------------------------------------------
# forward: LUT-BGEMM / GEMM / im2col / conv
# --------------------------------------------------------------------------

def bgemm_exact(xq, wq, lut) -> np.ndarray:
    """y[n,o,l] = sum_k lut[xq[n,k,l]][wq[o,k]] with exact accumulation.

    xq uint8 [N,K,L], wq uint8 [O,K] are LUT indices.  Integer-valued tables
    are summed in int64 (the serial integer sum of
    approxtorch/backend/csrc/naive_cuda/bgemm_naive.cu:50-55 without its int32
    overflow); other tables in float64.  ``wq`` may also be [N,O,K] (one weight
    matrix per batch item)."""
    xq = np.asarray(xq, dtype=np.uint8)
    wq = np.asarray(wq, dtype=np.uint8)
    t = np.asarray(lut, dtype=F32).reshape(256, 256)
    integer = bool(np.all(t == np.rint(t)))
    tab = t.astype(np.int64) if integer else t.astype(np.float64)
    N, K, L = xq.shape
    batched_w = wq.ndim == 3
    O = wq.shape[-2]
    y = np.zeros((N, L, O), dtype=tab.dtype)
    for n in range(N):
        wn = wq[n] if batched_w else wq
        acc = y[n]
        for k in range(K):
            cols = tab[:, wn[:, k]]          # [256, O]: table column per output channel
            acc += cols[xq[n, k, :]]         # [L, O]
    return np.ascontiguousarray(y.transpose(0, 2, 1))


def bgemm_f32_ascending(xq, wq, lut) -> np.ndarray:
    """Same sum accumulated the way the reference kernel does without split-K:
    fp32 adds in ascending k
    (approxtorch/backend/csrc/claude/bgemm_lut_kernels.cuh:278-281, 337-341)."""
    xq = np.asarray(xq, dtype=np.uint8)
    wq = np.asarray(wq, dtype=np.uint8)
    tab = np.asarray(lut, dtype=F32).reshape(256, 256)
    N, K, L = xq.shape
    O = wq.shape[0]
    y = np.zeros((N, L, O), dtype=F32)
    for n in range(N):
        acc = y[n]
        for k in range(K):
            acc += tab[:, wq[:, k]][xq[n, k, :]]
    return np.ascontiguousarray(y.transpose(0, 2, 1))


def gemm_exact(aq, bq_kn, lut) -> np.ndarray:
    """torch.mm layout: y[m,n] = sum_k lut[aq[m,k]][bq[k,n]]
    (approxtorch/backend/csrc/claude/gemm.cu:6-9)."""
    aq = np.asarray(aq, dtype=np.uint8)
    bq = np.asarray(bq_kn, dtype=np.uint8)
    M, K = aq.shape
    x = aq.T.reshape(1, K, M)                      # [1, K, L=M]
    y = bgemm_exact(x, np.ascontiguousarray(bq.T), lut)   # [1, N, M]
    return np.ascontiguousarray(y[0].T)


def conv_out_hw(H, W, kh, kw, sh, sw, ph, pw, dh, dw):
    OH = (H + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    OW = (W + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    return OH, OW


def im2col_index(img_idx, kh, kw, sh=1, sw=1, ph=0, pw=0, dh=1, dw=1, pad_idx=128) -> np.ndarray:
    """uint8 LUT-index unfold [B,C,H,W] -> [B, C*kh*kw, OH*OW]; taps outside the
    image are the index of quantised zero (128 for int8; the activation zero
    point for uint8) and are still looked up, never skipped
    (approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:216-269;
    approxtorch/nn/Conv2d_uint8.py:283-286).  k order is (c, kh, kw) as in
    torch.nn.functional.unfold."""
    a = np.asarray(img_idx, dtype=np.uint8)
    B, C, H, W = a.shape
    OH, OW = conv_out_hw(H, W, kh, kw, sh, sw, ph, pw, dh, dw)
    pad = np.full((B, C, H + 2 * ph, W + 2 * pw), pad_idx, dtype=np.uint8)
    pad[:, :, ph:ph + H, pw:pw + W] = a
    out = np.empty((B, C, kh, kw, OH, OW), dtype=np.uint8)
    for i in range(kh):
        for j in range(kw):
            out[:, :, i, j] = pad[:, :, i * dh:i * dh + (OH - 1) * sh + 1:sh,
                                   j * dw:j * dw + (OW - 1) * sw + 1:sw]
    return out.reshape(B, C * kh * kw, OH * OW)


# --------------------------------------------------------------------------
# fake quantisation, EMA statistics, dequantisation
# --------------------------------------------------------------------------

def fakequant_sym(x, scale, qmin, qmax):
    """(q, mask): s = max(scale, 1e-12); v = x / s (an fp32 DIVISION);
    mask = qmin <= v <= qmax on the pre-round value; q = clamp(rint(v)) with
    round-half-even (approxtorch/backend/csrc/claude/quantization.cu:54-62, 85;
    approxtorch/nn/quantization.py:47-52).  ``scale`` broadcasts (scalar, or a
    per-channel array already shaped for broadcasting)."""
    x = np.asarray(x, dtype=F32)
    s = np.maximum(np.asarray(scale, dtype=F32), F32(1e-12))
    v = (x / s).astype(F32)
    mask = (v >= F32(qmin)) & (v <= F32(qmax))
    q = np.clip(np.rint(v), F32(qmin), F32(qmax)).astype(F32)
    return q, mask


def fakequant_asym(x, scale, zero_point, qmin, qmax):
    """(q, mask) with v = x / s + z (fp32 divide, then fp32 add)
    (approxtorch/backend/csrc/claude/quantization.cu:67-75;
    approxtorch/nn/quantization.py:76-80)."""
    x = np.asarray(x, dtype=F32)
    s = np.maximum(np.asarray(scale, dtype=F32), F32(1e-12))
    v = ((x / s).astype(F32) + np.asarray(zero_point, dtype=F32)).astype(F32)
    mask = (v >= F32(qmin)) & (v <= F32(qmax))
    q = np.clip(np.rint(v), F32(qmin), F32(qmax)).astype(F32)
    return q, mask


def fakequant_bwd(grad_out, mask, scale):
    """gx = (mask ? go : 0) / max(scale, 1e-12)
    (approxtorch/backend/csrc/claude/quantization.cu:113-143)."""
    s = np.maximum(np.asarray(scale, dtype=F32), F32(1e-12))
    g = np.where(mask, np.asarray(grad_out, dtype=F32), F32(0))
    return (g / s).astype(F32)


def ema_scale_x(x_absmax, old_scale, momentum, qmin=-127, qmax=127):
    """scale_x <- m * absmax / ((qmax-qmin)/2) + (1-m) * scale_x in fp32
    (approxtorch/nn/Conv2d_int8.py:137-146)."""
    cur = F32(x_absmax) / F32((qmax - qmin) / 2)
    return F32(F32(momentum) * cur + F32(1 - momentum) * F32(old_scale))


def weight_absmax_scale(w, bits, old=None):
    """per-output-channel absmax / (2^(bits-1)-1); channels that are all zero
    keep ``old`` (or 1 at reset)
    (approxtorch/nn/Conv2d_int8.py:148-167)."""
    w = np.asarray(w, dtype=F32)
    qmax = F32(2 ** (bits - 1) - 1)
    am = np.abs(w).reshape(w.shape[0], -1).max(axis=1)
    fallback = np.ones_like(am) if old is None else np.asarray(old, dtype=F32)
    return np.where(am > 0, (am / qmax).astype(F32), fallback).astype(F32)


def ema(cur, old, momentum):
    """new = m * cur + (1 - m) * old in fp32 (approxtorch/nn/Conv2d_int8.py:145,157)."""
    return (F32(momentum) * np.asarray(cur, dtype=F32)
            + F32(1 - momentum) * np.asarray(old, dtype=F32)).astype(F32)


def uint8_qparams(mn, mx, qmax=255):
    """(scale, zero_point) from min/max statistics, range forced to contain 0
    (approxtorch/nn/Conv2d_uint8.py:11-23)."""
    mn = np.minimum(np.asarray(mn, dtype=F32), F32(0))
    mx = np.maximum(np.asarray(mx, dtype=F32), F32(0))
    scale = np.maximum(((mx - mn) / F32(qmax)).astype(F32), F32(1e-12))
    zero = np.clip(np.rint((-mn / scale).astype(F32)), F32(0), F32(qmax)).astype(F32)
    return scale, zero


def dequant(y_int, scale_x, scale_w, bias=None):
    """y = bias[o] + y_int * (scale_x * scale_w[o]); the product of the two
    scales is formed first in fp32 (approxtorch/nn/Conv2d_int8.py:213-218).
    y_int is [B, O, ...]."""
    y_int = np.asarray(y_int)
    s = (F32(scale_x) * np.asarray(scale_w, dtype=F32)).astype(F32)
    shape = (1, -1) + (1,) * (y_int.ndim - 2)
    out = y_int.astype(F32) * s.reshape(shape)
    if bias is not None:
        out = out + np.asarray(bias, dtype=F32).reshape(shape)
    return out.astype(F32)


def uint8_zero_point_correction(lutsum, xq, wq, zero_x, zero_w):
    """sum_k (qx - zx)(qw - zw[o]) = LUTSUM - zw[o]*sum_k qx - zx*sum_k qw + K*zx*zw[o]
    evaluated exactly (approxtorch/nn/Conv2d_uint8.py:308-315).  lutsum [N,O,L],
    xq uint8 [N,K,L], wq uint8 [O,K]; returns float64 [N,O,L]."""
    K = xq.shape[1]
    xs = np.asarray(xq, dtype=np.float64).sum(axis=1)[:, None, :]
    ws = np.asarray(wq, dtype=np.float64).sum(axis=1)[None, :, None]
    zw = np.asarray(zero_w, dtype=np.float64).reshape(1, -1, 1)
    zx = float(zero_x)
    return np.asarray(lutsum, dtype=np.float64) - zw * xs - zx * ws + K * zx * zw


# --------------------------------------------------------------------------
# backward: STE / LRE / custom pair
# --------------------------------------------------------------------------

def lre_backward(go, xq, wq_ok, dx, dw):
    """grad_x[n,k,l] = sum_o go[n,o,l] * dx[wq[o,k]];
    grad_w[o,k] = sum_{n,l} go[n,o,l] * dw[xq[n,k,l]]  (float64)
    (approxtorch/backend/csrc/naive_cuda/bgeem_lre_navie.cu:25-88).  xq, wq are
    LUT indices; dx is indexed by the WEIGHT, dw by the ACTIVATION."""
    go = np.asarray(go, dtype=np.float64)
    wp = np.asarray(dx, dtype=np.float64)[np.asarray(wq_ok, dtype=np.uint8)]   # [O,K]
    xp = np.asarray(dw, dtype=np.float64)[np.asarray(xq, dtype=np.uint8)]      # [N,K,L]
    gx = np.einsum("nol,ok->nkl", go, wp)
    gw = np.einsum("nol,nkl->ok", go, xp)
    return gx, gw


def ste_backward(go, xq, wq_ok, offset=128):
    """STE treats the multiplier as exact: the LRE formulas with the decode
    table dx = dw = arange(256) - offset
    (approxtorch/nn/bgemm_int8.py:19-20, 220-226)."""
    dec = np.arange(256, dtype=np.float64) - offset
    return lre_backward(go, xq, wq_ok, dec, dec)


def custom_backward(go, xq, wq_ok, dx_lut, dw_lut):
    """grad_x[n,k,l] = sum_o go * DX[xq][wq[o,k]]; grad_w[o,k] = sum_{n,l} go *
    DW[xq[n,k,l]][wq]  (float64)
    (approxtorch/backend/csrc/naive_cuda/bgemm_custom_grad_naive.cu:25-92)."""
    go = np.asarray(go, dtype=np.float64)
    xq = np.asarray(xq, dtype=np.uint8)
    wq = np.asarray(wq_ok, dtype=np.uint8)
    DX = np.asarray(dx_lut, dtype=np.float64).reshape(256, 256)
    DW = np.asarray(dw_lut, dtype=np.float64).reshape(256, 256)
    N, K, L = xq.shape
    O = wq.shape[0]
    gx = np.zeros((N, K, L))
    gw = np.zeros((O, K))
    for k in range(K):
        colsx = DX[:, wq[:, k]]                     # [256, O]
        colsw = DW[:, wq[:, k]]
        for n in range(N):
            gx[n, k, :] = np.einsum("lo,ol->l", colsx[xq[n, k, :]], go[n])
            gw[:, k] += np.einsum("lo,ol->o", colsw[xq[n, k, :]], go[n])
    return gx, gw


def fold(cols, C, H, W, kh, kw, sh=1, sw=1, ph=0, pw=0, dh=1, dw=1):
    """Adjoint of unfold: [B, C*kh*kw, L] -> [B, C, H, W] (float64), what
    torch.nn.functional.fold computes (approxtorch/nn/bgemm_int8.py:116-118)."""
    cols = np.asarray(cols, dtype=np.float64)
    B = cols.shape[0]
    OH, OW = conv_out_hw(H, W, kh, kw, sh, sw, ph, pw, dh, dw)
    c6 = cols.reshape(B, C, kh, kw, OH, OW)
    img = np.zeros((B, C, H + 2 * ph, W + 2 * pw))
    for i in range(kh):
        for j in range(kw):
            img[:, :, i * dh:i * dh + (OH - 1) * sh + 1:sh,
                j * dw:j * dw + (OW - 1) * sw + 1:sw] += c6[:, :, i, j]
    return img[:, :, ph:ph + H, pw:pw + W]


def lut_map(values, table256, signed=True):
    """out = table[idx(values)] for a 256-entry table
    (approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:96-130)."""
    return np.asarray(table256, dtype=F32)[index_of(values, signed)]


def lut_map_pad(img, table256, ph, pw, signed=True):
    """Mapped image with a constant border table[128]
    (approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu:277-311)."""
    t = np.asarray(table256, dtype=F32)
    m = t[index_of(img, signed)]
    B, C, H, W = m.shape
    out = np.full((B, C, H + 2 * ph, W + 2 * pw), t[128], dtype=F32)
    out[:, :, ph:ph + H, pw:pw + W] = m
    return out


def lre_slopes(lut):
    """(dx, dw) of the signed table: dx[w+128] = least-squares slope of column
    lut[:, w+128] against x in [-128,127]; dw[x+128] = slope of row lut[x+128,:]
    against w (approxtorch/grad_lut.py:14-37; scipy.stats.linregress' slope is
    the ordinary least-squares cov/var)."""
    t = np.asarray(lut, dtype=np.float64).reshape(256, 256)
    a = np.arange(-128, 128, dtype=np.float64)
    ac = a - a.mean()
    den = (ac * ac).sum()
    dx = (ac[:, None] * (t - t.mean(axis=0, keepdims=True))).sum(axis=0) / den
    dw = ((t - t.mean(axis=1, keepdims=True)) * ac[None, :]).sum(axis=1) / den
    return dx.astype(F32), dw.astype(F32)


# --------------------------------------------------------------------------
# tables used by the benchmark configurations and the tests
# --------------------------------------------------------------------------

def lut_exact_signed():
    a = np.arange(-128, 128, dtype=np.int64)
    return (a[:, None] * a[None, :]).astype(F32)


def lut_exact_unsigned():
    a = np.arange(256, dtype=np.int64)
    return (a[:, None] * a[None, :]).astype(F32)


def lut_signed_truncated(low_bits=4):
    """sign(p) * (|p| with its low bits cleared), p = (i-128)(j-128)."""
    p = lut_exact_signed().astype(np.int64)
    m = np.abs(p) & ~((1 << low_bits) - 1)
    return (np.sign(p) * m).astype(F32)


def lut_unsigned_truncated(low_bits=6):
    p = lut_exact_unsigned().astype(np.int64)
    return (p & ~((1 << low_bits) - 1)).astype(F32)


def lut_signed_noisy(amplitude=64, seed=0):
    """exact signed product + seeded uniform integer noise in [-a, a], clamped
    to the int16 range."""
    rng = np.random.default_rng(seed)
    p = lut_exact_signed().astype(np.int64)
    p = p + rng.integers(-amplitude, amplitude + 1, size=p.shape)
    return np.clip(p, -32768, 32767).astype(F32)


def lut_affine_asymmetric():
    """37*row - 19*col + 11: any operand swap changes the result
    (approxtorch/backend/csrc/naive_cuda/test_naive_lut_ops.py:57-59)."""
    r = np.arange(256, dtype=np.int64)
    return (37 * r[:, None] - 19 * r[None, :] + 11).astype(F32)
