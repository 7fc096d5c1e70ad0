"""Gradient-table generators with the reference's entry points (approxtorch/grad_lut.py:14-142).

``lre``  : per-column / per-row ordinary-least-squares slopes of a signed 256 x 256 table.
``DATE`` : moving-average smoothing followed by a central difference (pair-wise 256 x 256 tables).
Host-side numpy; these run once per multiplier, not per step.
"""

from __future__ import annotations

import numpy as np


def load_txt_lut(file_path):
    return np.loadtxt(file_path, dtype=np.float32).reshape(256, 256)


def fit_linear(x, y):
    """Least-squares slope of y against x (what scipy.stats.linregress reports as ``slope``)."""
    x = np.asarray(x, dtype=np.float64)
    y = np.asarray(y, dtype=np.float64)
    xc = x - x.mean()
    return float((xc * (y - y.mean())).sum() / (xc * xc).sum())


def lre(multiplier, qtype, save_path):
    """(grad_a, grad_b): grad_a[w + 128] is the slope of column ``lut[:, w + 128]`` against the first
    operand (the table ``dx``, indexed by the weight); grad_b[x + 128] the slope of row
    ``lut[x + 128, :]`` against the second operand (``dw``, indexed by the activation).  Only
    ``qtype='int8'`` is defined.  With ``save_path`` the tables are also written with 4 decimals."""
    lut = load_txt_lut(multiplier) if not isinstance(multiplier, np.ndarray) else multiplier.reshape(256, 256)
    if qtype != 'int8':
        return None
    axis = np.arange(-128, 128, dtype=np.float64)
    centred = axis - axis.mean()
    denom = (centred * centred).sum()
    t = lut.astype(np.float64)
    grad_a = ((centred[:, None] * (t - t.mean(axis=0, keepdims=True))).sum(axis=0) / denom).astype(np.float32)
    grad_b = (((t - t.mean(axis=1, keepdims=True)) * centred[None, :]).sum(axis=1) / denom).astype(np.float32)
    if save_path is not None:
        np.savetxt(f'{save_path}_lre_grad_a.txt', grad_a, fmt='%.4f')
        np.savetxt(f'{save_path}_lre_grad_b.txt', grad_b, fmt='%.4f')
    return grad_a, grad_b


def _moving_average(lut, half_ws, axis):
    """Centred window mean along ``axis`` where the full window fits, the raw value elsewhere."""
    t = np.moveaxis(lut.astype(np.float32), axis, -1)
    out = t.copy()
    n = t.shape[-1]
    for i in range(half_ws, n - half_ws):
        out[..., i] = t[..., i - half_ws:i + half_ws + 1].mean(axis=-1)
    return np.moveaxis(out, -1, axis)


def _difference(smooth, half_ws, axis):
    """Central difference of the smoothed table strictly inside (half_ws, 255 - half_ws); the end-to-end
    secant slope of the same line elsewhere."""
    s = np.moveaxis(smooth.astype(np.float32), axis, -1)
    n = s.shape[-1]
    grad = np.empty_like(s)
    grad[...] = ((s[..., -1] - s[..., 0]) / np.float32(255.0))[..., None]
    lo, hi = half_ws + 1, n - 1 - half_ws          # indices with half_ws < i < 255 - half_ws
    if hi > lo:
        grad[..., lo:hi] = (s[..., lo + 1:hi + 1] - s[..., lo - 1:hi - 1]) / np.float32(2.0)
    return np.moveaxis(grad, -1, axis)


def DATE(multiplier, half_ws=32, save_path=None):
    """Smoothing + difference gradients: returns (grad_a, grad_b), both (256, 256) float32, the
    derivative along the first (row) and second (column) operand."""
    lut = multiplier.astype(np.float32) if isinstance(multiplier, np.ndarray) \
        else np.loadtxt(multiplier).astype(np.float32)
    assert lut.shape == (256, 256), f"Expected (256, 256), got {lut.shape}"
    grad_a = _difference(_moving_average(lut, half_ws, 0), half_ws, 0)
    grad_b = _difference(_moving_average(lut, half_ws, 1), half_ws, 1)
    if save_path is not None:
        np.savetxt(f'{save_path}_date_{half_ws}_grad_a.txt', grad_a)
        np.savetxt(f'{save_path}_date_{half_ws}_grad_b.txt', grad_b)
    return grad_a, grad_b
