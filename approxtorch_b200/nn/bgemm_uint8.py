"""Unsigned (uint8 x uint8) LUT-BGEMM autograd Functions, same names and argument lists as
approxtorch/nn/bgemm_uint8.py:27-127.

    y[n, o, l] = sum_k lut[x[n,k,l] * 256 + w[o,k]]        x [N,K,L], w [O,K] raw values in [0,255]

The output is the raw LUT sum; the zero-point cross terms of asymmetric quantisation are added by the
caller (the layer) with differentiable torch ops, so these backwards only provide the surrogate
derivative of the raw product.  All three backwards keep the uint8 index images the forward kernel
produced (the reference's STE variant keeps both operands in fp32, approxtorch/nn/bgemm_uint8.py:30-46).
"""

from __future__ import annotations

from torch.autograd import Function

from ..backend import ops as _ops

__all__ = ["bgemm_uint8", "bgemm_uint8_ste", "bgemm_uint8_lre", "bgemm_uint8_custom"]


class _bgemm_uint8_ste(Function):
    # d/dq_x = q_w and d/dq_w = q_x: the slope-table kernels with the identity decode table.

    @staticmethod
    def forward(ctx, x, w, lut):
        y, xq, wq = _ops.bgemm_fake_uint8_claude_save(x, w, lut)
        ctx.save_for_backward(xq, wq)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        xq, wq = ctx.saved_tensors
        dec = _ops.decode_table(xq.device, 0)
        gx, gw = _ops.lre_backward_launch(grad_output.contiguous(), xq, wq, True, dec, dec,
                                          ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return gx, gw, None


def bgemm_uint8_ste(x, w, lut):
    return _bgemm_uint8_ste.apply(x, w, lut)


class _bgemm_uint8_lre(Function):
    """``dx`` (indexed by the raw weight value) and ``dw`` (indexed by the raw activation value) hold
    256 fp32 slopes each."""

    @staticmethod
    def forward(ctx, x, w, lut, dx, dw):
        y, xq, wq = _ops.bgemm_fake_uint8_claude_save(x, w, lut)
        ctx.save_for_backward(xq, wq, dx, dw)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        xq, wq, dx, dw = ctx.saved_tensors
        gx, gw = _ops.lre_backward_launch(grad_output.contiguous(), xq, wq, True,
                                          dx.contiguous(), dw.contiguous(),
                                          ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return gx, gw, None, None, None


def bgemm_uint8_lre(x, w, lut, dx, dw):
    return _bgemm_uint8_lre.apply(x, w, lut, dx, dw)


class _bgemm_uint8_custom(Function):
    """Pair-wise derivative tables: 256 x 256 fp32 each, entry [x, w]."""

    @staticmethod
    def forward(ctx, x, w, lut, dx_lut, dw_lut):
        y, xq, wq = _ops.bgemm_fake_uint8_claude_save(x, w, lut)
        ctx.save_for_backward(xq, wq, dx_lut, dw_lut)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        xq, wq, dx_lut, dw_lut = ctx.saved_tensors
        gx = _ops.bgemm_custom_grad_uint8_dx(xq, wq, grad_output, dx_lut) if ctx.needs_input_grad[0] else None
        gw = _ops.bgemm_custom_grad_uint8_dw(xq, wq, grad_output, dw_lut) if ctx.needs_input_grad[1] else None
        return gx, gw, None, None, None


def bgemm_uint8_custom(x, w, lut, dx_lut, dw_lut):
    return _bgemm_uint8_custom.apply(x, w, lut, dx_lut, dw_lut)


class _bgemm_uint8(Function):
    # forward only: a backward through it is a usage error, not a silent wrong gradient

    @staticmethod
    def forward(ctx, x, w, lut):
        return _ops.bgemm_fake_uint8_claude(x, w, lut)

    @staticmethod
    def backward(ctx, grad_output):
        raise NotImplementedError(
            "bgemm_uint8 is forward-only; use bgemm_uint8_ste, bgemm_uint8_lre or bgemm_uint8_custom for training")


def bgemm_uint8(x, w, lut):
    return _bgemm_uint8.apply(x, w, lut)
