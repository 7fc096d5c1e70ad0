"""Unsigned (uint8 x uint8) LUT-BGEMM autograd Functions, same names and argument lists as
approxtorch/nn/bgemm_uint8.py:27-127.

    y[n, o, l] = sum_k lut[x[n,k,l] * 256 + w[o,k]]        x [N,K,L], w [O,K] raw values in [0,255]

The output is the raw LUT sum; the zero-point cross terms of asymmetric quantisation are added by the
caller (the layer) with differentiable torch ops, so these backwards only provide the surrogate
derivative of the raw product.  All three backwards keep the uint8 index images the forward kernel
produced (the reference's STE variant keeps both operands in fp32, approxtorch/nn/bgemm_uint8.py:30-46).
"""

from __future__ import annotations

import torch
from torch.autograd import Function

from ..backend import ops as _ops

__all__ = ["bgemm_uint8", "bgemm_uint8_ste", "bgemm_uint8_lre", "bgemm_uint8_custom", "approx_conv2d_uint8"]


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


# ----------------------------------------------------------------------------- fused layer path
class _approx_conv2d_uint8(Function):
    """Whole unsigned layer without the unfolded fp32 operand: fake-quant of the activation to a uint8 index
    image (+ mask), per-channel asymmetric weight fake-quant to uint8 indices (+ mask, + index sums), im2col-free
    LUT conv whose epilogue applies the zero-point correction in integer arithmetic, the scale and the bias.

    The same function as the chain of approxtorch/nn/Conv2d_uint8.py:257-325 (static_quantize_uint8 -> pad with
    z_x -> unfold -> bgemm_uint8_{ste,lre} -> differentiable correction -> addcmul).  Its gradients, with
    s[o] = scale_x * scale_w[o] and T_x, T_w the slope tables (identity for STE):

        d out / d q_x[n,k,l] = sum_o go[n,o,l] * s[o] * (T_x[q_w[o,k]] - z_w[o])
        d out / d q_w[o,k]   = sum_{n,l} go[n,o,l] * s[o] * (T_w[q_x[n,k,l]] - z_x)

    where the -z terms are what autograd derives from the correction in the reference's chain.  Padded taps
    carry q_x = z_x, so they contribute T_w[z_x] - z_x to grad_w (zero for STE).  ``mode`` is 'ste' or 'lre';
    scales and zero points are buffers and get no gradient."""

    @staticmethod
    def forward(ctx, x, weight, bias, scale_x, zero_x, scale_w, zero_w, lut, dx, dw, g4, mode, qmin, qmax):
        need_gx, need_gw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        xq8, xmask = _ops.quantize_image(x.detach(), scale_x, zero_x, qmin, qmax, want_mask=need_gx)
        widx, wmask, _, wsum = _ops.quantize_weight(weight.detach(), scale_w, zero_w, qmin, qmax, 0,
                                                    want_mask=need_gw, want_sum=True)
        alpha = (scale_x * scale_w).contiguous()
        beta = None if bias is None else bias.detach().contiguous()
        zw = zero_w.contiguous()
        if need_gx or need_gw:
            # private copies: the module rewrites these buffers in place on its next training forward
            scale_x, zero_x, scale_w, zw = scale_x.clone(), zero_x.clone(), scale_w.clone(), zw.clone()
        y = _ops.lut_conv2d_launch(xq8, widx, _ops.lut_image(lut), g4, -1, alpha=alpha, beta=beta,
                                   zero_x=zero_x, zero_w=zw, wsum=wsum)
        if need_gx or need_gw or (bias is not None and ctx.needs_input_grad[2]):
            keep = [xq8, widx, alpha, scale_x, zero_x, scale_w, zw]
            keep += [t for t in (xmask, wmask) if t is not None]
            if mode == 'lre':
                keep += [dx, dw]
            ctx.save_for_backward(*keep)
            ctx.have = (xmask is not None, wmask is not None)
            ctx.g4, ctx.mode, ctx.wshape = g4, mode, tuple(weight.shape)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        saved = list(ctx.saved_tensors)
        xq8, widx, alpha, scale_x, zero_x, scale_w, zw = saved[:7]
        rest = saved[7:]
        xmask = rest.pop(0) if ctx.have[0] else None
        wmask = rest.pop(0) if ctx.have[1] else None
        if ctx.mode == 'lre':
            t_x, t_w = rest[0].contiguous().float().view(-1), rest[1].contiguous().float().view(-1)
        else:
            t_x = t_w = _ops.decode_table(xq8.device, 0)
        # grad_w table: T_w[q] - z_x, with the padded taps' value T_w[z_x] - z_x appended as entry 256
        zx = zero_x.reshape(1)
        pad = t_w.gather(0, zx.round().clamp(0, 255).long())
        t_w_ext = torch.cat([t_w, pad]) - zx
        go = grad_output.contiguous()
        need_gx, need_gw, need_gb = ctx.needs_input_grad[:3]
        gx = gw = gb = None
        if need_gx or need_gw:
            gx, gwq = _ops.lre_conv_backward(go, xq8, widx, t_x, t_w_ext, ctx.g4, 256, go_scale=alpha,
                                             need_x=need_gx, need_w=need_gw, w_zero=zw, exact_tables=ctx.mode != 'lre',
                                             x_mask=xmask if need_gx else None, x_scale=scale_x if need_gx else None)
            if need_gw:
                s = torch.clamp(scale_w, min=1e-12).view(-1, 1, 1, 1)
                gw = gwq.view(ctx.wshape) * wmask.to(gwq.dtype) / s
        if need_gb:
            gb = go.sum(dim=(0, 2, 3))
        return gx, gw, gb, None, None, None, None, None, None, None, None, None, None, None


def approx_conv2d_uint8(x, weight, bias, scale_x, zero_x, scale_w, zero_w, lut, dx, dw, g4, mode, qmin=0, qmax=255):
    return _approx_conv2d_uint8.apply(x, weight, bias, scale_x, zero_x, scale_w, zero_w, lut, dx, dw, g4, mode,
                                      qmin, qmax)

