"""Signed (int8) LUT-GEMM autograd Functions with the reference's names and argument lists
(approxtorch/nn/bgemm_int8.py:5-298).

GEMM level (``x`` already unfolded, [N,K,L]): ``bgemm_int8_ste / _lre / _custom``.
Conv level (``x`` the fake-quantised image, [B,C,H,W]): ``conv2d_int8_ste / _lre / _custom`` take
``geom = (kernel_size, stride, padding, dilation, groups)`` and return y [B,O,L].

What differs from the reference is only what runs underneath:
* the conv forward gathers the taps inside the LUT kernel's tile loader, so no [B,K,L] index matrix
  is written (the reference calls im2col_u8 first, approxtorch/nn/bgemm_int8.py:246-249);
* the STE / LRE conv backward is one fused fp32 kernel pair of this package (table map, gather and
  fold inside the operand fetch) instead of lut_map + lut_map_pad + two cuDNN calls
  (approxtorch/nn/bgemm_int8.py:165-212, 259-295); the depthwise case has per-channel kernels of its own;
* every backward keeps 1-byte payloads (int8 image / uint8 indices).
"""

from __future__ import annotations

import torch
from torch.autograd import Function

from ..backend import ops as _ops

_PAD_INDEX = 128        # quantised zero of the signed path


def _geom4(geom):
    kernel_size, stride, padding, dilation, groups = geom
    return (tuple(kernel_size), tuple(stride), tuple(padding), tuple(dilation)), groups


def _out_hw(shape, g4):
    (kh, kw), (sh, sw), (ph, pw), (dh, dw) = g4
    return _ops.conv_out_hw(shape[2], shape[3], kh, kw, sh, sw, ph, pw, dh, dw)


# ----------------------------------------------------------------------------- GEMM level
class _bgemm_int8_base(Function):

    @staticmethod
    def forward(ctx, x, w, lut):
        y, xq, wq = _ops.bgemm_fake_int8_claude_save(x, w, lut)
        ctx.save_for_backward(xq, wq)
        return y


class _bgemm_int8_ste(_bgemm_int8_base):
    # STE treats the multiplier as exact: grad_x = W^T go, grad_w = go X^T on the quantised values,
    # i.e. the LRE kernels with the decode table idx - 128 (operands are integer-valued, so the saved
    # indices carry them losslessly).

    @staticmethod
    def backward(ctx, grad_output):
        xq, wq = ctx.saved_tensors
        dec = _ops.decode_table(xq.device, 128)
        gx, gw = _ops.lre_backward_launch(grad_output.contiguous(), xq, wq, True, dec, dec,
                                          ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return gx, gw, None


def bgemm_int8_ste(x, w, lut):
    return _bgemm_int8_ste.apply(x, w, lut)


class _bgemm_int8_lre(Function):

    @staticmethod
    def forward(ctx, x, w, lut, dx, dw):
        y, xq, wq = _ops.bgemm_fake_int8_claude_save(x, w, lut)
        ctx.save_for_backward(xq, wq, dx, dw)
        return y

    @staticmethod
    def backward(ctx, grad_outputs):
        xq, wq, dx, dw = ctx.saved_tensors
        gx, gw = _ops.lre_backward_launch(grad_outputs.contiguous(), xq, wq, True,
                                          dx.contiguous(), dw.contiguous(),
                                          ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return gx, gw, None, None, None


def bgemm_int8_lre(x, w, lut, dx, dw):
    return _bgemm_int8_lre.apply(x, w, lut, dx, dw)


class _bgemm_int8_custom(Function):
    """One surrogate derivative per quantised (x, w) pair: ``dx_lut`` / ``dw_lut`` hold 256 x 256
    entries, row-major, entry [x + 128, w + 128]."""

    @staticmethod
    def forward(ctx, x, w, lut, dx_lut, dw_lut):
        y, xq, wq = _ops.bgemm_fake_int8_claude_save(x, w, lut)
        ctx.save_for_backward(xq, wq, dx_lut, dw_lut)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        xq, wq, dx_lut, dw_lut = ctx.saved_tensors
        gx = _ops.bgemm_custom_grad_uint8_dx(xq, wq, grad_output, dx_lut) if ctx.needs_input_grad[0] else None
        gw = _ops.bgemm_custom_grad_uint8_dw(xq, wq, grad_output, dw_lut) if ctx.needs_input_grad[1] else None
        return gx, gw, None, None, None


def bgemm_int8_custom(x, w, lut, dx_lut, dw_lut):
    return _bgemm_int8_custom.apply(x, w, lut, dx_lut, dw_lut)


# ----------------------------------------------------------------------------- conv level
def _conv_forward(x, w, lut, g4, groups):
    """(y [B,O,L], xq8 int8 image, wq uint8 [O,K]) for a fake-quantised fp32 image x."""
    xq8 = x.detach().to(torch.int8)
    if groups == 1:
        wq = _ops.quantize_u8(w.detach(), 128)
        y = _ops.lut_conv2d_launch(xq8, wq, _ops.lut_image(lut), g4, _PAD_INDEX)
    else:
        (kh, kw), stride, padding, dilation = g4
        y, wq = _ops.dwconv_fake_int8_claude(xq8, w.detach(), lut, (kh, kw), stride, padding, dilation)
    return y.flatten(2), xq8, wq


class _conv2d_int8_ste(Function):

    @staticmethod
    def forward(ctx, x, w, lut, geom):
        g4, groups = _geom4(geom)
        y, xq8, wq = _conv_forward(x, w, lut, g4, groups)
        ctx.save_for_backward(xq8, wq)
        ctx.geom = (g4, groups)
        return y

    @staticmethod
    def backward(ctx, grad_outputs):
        xq8, wq = ctx.saved_tensors
        g4, groups = ctx.geom
        B, C, H, W = xq8.shape
        O = wq.shape[0]
        OH, OW = _out_hw(xq8.shape, g4)
        go = grad_outputs.reshape(B, O, OH, OW).contiguous()
        if groups == 1:
            dec = _ops.decode_table(xq8.device, 128)     # dec[128] == 0: padded taps add nothing
            gx, gw = _ops.lre_conv_backward(go, xq8, wq, dec, dec, g4, _PAD_INDEX, exact_tables=True,
                                            need_x=ctx.needs_input_grad[0], need_w=ctx.needs_input_grad[1])
            return gx, gw, None, None
        dec = _ops.decode_table(xq8.device, 128)         # depthwise: per-channel gather / reduction kernels
        gx, gw = _ops.dwconv_backward(go, xq8, wq, dec, dec, g4, _PAD_INDEX,
                                      need_x=ctx.needs_input_grad[0], need_w=ctx.needs_input_grad[1])
        return gx, gw, None, None


def conv2d_int8_ste(x, w, lut, geom):
    return _conv2d_int8_ste.apply(x, w, lut, geom)


class _conv2d_int8_lre(Function):

    @staticmethod
    def forward(ctx, x, w, lut, dx, dw, geom):
        g4, groups = _geom4(geom)
        y, xq8, wq = _conv_forward(x, w, lut, g4, groups)
        ctx.save_for_backward(xq8, wq, dx, dw)
        ctx.geom = (g4, groups)
        return y

    @staticmethod
    def backward(ctx, grad_outputs):
        xq8, wq, dx, dw = ctx.saved_tensors
        g4, groups = ctx.geom
        B, C, H, W = xq8.shape
        O = wq.shape[0]
        OH, OW = _out_hw(xq8.shape, g4)
        go = grad_outputs.reshape(B, O, OH, OW).contiguous()
        if groups == 1:
            # a tap outside the image is quantised zero, whose slope dw[128] is generally not 0
            gx, gw = _ops.lre_conv_backward(go, xq8, wq, dx.contiguous(), dw.contiguous(), g4, _PAD_INDEX,
                                            need_x=ctx.needs_input_grad[0], need_w=ctx.needs_input_grad[1])
            return gx, gw, None, None, None, None
        gx, gw = _ops.dwconv_backward(go, xq8, wq, dx.contiguous(), dw.contiguous(), g4, _PAD_INDEX,
                                      need_x=ctx.needs_input_grad[0], need_w=ctx.needs_input_grad[1])
        return gx, gw, None, None, None, None


def conv2d_int8_lre(x, w, lut, dx, dw, geom):
    return _conv2d_int8_lre.apply(x, w, lut, dx, dw, geom)


class _conv2d_int8_custom(Function):
    """Conv wrapper of the pair-wise custom-gradient kernels (groups == 1 only).  The forward is the im2col-free LUT
    conv; the backward gathers the taps from the saved int8 image and folds the column gradient back into the image
    inside the kernels, so neither the [N,K,L] index matrix nor an [N,K,L] gradient is ever written (the reference
    unfolds with im2col_u8 and folds with F.fold, approxtorch/nn/bgemm_int8.py:87-118)."""

    @staticmethod
    def forward(ctx, x, w, lut, dx_lut, dw_lut, geom):
        g4, groups = _geom4(geom)
        if groups != 1:
            raise NotImplementedError("custom gradient currently supports only groups=1")
        y, xq8, wq = _conv_forward(x, w, lut, g4, 1)
        ctx.save_for_backward(xq8, wq, dx_lut, dw_lut)
        ctx.geom = g4
        return y

    @staticmethod
    def backward(ctx, grad_output):
        xq8, wq, dx_lut, dw_lut = ctx.saved_tensors
        B = xq8.shape[0]
        O = wq.shape[0]
        OH, OW = _out_hw(xq8.shape, ctx.geom)
        go = grad_output.reshape(B, O, OH, OW).contiguous()
        gx, gw = _ops.custom_conv_backward(go, xq8, wq, dx_lut, dw_lut, ctx.geom, _PAD_INDEX,
                                           need_x=ctx.needs_input_grad[0], need_w=ctx.needs_input_grad[1])
        return gx, gw, None, None, None, None


def conv2d_int8_custom(x, w, lut, dx_lut, dw_lut, geom):
    return _conv2d_int8_custom.apply(x, w, lut, dx_lut, dw_lut, geom)


# ----------------------------------------------------------------------------- fused layer path
class _approx_conv2d_int8(Function):
    """Whole signed layer in three kernels: fake-quant of the activation to an int8 image (+ mask),
    per-channel weight fake-quant to uint8 indices (+ mask), im2col-free LUT conv with the
    dequantisation ``bias + acc * (scale_x * scale_w[o])`` in its epilogue.  Same arithmetic as the
    chain static_quantize_int8 -> conv2d_int8_{ste,lre} -> addcmul of approxtorch/nn/Conv2d_int8.py:189-218.
    ``mode`` is 'ste' or 'lre'; scales are buffers and get no gradient."""

    @staticmethod
    def forward(ctx, x, weight, bias, scale_x, scale_w, lut, dx, dw, g4, mode, qmax_w):
        need_gx, need_gw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        xq8, xmask = _ops.quantize_image(x.detach(), scale_x, None, -127, 127, want_mask=need_gx)
        widx, wmask, _, _ = _ops.quantize_weight(weight.detach(), scale_w, None, -qmax_w, qmax_w, 128,
                                                 want_mask=need_gw)
        alpha = (scale_x * scale_w).contiguous()
        beta = None if bias is None else bias.detach().contiguous()
        y = _ops.lut_conv2d_launch(xq8, widx, _ops.lut_image(lut), g4, _PAD_INDEX, alpha=alpha, beta=beta)
        if need_gx or need_gw or (bias is not None and ctx.needs_input_grad[2]):
            # copies of the scale buffers: the module updates them in place on its next training forward, which may
            # come before this backward (the reference keeps a clamped copy for the same reason)
            keep = [xq8, widx, alpha, scale_x.clone(), scale_w.clone()]
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
        xq8, widx, alpha, scale_x, scale_w = saved[:5]
        rest = saved[5:]
        xmask = rest.pop(0) if ctx.have[0] else None
        wmask = rest.pop(0) if ctx.have[1] else None
        if ctx.mode == 'lre':
            dxt, dwt = rest[0].contiguous(), rest[1].contiguous()
        else:
            dxt = dwt = _ops.decode_table(xq8.device, 128)
        go = grad_output.contiguous()
        need_gx, need_gw, need_gb = ctx.needs_input_grad[:3]
        gx = gw = gb = None
        if need_gx or need_gw:
            # the activation's fake-quant backward (mask / scale) is applied in the store of the image gradient
            gx, gwq = _ops.lre_conv_backward(go, xq8, widx, dxt, dwt, ctx.g4, _PAD_INDEX, go_scale=alpha,
                                             need_x=need_gx, need_w=need_gw, exact_tables=ctx.mode != 'lre',
                                             x_mask=xmask if need_gx else None, x_scale=scale_x if need_gx else None)
            if need_gw:
                s = torch.clamp(scale_w, min=1e-12).view(-1, 1, 1, 1)
                gw = gwq.view(ctx.wshape) * wmask.to(gwq.dtype) / s
        if need_gb:
            gb = go.sum(dim=(0, 2, 3))
        return gx, gw, gb, None, None, None, None, None, None, None, None


def approx_conv2d_int8(x, weight, bias, scale_x, scale_w, lut, dx, dw, g4, mode, qmax_w):
    return _approx_conv2d_int8.apply(x, weight, bias, scale_x, scale_w, lut, dx, dw, g4, mode, qmax_w)
