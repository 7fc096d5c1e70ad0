"""Static fake-quantisation Functions with the reference's public surface
(approxtorch/nn/quantization.py:37-191): ``static_quantize_int8`` / ``static_quantize_uint8`` return the
integer-valued fp32 tensor q; scale and zero point are static (calibration / EMA) and get no gradient;
the backward is the straight-through ``go * mask / s`` with the mask taken on the pre-round value.

Every path runs a kernel of this package on CUDA fp32 tensors: per-tensor through the
``fakequant_per_tensor_*`` operators, per-channel through the per-output-channel weight kernel.
There is no CPU implementation.
"""

from __future__ import annotations

import torch
from torch.autograd import Function

from ..backend import ops as _ops


def _need_cuda_fp32(x: torch.Tensor, what: str) -> None:
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float32):
        raise RuntimeError(f"{what} must be a float32 CUDA tensor (approxtorch_b200 has no CPU path)")


class _static_quantize_per_tensor_symmetric(Function):

    @staticmethod
    def forward(ctx, x, scale, qmin, qmax):
        _need_cuda_fp32(x, "x")
        q, mask = torch.ops.approxtorch.fakequant_per_tensor_claude.default(x, scale, qmin, qmax)
        ctx.save_for_backward(mask, scale)
        return q

    @staticmethod
    def backward(ctx, grad_output):
        mask, scale = ctx.saved_tensors
        gx = torch.ops.approxtorch.fakequant_per_tensor_backward_claude.default(grad_output, mask, scale)
        return gx, None, None, None


class _static_quantize_per_tensor_asymmetric(Function):

    @staticmethod
    def forward(ctx, x, scale, zero_point, qmin, qmax):
        _need_cuda_fp32(x, "x")
        q, mask = torch.ops.approxtorch.fakequant_per_tensor_asymmetric_claude.default(
            x, scale, zero_point, qmin, qmax)
        ctx.save_for_backward(mask, scale)
        return q

    @staticmethod
    def backward(ctx, grad_output):
        mask, scale = ctx.saved_tensors
        gx = torch.ops.approxtorch.fakequant_per_tensor_asymmetric_backward_claude.default(
            grad_output, mask, scale)
        return gx, None, None, None, None


def _channel_first(x, ch_axis):
    """View of x with the channel axis first (contiguous copy only when it is not already first)."""
    ch_axis = ch_axis % x.dim()
    return (x if ch_axis == 0 else x.movedim(ch_axis, 0)).contiguous(), ch_axis


class _static_quantize_per_channel(Function):
    """Shared body of the symmetric / asymmetric per-channel Functions."""

    @staticmethod
    def _run(ctx, x, scale, zero_point, ch_axis, qmin, qmax):
        _need_cuda_fp32(x, "x")
        xc, axis = _channel_first(x, ch_axis)
        _, mask, q, _ = _ops.quantize_weight(xc, scale.to(torch.float32),
                                             None if zero_point is None else zero_point.to(torch.float32),
                                             int(qmin), int(qmax), 0, want_mask=True, want_q=True)
        view = [1] * x.dim()
        view[0] = -1
        s = torch.clamp(scale, min=1e-12).view(view)
        ctx.save_for_backward(mask, s)
        ctx.axis = axis
        return q if axis == 0 else q.movedim(0, axis)

    @staticmethod
    def _grad(ctx, grad_output):
        mask, s = ctx.saved_tensors
        g = grad_output if ctx.axis == 0 else grad_output.movedim(ctx.axis, 0)
        g = g * mask.to(g.dtype) / s
        return g if ctx.axis == 0 else g.movedim(0, ctx.axis)


class _static_quantize_per_channel_symmetric(_static_quantize_per_channel):

    @staticmethod
    def forward(ctx, x, scale, ch_axis, qmin, qmax):
        return _static_quantize_per_channel._run(ctx, x, scale, None, ch_axis, qmin, qmax)

    @staticmethod
    def backward(ctx, grad_output):
        return _static_quantize_per_channel._grad(ctx, grad_output), None, None, None, None


class _static_quantize_per_channel_asymmetric(_static_quantize_per_channel):

    @staticmethod
    def forward(ctx, x, scale, zero_point, ch_axis, qmin, qmax):
        return _static_quantize_per_channel._run(ctx, x, scale, zero_point, ch_axis, qmin, qmax)

    @staticmethod
    def backward(ctx, grad_output):
        return _static_quantize_per_channel._grad(ctx, grad_output), None, None, None, None, None


def _param(v, x):
    if isinstance(v, torch.Tensor):
        return v
    return torch.tensor(float(v), dtype=torch.float32, device=x.device)


def _check_channels(name, p, x, ch_axis):
    if p.numel() != x.shape[ch_axis]:
        raise ValueError(f"per-channel {name} must have {x.shape[ch_axis]} elements "
                         f"(= x.shape[{ch_axis}]), got {p.numel()}")


def static_quantize_int8(x, scale, qmin=-127, qmax=127, ch_axis=None):
    """Symmetric static quantisation q = clamp(round(x / scale), qmin, qmax), returned as fp32.

    ``ch_axis=None``: per-tensor (scale has one element); ``ch_axis=int``: per-channel, scale has
    ``x.shape[ch_axis]`` elements (activations NCHW use 1, weights OIHW use 0).  Custom bounds are
    allowed, e.g. [-31, 31] for 6-bit weights."""
    if qmin >= qmax:
        raise ValueError(f"qmin must be < qmax, got [{qmin}, {qmax}]")
    scale = _param(scale, x)
    if ch_axis is None:
        return _static_quantize_per_tensor_symmetric.apply(x, scale, qmin, qmax)
    _check_channels("scale", scale, x, ch_axis)
    return _static_quantize_per_channel_symmetric.apply(x, scale, ch_axis, qmin, qmax)


def static_quantize_uint8(x, scale, zero_point, qmin=0, qmax=255, ch_axis=None):
    """Asymmetric static quantisation q = clamp(round(x / scale + zero_point), qmin, qmax) as fp32;
    ``zero_point`` is integer-valued by convention so that real 0 lies on the grid."""
    if qmin >= qmax:
        raise ValueError(f"qmin must be < qmax, got [{qmin}, {qmax}]")
    scale = _param(scale, x)
    zero_point = _param(zero_point, x)
    if ch_axis is None:
        return _static_quantize_per_tensor_asymmetric.apply(x, scale, zero_point, qmin, qmax)
    _check_channels("scale", scale, x, ch_axis)
    _check_channels("zero_point", zero_point, x, ch_axis)
    return _static_quantize_per_channel_asymmetric.apply(x, scale, zero_point, ch_axis, qmin, qmax)
