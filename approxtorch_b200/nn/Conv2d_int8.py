"""Signed approximate convolution layer: drop-in for approxtorch/nn/Conv2d_int8.py:9-220.

Same constructor, buffers (``lut``, ``scale_x``, ``scale_w``, ``dx``, ``dw``), parameters and
state_dict keys, so reference checkpoints load.  Per-tensor symmetric activations in [-127, 127],
per-output-channel symmetric weights at 3..8 bits, EMA scales, LUT convolution in the integer
domain, dequantisation at the end.  groups is 1 or depthwise (groups == in == out).

The forward of the common case (groups == 1, grad 'ste' or 'lre') is three kernels of this package
(see ``bgemm_int8._approx_conv2d_int8``); the activation statistic is one fused abs-max reduction.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.modules.utils import _pair

from . import bgemm_int8, quantization
from ..backend import ops as _ops


class Conv2d_int8(nn.Module):
    def __init__(self,
                 in_channels: int,
                 out_channels: int,
                 kernel_size: int | tuple[int, int],
                 lut: torch.Tensor,
                 grad: str = 'ste',
                 dx: torch.Tensor | None = None,
                 dw: torch.Tensor | None = None,
                 bias: torch.Tensor | bool | None = None,
                 stride: int | tuple[int, int] = 1,
                 padding: int | tuple[int, int] = 0,
                 dilation: int | tuple[int, int] = 1,
                 groups: int = 1,
                 update_scale: bool = True,
                 scale_momentum: float = 0.05,
                 weight_bits: int = 8):
        super().__init__()
        depthwise = groups == in_channels and out_channels == in_channels
        if groups != 1 and not depthwise:
            raise NotImplementedError(
                "Conv2d_int8 supports groups=1 or depthwise (groups == in_channels == out_channels), "
                f"got groups={groups}, in={in_channels}, out={out_channels}")
        if grad not in ('ste', 'lre', 'custom'):
            raise ValueError(f"grad must be 'ste', 'lre' or 'custom', got {grad}")
        if grad == 'custom' and groups != 1:
            raise NotImplementedError("custom gradient currently supports only groups=1")
        if not 3 <= weight_bits <= 8:
            raise ValueError(f"weight_bits must be between 3 and 8, got {weight_bits}")
        if not 0.0 <= scale_momentum <= 1.0:
            raise ValueError(f"scale_momentum must be between 0 and 1, got {scale_momentum}")

        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride = _pair(kernel_size), _pair(stride)
        self.padding, self.dilation = _pair(padding), _pair(dilation)
        self.groups, self.grad = groups, grad
        self.qmin, self.qmax = -127, 127
        self.weight_bits = weight_bits
        self.scale_momentum = scale_momentum
        self.update_scale = update_scale

        self.register_buffer('lut', lut)
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels // groups, *self.kernel_size))
        self.register_buffer('scale_x', torch.tensor(1.0))
        self.register_buffer('scale_w', torch.ones(out_channels))   # dequant scale absmax/qmax, per channel

        if isinstance(bias, torch.Tensor) or bias == True:       # noqa: E712 (accepts 1 as the reference does)
            self.bias = nn.Parameter(torch.empty(out_channels))
        elif bias == False or bias is None:                       # noqa: E712
            self.bias = None
        else:
            raise ValueError("Invalid bias type")

        self.reset_parameters()
        self._reset_scale_w_from_weight()

        if isinstance(bias, torch.Tensor):
            if bias.shape != (out_channels,):
                raise ValueError(f"bias must have shape ({out_channels},), got {tuple(bias.shape)}")
            with torch.no_grad():
                self.bias.copy_(bias)

        if grad in ('lre', 'custom'):
            if dx is None or dw is None:
                raise ValueError(f"dx and dw are required when grad='{grad}'")
        if grad == 'lre':
            self.register_buffer('dx', dx)
            self.register_buffer('dw', dw)
        elif grad == 'custom':
            if not isinstance(dx, torch.Tensor) or not isinstance(dw, torch.Tensor):
                raise TypeError("custom dx and dw must be torch.Tensor objects")
            if dx.numel() != 65536 or dw.numel() != 65536:
                raise ValueError("custom dx and dw must each have 65536 elements for grad_lut[x + 128][w + 128]")
            if dx.dtype != torch.float32 or dw.dtype != torch.float32:
                raise TypeError("custom dx and dw must have dtype torch.float32")
            self.register_buffer('dx', dx.contiguous().view(-1))
            self.register_buffer('dw', dw.contiguous().view(-1))

    # ------------------------------------------------------------------ parameters and statistics
    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))    # nn.Conv2d's default
        if self.bias is not None:
            fan_in = (self.in_channels // self.groups) * self.kernel_size[0] * self.kernel_size[1]
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            nn.init.uniform_(self.bias, -bound, bound)

    def __repr__(self):
        return (f"Conv2d_int8(in_channels={self.in_channels}, out_channels={self.out_channels}, "
                f"kernel_size={self.kernel_size}, stride={self.stride}, padding={self.padding}, "
                f"dilation={self.dilation}, groups={self.groups}, grad={self.grad}, "
                f"weight_bits={self.weight_bits})")

    def unfreeze_scale(self):
        self.update_scale = True

    def freeze_scale(self):
        self.update_scale = False

    @property
    def _qmax_w(self) -> int:
        return 2 ** (self.weight_bits - 1) - 1

    def _weight_absmax(self):
        return self.weight.detach().abs().amax(dim=tuple(range(1, self.weight.dim())))

    def _update_scale(self, x):
        """EMA of the activation scale.  Under DDP the abs-max is MAX-all-reduced first so that every
        rank derives the same scale (one 4-byte message per layer per step)."""
        with torch.no_grad():
            if x.is_cuda and x.dtype == torch.float32:
                abs_max = _ops.absmax(x)[0]
            else:
                abs_max = x.abs().max()
            if dist.is_available() and dist.is_initialized():
                dist.all_reduce(abs_max, op=dist.ReduceOp.MAX)
            current = abs_max / ((self.qmax - self.qmin) / 2)
            m = self.scale_momentum
            self.scale_x.copy_(m * current + (1 - m) * self.scale_x)

    def _update_scale_w(self):
        """EMA of the per-channel weight scale; weights are bit-identical on all ranks, no collective."""
        with torch.no_grad():
            absmax = self._weight_absmax()
            current = torch.where(absmax > 0, absmax / self._qmax_w, self.scale_w)
            m = self.scale_momentum
            self.scale_w.copy_(m * current + (1 - m) * self.scale_w)

    def _reset_scale_w_from_weight(self):
        """Re-seed the weight scale from the present weights (construction and model conversion)."""
        with torch.no_grad():
            absmax = self._weight_absmax()
            self.scale_w.copy_(torch.where(absmax > 0, absmax / self._qmax_w, torch.ones_like(absmax)))

    # ------------------------------------------------------------------ forward
    def _frozen_operands(self):
        """(weight indices, alpha = s_x * s_w[o]) for the no-gradient forward, rebuilt only when the weights or the
        scales have changed (in-place versions and storage are the key): a frozen eval model quantises its weights
        once, not once per forward."""
        srcs = (self.weight, self.scale_x, self.scale_w)
        key = tuple((t._version, t.data_ptr(), t.device) for t in srcs)
        hit = getattr(self, "_frozen", None)
        if hit is None or hit[0] != key:
            widx, _, _, _ = _ops.quantize_weight(self.weight.detach(), self.scale_w, None, -self._qmax_w, self._qmax_w,
                                                 128, want_mask=False)
            hit = (key, widx, (self.scale_x * self.scale_w).contiguous())
            self._frozen = hit
        return hit[1:]

    def _forward_no_grad(self, x, g4):
        """Inference: int8 image, cached weight indices, LUT conv with the dequantisation in its epilogue.  The same
        arithmetic, bit for bit, as the fused training route."""
        xq8, _ = _ops.quantize_image(x, self.scale_x, None, self.qmin, self.qmax, want_mask=False)
        widx, alpha = self._frozen_operands()
        beta = None if self.bias is None else self.bias.detach().contiguous()
        return _ops.lut_conv2d_launch(xq8, widx, _ops.lut_image(self.lut), g4, 128, alpha=alpha, beta=beta)

    def forward(self, x: torch.Tensor):
        if self.training and self.update_scale:
            self._update_scale(x)
            self._update_scale_w()

        g4 = (tuple(self.kernel_size), tuple(self.stride), tuple(self.padding), tuple(self.dilation))
        fused = self.groups == 1 and self.grad in ('ste', 'lre') and x.is_cuda and x.dtype == torch.float32
        wants_grad = torch.is_grad_enabled() and (
            x.requires_grad or self.weight.requires_grad or (self.bias is not None and self.bias.requires_grad))
        if fused and not wants_grad:
            return self._forward_no_grad(x, g4)
        if fused:
            return bgemm_int8.approx_conv2d_int8(
                x, self.weight, self.bias, self.scale_x, self.scale_w, self.lut,
                getattr(self, 'dx', None), getattr(self, 'dw', None), g4, self.grad, self._qmax_w)

        # decoupled chain (depthwise and custom-gradient layers)
        B, _, H, W = x.shape
        O = self.out_channels
        OH, OW = _ops.conv_out_hw(H, W, *self.kernel_size, *self.stride, *self.padding, *self.dilation)
        xq = quantization.static_quantize_int8(x, self.scale_x, self.qmin, self.qmax)
        wq = quantization.static_quantize_int8(self.weight, self.scale_w, -self._qmax_w, self._qmax_w, ch_axis=0)
        geom = (self.kernel_size, self.stride, self.padding, self.dilation, self.groups)
        w2 = wq.view(O, -1)
        if self.grad == 'lre':
            y = bgemm_int8.conv2d_int8_lre(xq, w2, self.lut, self.dx, self.dw, geom)
        elif self.grad == 'custom':
            y = bgemm_int8.conv2d_int8_custom(xq, w2, self.lut, self.dx, self.dw, geom)
        else:
            y = bgemm_int8.conv2d_int8_ste(xq, w2, self.lut, geom)
        y = y.view(B, O, OH, OW)
        s = (self.scale_x * self.scale_w).view(1, -1, 1, 1)
        if self.bias is not None:
            return torch.addcmul(self.bias.view(1, -1, 1, 1), y, s)
        return y * s
