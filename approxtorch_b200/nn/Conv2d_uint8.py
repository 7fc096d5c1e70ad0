"""Unsigned asymmetric approximate convolution layer: drop-in for approxtorch/nn/Conv2d_uint8.py:11-325.

Activations per-tensor asymmetric q_x = clamp(round(x / s_x) + z_x, 0, 255); weights per-channel
asymmetric; both table operands are the raw uint8 values, ``lut[q_x][q_w]``.  Dequantisation needs the
zero-point cross terms (K taps per output):

    sum_k (q_x - z_x)(q_w - z_w[o]) = LUTSUM - z_w[o] * sum_k q_x - z_x * sum_k q_w + K * z_x * z_w[o]

with LUTSUM from the approximate multiplier and the correction in exact arithmetic.  Padding injects
z_x (the image of real 0), so padded taps cancel in the correction.

Buffers, parameters and state_dict behaviour match the reference (min/max statistics, explicit
scale / zero-point buffers, legacy min/max-only checkpoints, integer-valued zero-point validation).

Execution routes, numerically the same function:
* no gradient needed (inference): one fused sequence — uint8 index image, weight indices with their
  row sums, im2col-free LUT conv whose epilogue applies the correction in integer arithmetic, the
  scale and the bias;
* training with the STE or LRE estimator (``fused_training``, the default): the same fused forward keeping
  the uint8 image, and an image-space backward that folds the -z terms into its operand maps
  (``bgemm_uint8.approx_conv2d_uint8``) — no unfolded fp32 operand, no unfold;
* training with the custom estimator, or ``fused_training = False``: the reference's decoupled chain
  (fake-quant -> pad with z_x -> unfold -> LUT-BGEMM Function -> differentiable correction), where
  autograd supplies the -z terms.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.nn.modules.utils import _pair

from . import bgemm_uint8, quantization
from ..backend import ops as _ops


def uint8_qparams(mn, mx, qmax=255):
    """(scale, zero_point) from min/max statistics (scalars or per-channel vectors).

    The range is first widened to contain 0 so that the zero point lies in [0, qmax] and real 0 is
    exactly representable; the zero point is an integer stored as float."""
    lo = torch.clamp(mn, max=0.0)
    hi = torch.clamp(mx, min=0.0)
    scale = torch.clamp((hi - lo) / qmax, min=1e-12)
    zero = torch.round(-lo / scale).clamp(0.0, float(qmax))
    return scale, zero


class Conv2d_uint8(nn.Module):
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
                 scale_momentum: float = 0.05):
        super().__init__()
        if groups != 1:
            raise NotImplementedError(f"Conv2d_uint8 only supports groups=1 for now, got groups={groups}")
        if grad not in ('ste', 'lre', 'custom'):
            raise ValueError(f"grad must be 'ste', 'lre' or 'custom', got {grad}")
        if not 0.0 <= scale_momentum <= 1.0:
            raise ValueError(f"scale_momentum must be between 0 and 1, got {scale_momentum}")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride = _pair(kernel_size), _pair(stride)
        self.padding, self.dilation = _pair(padding), _pair(dilation)
        self.groups, self.grad = groups, grad
        self.qmin, self.qmax = 0, 255
        self.scale_momentum = scale_momentum
        self.update_scale = update_scale
        # route STE / LRE training through the fused image-space Function (False: the reference's decoupled chain)
        self.fused_training = True

        self.register_buffer('lut', lut)
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels, *self.kernel_size))
        # statistics (activation range starts at [0, 1]) and the qparams derived from them
        self.register_buffer('x_min', torch.tensor(0.0))
        self.register_buffer('x_max', torch.tensor(1.0))
        self.register_buffer('w_min', torch.zeros(out_channels))
        self.register_buffer('w_max', torch.ones(out_channels))
        self.register_buffer('scale_x', torch.tensor(1.0 / self.qmax))
        self.register_buffer('zero_x', torch.tensor(0.0))
        self.register_buffer('scale_w', torch.ones(out_channels))
        self.register_buffer('zero_w', torch.zeros(out_channels))

        if isinstance(bias, torch.Tensor) or bias == True:       # noqa: E712
            self.bias = nn.Parameter(torch.empty(out_channels))
        elif bias == False or bias is None:                       # noqa: E712
            self.bias = None
        else:
            raise ValueError("Invalid bias type")

        self.reset_parameters()
        with torch.no_grad():
            dims = tuple(range(1, self.weight.dim()))
            self.w_min.copy_(self.weight.detach().amin(dim=dims))
            self.w_max.copy_(self.weight.detach().amax(dim=dims))
        self._reset_qparams_from_stats()

        if isinstance(bias, torch.Tensor):
            if bias.shape != (out_channels,):
                raise ValueError(f"bias must have shape ({out_channels},), got {tuple(bias.shape)}")
            with torch.no_grad():
                self.bias.copy_(bias)

        if grad in ('lre', 'custom'):
            want = 256 if grad == 'lre' else 65536
            if dx is None or dw is None:
                raise ValueError(f"dx and dw are required when grad='{grad}'")
            if not isinstance(dx, torch.Tensor) or not isinstance(dw, torch.Tensor):
                raise TypeError(f"{grad} dx and dw must be torch.Tensor objects")
            if dx.numel() != want or dw.numel() != want:
                raise ValueError(f"{grad} dx and dw must each have {want} elements, indexed by the raw uint8 "
                                 "operand value" + ("s [x][w]" if grad == 'custom' else ""))
            if dx.dtype != torch.float32 or dw.dtype != torch.float32:
                raise TypeError(f"{grad} dx and dw must have dtype torch.float32")
            self.register_buffer('dx', dx.contiguous().view(-1))
            self.register_buffer('dw', dw.contiguous().view(-1))

    # ------------------------------------------------------------------ parameters and statistics
    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in = self.in_channels * self.kernel_size[0] * self.kernel_size[1]
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            nn.init.uniform_(self.bias, -bound, bound)

    def __repr__(self):
        return (f"Conv2d_uint8(in_channels={self.in_channels}, out_channels={self.out_channels}, "
                f"kernel_size={self.kernel_size}, stride={self.stride}, padding={self.padding}, "
                f"dilation={self.dilation}, groups={self.groups}, grad={self.grad})")

    def unfreeze_scale(self):
        self.update_scale = True

    def freeze_scale(self):
        self.update_scale = False

    def _reset_qparams_from_stats(self):
        """Refresh the explicit scale / zero-point buffers from the current min/max statistics."""
        with torch.no_grad():
            sx, zx = uint8_qparams(self.x_min, self.x_max, self.qmax)
            sw, zw = uint8_qparams(self.w_min, self.w_max, self.qmax)
            self.scale_x.copy_(sx)
            self.zero_x.copy_(zx)
            self.scale_w.copy_(sw)
            self.zero_w.copy_(zw)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict,
                              missing_keys, unexpected_keys, error_msgs):
        qparams = ('scale_x', 'zero_x', 'scale_w', 'zero_w')
        stats_only = all(prefix + n not in state_dict for n in qparams)     # early checkpoints
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict,
                                      missing_keys, unexpected_keys, error_msgs)
        if stats_only:
            self._reset_qparams_from_stats()
            for n in qparams:
                if prefix + n in missing_keys:
                    missing_keys.remove(prefix + n)
        for n in ('zero_x', 'zero_w'):
            z = getattr(self, n)
            ok = (torch.isfinite(z).all() and (z >= self.qmin).all() and (z <= self.qmax).all()
                  and torch.equal(z, torch.round(z)))
            if not ok:
                error_msgs.append(f"{prefix}{n} must contain integer-valued values in [{self.qmin}, {self.qmax}]")

    def _update_scale(self, x):
        """EMA of the activation min / max; MIN / MAX all-reduced across ranks first under DDP."""
        with torch.no_grad():
            if x.is_cuda and x.dtype == torch.float32:
                st = _ops.absmax(x, want_minmax=True)
                mn, mx = st[1], st[2]
            else:
                mn, mx = x.amin(), x.amax()
            if dist.is_available() and dist.is_initialized():
                dist.all_reduce(mn, op=dist.ReduceOp.MIN)
                dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            m = self.scale_momentum
            self.x_min.copy_(m * mn + (1 - m) * self.x_min)
            self.x_max.copy_(m * mx + (1 - m) * self.x_max)
            sx, zx = uint8_qparams(self.x_min, self.x_max, self.qmax)
            self.scale_x.copy_(sx)
            self.zero_x.copy_(zx)

    def _update_scale_w(self):
        with torch.no_grad():
            dims = tuple(range(1, self.weight.dim()))
            mn = self.weight.detach().amin(dim=dims)
            mx = self.weight.detach().amax(dim=dims)
            m = self.scale_momentum
            self.w_min.copy_(m * mn + (1 - m) * self.w_min)
            self.w_max.copy_(m * mx + (1 - m) * self.w_max)
            sw, zw = uint8_qparams(self.w_min, self.w_max, self.qmax)
            self.scale_w.copy_(sw)
            self.zero_w.copy_(zw)

    # ------------------------------------------------------------------ forward
    def _frozen_operands(self):
        """(weight indices, their row sums, alpha = s_x * s_w, zero_w) for the no-gradient forward, rebuilt only when
        the weights or the quantisation buffers they derive from have changed (in-place versions and storage are
        the key): a frozen eval model quantises its weights once, not once per forward."""
        srcs = (self.weight, self.scale_x, self.scale_w, self.zero_w)
        key = tuple((t._version, t.data_ptr(), t.device) for t in srcs)
        hit = getattr(self, "_frozen", None)
        if hit is None or hit[0] != key:
            widx, _, _, wsum = _ops.quantize_weight(self.weight.detach(), self.scale_w, self.zero_w, self.qmin,
                                                    self.qmax, 0, want_mask=False, want_sum=True)
            alpha = (self.scale_x * self.scale_w).contiguous()
            hit = (key, widx, wsum, alpha, self.zero_w.contiguous())
            self._frozen = hit
        return hit[1:]

    def _forward_fused(self, x):
        xq8, _ = _ops.quantize_image(x, self.scale_x, self.zero_x, self.qmin, self.qmax, want_mask=False)
        widx, wsum, alpha, zero_w = self._frozen_operands()
        beta = None if self.bias is None else self.bias.detach().contiguous()
        g4 = (tuple(self.kernel_size), tuple(self.stride), tuple(self.padding), tuple(self.dilation))
        return _ops.lut_conv2d_launch(xq8, widx, _ops.lut_image(self.lut), g4, -1, alpha=alpha, beta=beta,
                                      zero_x=self.zero_x, zero_w=zero_w, wsum=wsum)

    def forward(self, x: torch.Tensor):
        B, C, H, W = x.shape
        O = self.out_channels
        kH, kW = self.kernel_size
        sH, sW = self.stride
        pH, pW = self.padding
        OH, OW = _ops.conv_out_hw(H, W, kH, kW, sH, sW, pH, pW, *self.dilation)

        if self.training and self.update_scale:
            self._update_scale(x)
            self._update_scale_w()

        wants_grad = torch.is_grad_enabled() and (
            x.requires_grad or self.weight.requires_grad or (self.bias is not None and self.bias.requires_grad))
        if not wants_grad and x.is_cuda and x.dtype == torch.float32:
            return self._forward_fused(x)
        if self.fused_training and self.grad in ('ste', 'lre') and x.is_cuda and x.dtype == torch.float32:
            g4 = (tuple(self.kernel_size), tuple(self.stride), tuple(self.padding), tuple(self.dilation))
            return bgemm_uint8.approx_conv2d_uint8(x, self.weight, self.bias, self.scale_x, self.zero_x, self.scale_w,
                                                   self.zero_w, self.lut, getattr(self, 'dx', None),
                                                   getattr(self, 'dw', None), g4, self.grad,
                                                   self.qmin, self.qmax)

        scale_x, zero_x, scale_w, zero_w = self.scale_x, self.zero_x, self.scale_w, self.zero_w
        xq = quantization.static_quantize_uint8(x, scale_x, zero_x, self.qmin, self.qmax)
        wq = quantization.static_quantize_uint8(self.weight, scale_w, zero_w, self.qmin, self.qmax, ch_axis=0)
        if pH or pW:
            # padding must carry z_x (not 0) or the correction is wrong on the border
            xq = F.pad(xq - zero_x, (pW, pW, pH, pH)) + zero_x
        if (kH, kW) == (1, 1):
            if self.stride != (1, 1):
                xq = xq[:, :, ::sH, ::sW]
            xu = xq.flatten(2)
        else:
            xu = F.unfold(xq, self.kernel_size, dilation=self.dilation, padding=0, stride=self.stride)
        wu = wq.view(O, -1)

        if self.grad == 'lre':
            y = bgemm_uint8.bgemm_uint8_lre(xu, wu, self.lut, self.dx, self.dw)
        elif self.grad == 'custom':
            y = bgemm_uint8.bgemm_uint8_custom(xu, wu, self.lut, self.dx, self.dw)
        else:
            y = bgemm_uint8.bgemm_uint8_ste(xu, wu, self.lut)

        K = wu.shape[1]
        zw = zero_w.view(1, -1, 1)
        y = y - zw * xu.sum(dim=1).unsqueeze(1) - (zero_x * wu.sum(dim=1)).view(1, -1, 1) + K * zero_x * zw
        y = y.view(B, O, OH, OW)
        s = (scale_x * scale_w).view(1, -1, 1, 1)
        if self.bias is not None:
            return torch.addcmul(self.bias.view(1, -1, 1, 1), y, s)
        return y * s
