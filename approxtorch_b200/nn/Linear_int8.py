"""Signed approximate fully connected layer on the LUT GEMM.

The reference ships the ``gemm_fake_int8`` operators (approxtorch/backend/csrc/claude/gemm.cu:97-232) but no
layer that uses them; this one applies the conventions of its convolution layer
(approxtorch/nn/Conv2d_int8.py:137-218) to ``y = x W^T + b``: per-tensor symmetric activation scale with an
EMA of abs-max / 127 (MAX all-reduced under DDP), per-output-feature weight scale abs-max / (2^(bits-1) - 1),
every product looked up in the 256 x 256 table, dequantisation ``bias + acc * (scale_x * scale_w[o])``, and
the STE, LRE or custom-pair estimator in the backward pass.

A fully connected layer is the 1 x 1 convolution of a [B, in, 1, 1] image, so the layer is a view around
``Conv2d_int8``: same buffers (``lut``, ``scale_x``, ``scale_w``, ``dx``, ``dw``), same kernels, and a
``state_dict`` whose ``weight`` is [out, in].
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .Conv2d_int8 import Conv2d_int8


class Linear_int8(nn.Module):
    def __init__(self, in_features: int, out_features: int, lut: torch.Tensor, grad: str = 'ste',
                 dx: torch.Tensor | None = None, dw: torch.Tensor | None = None,
                 bias: torch.Tensor | bool | None = True, scale_momentum: float = 0.1,
                 update_scale: bool = True, weight_bits: int = 8):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.conv = Conv2d_int8(in_features, out_features, 1, lut, grad=grad, dx=dx, dw=dw, bias=bias,
                                scale_momentum=scale_momentum, update_scale=update_scale, weight_bits=weight_bits)

    # the parameters under their usual names
    @property
    def weight(self) -> torch.Tensor:
        return self.conv.weight.view(self.out_features, self.in_features)

    @property
    def bias(self):
        return self.conv.bias

    def freeze_scale(self):
        self.conv.freeze_scale()

    def unfreeze_scale(self):
        self.conv.unfreeze_scale()

    def state_dict(self, *args, destination=None, prefix='', keep_vars=False):
        sd = super().state_dict(*args, destination=destination, prefix=prefix, keep_vars=keep_vars)
        out = type(sd)()
        for k, v in sd.items():
            if k.startswith(prefix + 'conv.'):
                name = k[len(prefix) + 5:]
                out[prefix + name] = v.view(self.out_features, self.in_features) if name == 'weight' else v
            else:
                out[k] = v
        if hasattr(sd, '_metadata'):
            out._metadata = sd._metadata
        return out

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        # accept the flat names this layer saves: move them under the inner layer and give weight its 4-D shape
        for name in ('weight', 'bias', 'lut', 'scale_x', 'scale_w', 'dx', 'dw'):
            k = prefix + name
            if k in state_dict:
                v = state_dict.pop(k)
                if name == 'weight':
                    v = v.reshape(self.out_features, self.in_features, 1, 1)
                state_dict[prefix + 'conv.' + name] = v
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.in_features:
            raise RuntimeError(f"expected last dimension {self.in_features}, got {tuple(x.shape)}")
        lead = x.shape[:-1]
        y = self.conv(x.reshape(-1, self.in_features, 1, 1))
        return y.reshape(*lead, self.out_features)

    def __repr__(self):
        return (f"Linear_int8(in_features={self.in_features}, out_features={self.out_features}, "
                f"grad={self.conv.grad}, weight_bits={self.conv.weight_bits})")
