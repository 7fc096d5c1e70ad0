"""Text-file loaders for multiplier tables and gradient tables (same functions and return types as
approxtorch/load_lut.py:5-55).  A table file holds 256 x 256 whitespace-separated integers, row i
being the first operand A = i - 128 (signed) or i (unsigned)."""

from __future__ import annotations

from typing import Literal

import numpy as np
import torch


def load_lut(file_path, qtype: Literal['int8', 'int4', 'uint8'] = 'int8'):
    """Flattened int32 table (65536 entries; 256 for 'int4'); cast to float32 and move to the GPU
    before handing it to a layer."""
    side = 256 if qtype in ('int8', 'uint8') else 16
    table = np.loadtxt(file_path, dtype=np.int32).reshape(side, side)
    out = torch.tensor(table).view(side * side).to(torch.int)
    out.requires_grad_(False)
    return out


def _flat_float(path):
    t = torch.tensor(np.loadtxt(path, dtype=np.float32)).view(-1)
    t.requires_grad_(False)
    return t


def load_lre_grad_lut(da_file_path, db_file_path):
    """(dx, dw): 256 fp32 slopes each."""
    return _flat_float(da_file_path), _flat_float(db_file_path)


def load_half_custom_grad_lut(file_path):
    """Single custom table (weight-side gradients only)."""
    return torch.tensor(np.loadtxt(file_path, dtype=np.float32)).view(-1)


def load_custom_grad_lut(dx_file_path, dw_file_path):
    """Pair-wise custom gradients indexed ``[x + 128, w + 128]``, flattened to 65536 entries each."""
    return _flat_float(dx_file_path), _flat_float(dw_file_path)
