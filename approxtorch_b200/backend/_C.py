"""Loader of the C-ABI CUDA library (the counterpart of the reference's empty ``_C`` stub module,
approxtorch/backend/csrc/dummy_module.cpp:6-22, whose only job is to load the operator library).

The library is ``approxtorch_b200/lib/libapproxtorch_b200.so``, built in-tree by
``python -m approxtorch_b200.build`` (and refreshed here when a source file is newer and nvcc is present).
There is no fallback: if it is missing the import fails.
"""

from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "lib", "libapproxtorch_b200.so")


def _refresh_if_stale() -> None:
    """Rebuild the library when a source is newer than it and a compiler is at hand (a no-op otherwise)."""
    from ..build import build_library, sources
    import shutil
    have_nvcc = os.path.exists("/usr/local/cuda/bin/nvcc") or shutil.which("nvcc") is not None
    if have_nvcc and sources():
        build_library()


_refresh_if_stale()
if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build the CUDA library first with "
        "`python -m approxtorch_b200.build` (needs nvcc; there is no CPU fallback)")

lib = ctypes.CDLL(LIB_PATH)

_vp, _i, _ll, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_size_t


class GemmPlan(ctypes.Structure):
    _fields_ = [("block_rows", _i), ("blocks", _i), ("units_per_block", _i), ("chunks_per_tile", _i), ("cut_tiles", _i),
                ("scratch_bytes", _sz)]


_SIGNATURES = {
    "atb_last_error": (ctypes.c_char_p, []),
    "atb_version": (_i, []),
    "atb_device_status": (_i, [ctypes.POINTER(ctypes.c_int)]),
    "atb_lut_image_bytes": (_sz, []),
    "atb_lut_prepare": (_i, [_vp, _vp, _vp]),
    "atb_lut_image_class": (_i, [_vp, ctypes.POINTER(ctypes.c_int), _vp]),
    "atb_quantize_u8": (_i, [_vp, _vp, _ll, _i, _vp]),
    "atb_quantize_transpose_u8": (_i, [_vp, _i, _i, _i, _ll, _ll, _i, _vp, _vp]),
    "atb_im2col_u8": (_i, [_vp, _i] + [_i] * 12 + [_i, _vp, _vp]),
    "atb_lut_gemm_plan": (_i, [_ll, _i, _i, _i, _i, ctypes.POINTER(GemmPlan)]),
    "atb_lut_bgemm_fwd": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _ll,
                               _vp, _vp, _vp, _vp, _vp, _i, _vp, _sz, _vp]),
    "atb_static_scratch_bytes": (_sz, []),
    "atb_lut_bgemm_fwd_noalloc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _ll,
                                       _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "atb_lut_conv2d_fwd": (_i, [_vp, _i, _vp, _vp, _vp] + [_i] * 13 + [_i]
                           + [_vp] * 5 + [_i, _vp, _sz, _vp]),
    "atb_pixel_rows_u8": (_i, [_vp, _i] + [_i] * 12 + [_i, _vp, _vp, _vp, _vp]),
    "atb_lut_gemm_rows_plan": (_i, [_i, _i, _ll, _i, ctypes.POINTER(GemmPlan)]),
    "atb_lut_conv2d_rows_fwd": (_i, [_vp, _vp, _vp, _vp, _i, _i, _ll, _i] + [_vp] * 5 + [_i, _vp, _sz, _vp]),
    "atb_absmax": (_i, [_vp, _ll, _i, _vp, _vp]),
    "atb_fakequant_fwd": (_i, [_vp, _vp, _vp, _i, _i, _vp, _vp, _ll, _vp]),
    "atb_fakequant_bwd": (_i, [_vp, _vp, _vp, _vp, _ll, _vp]),
    "atb_quantize_image": (_i, [_vp, _vp, _vp, _i, _i, _vp, _vp, _ll, _vp]),
    "atb_quantize_weight": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "atb_lut_map": (_i, [_vp, _i, _vp, _vp, _ll, _vp]),
    "atb_lut_map_pad": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "atb_lre_bwd": (_i, [_vp, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "atb_lre_conv_bwd": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp] + [_i] * 13 + [_i, _i, _vp, _sz, _vp]),
    "atb_lre_conv_bwd_scratch_bytes": (_sz, [_i] * 16),
    "atb_tensor_core_status": (_i, [ctypes.POINTER(ctypes.c_int)]),
    "atb_pair_table_bytes": (_sz, []),
    "atb_pair_table_prepare": (_i, [_vp, _vp, _vp]),
    "atb_pair_status": (_i, [ctypes.POINTER(ctypes.c_int)]),
    "atb_custom_bwd_dx": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "atb_custom_bwd_dw": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "atb_custom_conv_bwd": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp] + [_i] * 13 + [_i, _i, _vp]),
    "atb_lut_dwconv_fwd": (_i, [_vp, _i, _vp, _vp, _vp] + [_i] * 12 + [_i, _vp]),
    "atb_lut_dwconv_bwd": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp] + [_i] * 12 + [_i, _vp]),
    "atb_probe_shared_load": (_i, [_vp, _vp, _i, _i, _vp]),
}

for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here means header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTED = tuple(_SIGNATURES)


def last_error() -> str:
    msg = lib.atb_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status: int, what: str) -> None:
    """Turn a non-zero C-ABI status into the RuntimeError the reference's TORCH_CHECKs raise."""
    if status != 0:
        raise RuntimeError(f"{what}: {last_error()} (status {status})")
