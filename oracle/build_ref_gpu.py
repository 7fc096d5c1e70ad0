"""Build the reference's OWN maintained CUDA operators for sm_100a (TEST / BASELINE INFRASTRUCTURE ONLY).

Compiles, where they lie in the reference checkout (nothing is copied), the translation units of the
maintained hot path into one loadable operator library under ``oracle/_ref/``:

    approxtorch/backend/csrc/claude/bgemm_float_claude.cu     LUT-BGEMM forward (int8 / uint8, _cfg, _save)
    approxtorch/backend/csrc/claude/gemm.cu                   torch.mm-layout LUT GEMM
    approxtorch/backend/csrc/claude/quantization.cu           fused fake-quant
    approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu   LRE backward, im2col_u8, lut_map(_pad)
    approxtorch/backend/csrc/cuda/bgemm_custom_grad_optimize.cu    custom-pair backward

nvcc cross-compiles (no GPU needed, several minutes because of the torch headers).  The library registers the
same ``torch.ops.approxtorch`` schemas as this repository's binding, so it must be loaded in a process that has
NOT imported ``approxtorch_b200``: ``oracle/ref_gpu_worker.py`` is that process.
"""

from __future__ import annotations

import glob
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref", "gpu")
_NAME = "ref_gpu_ops"
SOURCES = [
    "approxtorch/backend/csrc/claude/bgemm_float_claude.cu",
    "approxtorch/backend/csrc/claude/gemm.cu",
    "approxtorch/backend/csrc/claude/quantization.cu",
    "approxtorch/backend/csrc/claude/bgemm_lre_backward_claude.cu",
    "approxtorch/backend/csrc/cuda/bgemm_custom_grad_optimize.cu",
]


def built_library() -> str | None:
    hits = sorted(glob.glob(os.path.join(REF_DIR, _NAME + "*.so")))
    return hits[0] if hits else None


def build(root: str | None = None) -> str | None:
    repo = os.path.dirname(_HERE)
    if repo not in sys.path:
        sys.path.insert(0, repo)
    from oracle.build_ref import reference_root
    root = root or reference_root()
    srcs = [os.path.join(root, s) for s in SOURCES] if root else []
    if not srcs or not all(os.path.exists(s) for s in srcs):
        return built_library()
    lib = built_library()
    if lib and all(os.path.getmtime(lib) >= os.path.getmtime(s) for s in srcs):
        return lib
    os.makedirs(REF_DIR, exist_ok=True)
    if os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    os.environ.setdefault("MAX_JOBS", "5")
    from torch.utils.cpp_extension import load
    load(name=_NAME, sources=srcs, build_directory=REF_DIR,
         extra_cflags=["-O3"], extra_cuda_cflags=["-O3", "-ccbin", "/usr/bin/g++"],
         is_python_module=False, verbose="--verbose" in sys.argv)
    return built_library()


if __name__ == "__main__":
    print(build())
