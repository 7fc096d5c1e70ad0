"""Build and load the reference's OWN CPU LUT-BGEMM operator (TEST INFRASTRUCTURE ONLY).

The reference ships a CPU implementation of the path in
``approxtorch/backend/csrc/cpu/bgemm.cpp`` (int8/uint8 operands, int32 table,
OpenMP).  ``build()`` compiles that file where it lies in the reference checkout
(no sources are copied) into ``oracle/_ref/``; ``load()`` loads the prebuilt
library, which is all that is possible on a machine without the checkout.

Operand order of that legacy operator: it evaluates ``lut[w][x]`` (weight is the
table row, approxtorch/backend/csrc/cpu/bgemm.cpp:70-72) whereas the maintained
path evaluates ``lut[x][w]``; callers here therefore pass the TRANSPOSED table.
"""

from __future__ import annotations

import glob
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")
_NAME = "ref_cpu_bgemm"
_loaded = False


def reference_root() -> str | None:
    """Where the reference checkout lies: ``$APPROXTORCH_REF`` when set, else a directory named ``reference``
    beside this repository; None when neither exists."""
    env = os.environ.get("APPROXTORCH_REF")
    if env:
        return env if os.path.isdir(env) else None
    sibling = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return sibling if os.path.isdir(sibling) else None


def _source(reference_root: str) -> str:
    return os.path.join(reference_root, "approxtorch", "backend", "csrc", "cpu", "bgemm.cpp")


def built_library() -> str | None:
    hits = sorted(glob.glob(os.path.join(REF_DIR, _NAME + "*.so")))
    return hits[0] if hits else None


def build(root: str | None = None) -> str | None:
    """Compile the reference CPU operator; returns the library path (a prebuilt one when the reference
    checkout is absent) or None."""
    root = root or reference_root()
    src = _source(root) if root else None
    if src is None or not os.path.exists(src):
        return built_library()
    lib = built_library()
    if lib and os.path.getmtime(lib) >= os.path.getmtime(src):
        return lib
    os.makedirs(REF_DIR, exist_ok=True)
    # the image's default g++ cannot link OpenMP; the system one can
    if os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    from torch.utils.cpp_extension import load
    load(name=_NAME, sources=[src], build_directory=REF_DIR,
         extra_cflags=["-O3", "-fopenmp"], extra_ldflags=["-fopenmp"],
         is_python_module=False, verbose=False)
    global _loaded
    _loaded = True
    return built_library()


def load() -> bool:
    """Load the prebuilt reference operator; False when it was never built."""
    global _loaded
    if _loaded:
        return True
    lib = built_library()
    if lib is None:
        return False
    import torch
    torch.ops.load_library(lib)
    _loaded = True
    return True


def bgemm_lut_xw(x_idx_u8, w_idx_u8, lut):
    """Reference CPU operator evaluated with the maintained ``lut[x][w]``
    meaning: uint8 LUT indices x [N,K,L], w [O,K], fp32 table -> int32 [N,O,L]."""
    import torch
    if not load():
        raise RuntimeError("reference CPU operator was not built (oracle/_ref is empty)")
    x = torch.as_tensor(x_idx_u8, dtype=torch.uint8)
    w = torch.as_tensor(w_idx_u8, dtype=torch.uint8)
    t = torch.as_tensor(lut, dtype=torch.float32).reshape(256, 256).t().contiguous()
    return torch.ops.approxtorch.bgemm_uint8(x, w, t.reshape(-1).to(torch.int32))


if __name__ == "__main__":
    print(build())
