"""ctypes front-end of ``lut_oracle_c.c`` (TEST INFRASTRUCTURE ONLY).

``build()`` compiles the C restatement with gcc + OpenMP into
``oracle/_build/liblut_oracle.so``; ``bgemm_u8`` calls it.  The product package
never imports this module.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "lut_oracle_c.c")
_OUT_DIR = os.path.join(_HERE, "_build")
_LIB = os.path.join(_OUT_DIR, "liblut_oracle.so")
_handle = None


def build(force: bool = False) -> str:
    """Compile the C oracle if it is missing or older than its source."""
    if (not force and os.path.exists(_LIB)
            and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC)):
        return _LIB
    os.makedirs(_OUT_DIR, exist_ok=True)
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    cmd = [cc, "-O3", "-march=native", "-fopenmp", "-shared", "-fPIC", _SRC, "-o", _LIB, "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB


def _lib():
    global _handle
    if _handle is None:
        _handle = ctypes.CDLL(build())
        _handle.oracle_bgemm_u8.restype = ctypes.c_int
        _handle.oracle_bgemm_u8.argtypes = [
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
            ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
            ctypes.c_longlong, ctypes.c_void_p]
        _handle.oracle_num_threads.restype = ctypes.c_int
    return _handle


def num_threads() -> int:
    return int(_lib().oracle_num_threads())


def bgemm_u8(xq, wq, lut) -> np.ndarray:
    """float64 [N,O,L] = sum_k lut[xq[n,k,l]][wq[(n,)o,k]] (exact for integer tables)."""
    xq = np.ascontiguousarray(xq, dtype=np.uint8)
    wq = np.ascontiguousarray(wq, dtype=np.uint8)
    lut = np.ascontiguousarray(np.asarray(lut, dtype=np.float32).reshape(-1))
    N, K, L = xq.shape
    O = wq.shape[-2]
    assert wq.shape[-1] == K and lut.size == 65536
    wstride = O * K if wq.ndim == 3 else 0
    y = np.empty((N, O, L), dtype=np.float64)
    rc = _lib().oracle_bgemm_u8(xq.ctypes.data, wq.ctypes.data, lut.ctypes.data,
                                N, K, L, O, wstride, y.ctypes.data)
    if rc != 0:
        raise MemoryError("oracle_bgemm_u8 failed to allocate")
    return y
