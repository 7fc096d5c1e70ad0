"""approxtorch_b200: the approximate-multiplier hot path of ApproxTorch on hand-written sm_100a CUDA.

Public surface (same names as the reference package, approxtorch/__init__.py:11-21):
``convert_model``, ``nn`` (Conv2d_int8, Conv2d_uint8, the autograd Functions, quantization),
``backend.ops`` (``torch.ops.approxtorch.*``), ``load_lut``, ``grad_lut``, ``calib``.
``install_as_approxtorch()`` makes ``import approxtorch`` resolve to this package.
"""

from . import backend
from . import nn
from .convert_model import convert_model
from . import load_lut
from . import grad_lut
from . import calib

__version__ = "0.1.0"


def install_as_approxtorch() -> None:
    """Alias this package as ``approxtorch`` in ``sys.modules`` (drop-in for code that imports the
    reference by name).  Refuses to shadow an already imported different package."""
    import sys
    me = sys.modules[__name__]
    other = sys.modules.get("approxtorch")
    if other is not None and other is not me:
        raise RuntimeError("a different 'approxtorch' package is already imported")
    sys.modules["approxtorch"] = me
    for sub in ("backend", "nn", "convert_model", "load_lut", "grad_lut", "calib"):
        sys.modules["approxtorch." + sub] = sys.modules[__name__ + "." + sub]
    sys.modules["approxtorch.backend.ops"] = sys.modules[__name__ + ".backend.ops"]
