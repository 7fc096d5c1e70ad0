"""Approximate convolution layers and their autograd Functions (same exports as approxtorch/nn/__init__.py:4-9,
minus the naive comparison operators), plus a fully connected layer on the same kernels."""
from .Conv2d_int8 import Conv2d_int8
from .Conv2d_uint8 import Conv2d_uint8
from .Linear_int8 import Linear_int8
from . import bgemm_int8
from . import bgemm_uint8
from . import quantization
