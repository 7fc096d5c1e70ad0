"""Operator boundary of the approximate-multiplier path: ``_C`` loads the CUDA library,
``ops`` registers ``torch.ops.approxtorch.*`` and the reference-named wrappers
(same layout as approxtorch/backend/__init__.py:1-2)."""
from . import _C, ops  # noqa: F401
