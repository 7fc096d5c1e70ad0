"""CPU oracle for the approximate-multiplier hot path (TEST INFRASTRUCTURE ONLY).

Everything under ``oracle/`` is a checker: a plain numpy / C restatement of the
reference algorithm that the CUDA path is compared with.  Only ``tests/``,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs
of ``bench.py`` may import or execute it.  The product package
``approxtorch_b200`` never imports it and has no CPU fallback.

Parity status: pinned.  ``tests/golden/`` holds outputs of the reference's own
Python modules and of its CPU BGEMM operator generated in the build container
(``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` checks this
restatement against every one of them.
"""

from . import lut_oracle  # noqa: F401
