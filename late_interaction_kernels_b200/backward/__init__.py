"""Backward strategies for MaxSim (counterpart of the reference's ``backward/`` package).

* :func:`maxsim_backward_lowmem`  — destination-owned reduction, gradients written once in the
  input dtype, no atomics, bitwise reproducible.
* :func:`maxsim_backward_unified` — fp32 atomic scatter for ``grad_D`` followed by a cast.
"""

from .lowmem import maxsim_backward_lowmem
from .unified import maxsim_backward_unified

__all__ = ["maxsim_backward_unified", "maxsim_backward_lowmem"]
