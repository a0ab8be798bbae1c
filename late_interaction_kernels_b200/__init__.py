"""B200-native MaxSim kernels with the public API of ``late_interaction_kernels``.

Every operator runs a hand-written sm_100a CUDA kernel from ``liblik_b200.so`` (C ABI in
``include/lik_b200.h``).  There is no Triton, no CPU path and no fallback: tensors that are not on
a CUDA device raise ``RuntimeError``.
"""

__version__ = "0.1.0"

from ._ops import check_device_status
from .autograd import maxsim, maxsim_pairs
from .colpali_compat import patch_colpali_engine, unpatch_colpali_engine
from .padded import maxsim_padded
from .pylate_compat import patch_pylate, unpatch_pylate
from .retrieve import MaxSimScorer, retrieve
from .varlen import maxsim_varlen

__all__ = [
    "__version__",
    "MaxSimScorer",
    "retrieve",
    "maxsim_padded",
    "patch_pylate",
    "unpatch_pylate",
    "patch_colpali_engine",
    "unpatch_colpali_engine",
    "maxsim",
    "maxsim_pairs",
    "maxsim_varlen",
    "check_device_status",
]
