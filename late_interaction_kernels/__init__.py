"""Import alias: ``import late_interaction_kernels`` resolves to the B200 engine.

Third-party code that binds the reference package by name (PyLate >= 1.5.1 and colpali-engine >= 0.3.17
call ``late_interaction_kernels.maxsim`` / ``maxsim_pairs`` by keyword) picks up this build when the
repository root is on ``sys.path`` ahead of an installed reference.  Every public submodule of the
reference that this build covers is aliased too (``late_interaction_kernels.plaid`` and so on).
"""

import importlib
import sys

import late_interaction_kernels_b200 as _impl
from late_interaction_kernels_b200 import *  # noqa: F401,F403
from late_interaction_kernels_b200 import __all__, __version__  # noqa: F401

for _name in ("autograd", "forward", "backward", "varlen", "score_pairs", "padded", "fp8", "topk", "retrieve", "plaid",
              "pylate_compat", "colpali_compat", "sharded"):
    _mod = importlib.import_module(f"late_interaction_kernels_b200.{_name}")
    sys.modules[f"{__name__}.{_name}"] = _mod
    # `retrieve` the function must stay the package attribute, as in the reference; the module is reachable by import
    if _name != "retrieve":
        globals()[_name] = _mod
for _sub in ("unified", "lowmem"):
    sys.modules[f"{__name__}.backward.{_sub}"] = importlib.import_module(f"late_interaction_kernels_b200.backward.{_sub}")
