"""B200-native render-to-observation path for GraDOOM vector environments.

Hand-written sm_100a CUDA kernels behind a C ABI (``csrc/``,
``include/gradoom_b200.h``) plus the Python host side that mirrors the
reference's ``GraDoomVecEnv`` device API for this path.  The directory name is
not a Python identifier; load it with ``__graft_entry__.load_package()``, which
registers it as ``gradoom_b200``.
"""

from . import scene, state, stepper  # noqa: F401

__all__ = ["scene", "state", "stepper"]
