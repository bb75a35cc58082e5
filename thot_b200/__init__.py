"""thot_b200 — B200-native (sm_100a) row-op path behind Nott's layer/activation API.

Only what the path needs: `csrc/` (CUDA kernels + the C ABI, built into
libnott_b200.so), `abi` (ctypes binding of that ABI), `host/` (the C++ libtorch
layer that mirrors Nott's modules) and `sharding` (row partition + the one
allreduce of the affine-gradient partials).
"""
from . import abi  # noqa: F401

__all__ = ["abi"]
