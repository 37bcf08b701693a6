"""B200-native CKKS encrypted-aggregation path behind CAHEL's API.

The compute lives in ``liblancelot_b200.so`` (hand-written CUDA for sm_100a, C ABI in
``include/lancelot_b200.h``).  This package is the host-side mirror of the reference's
``pyCAHEL`` module and of the encrypted-Krum driver that calls it; it never computes on
the CPU and raises if the CUDA library is missing.
"""
from ._lib import LancelotError, lib, lib_path  # noqa: F401

__all__ = ["LancelotError", "lib", "lib_path"]
