"""deepforge_b200: a B200-native execution backend for DeepForge's op hot path.

The product is two native libraries (see build.py): the sm_100a kernel library
behind the C ABI of include/dfgpu.h, and the C++ host side that mirrors the
reference's importer / planner / Executable interface. This package only loads
them through ctypes; there is no Python or CPU fallback for any kernel.
"""
from . import dfgpu  # noqa: F401

__all__ = ["dfgpu"]
