"""denno_beta_b200: B200-native quantised-MoE expert matmul path of denno-beta.

The product is ``libdnb200.so`` (CUDA, C ABI, declared in ``include/dnb200.h``);
this package is its Python host side, mirroring denno-engine's ``cuda::*``
dispatch functions for the path.  Importing it needs neither a GPU nor the built
library; using it needs both.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
