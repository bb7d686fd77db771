"""runit_mac_b200 — B200 (sm_100a) implementation of RunIT's quantized decode path.

The product is ``librunit_cuda.so`` (hand-written CUDA behind the C ABI of
``include/runit_cuda.h``); this package is the thin host-side mirror of the reference's
dispatch layer used by the tests and the benchmark.  Importing the package does not load the
library; creating a ``Context`` does, and fails loudly if it is missing or no B200 is present.
"""
from .dispatch import *  # noqa: F401,F403
from .dispatch import __all__ as _dispatch_all

__all__ = list(_dispatch_all)
