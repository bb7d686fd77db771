"""CPU oracle for the quantized decode path — TEST INFRASTRUCTURE ONLY.

Only the test-suite, ``__graft_entry__.smoke()`` and the benchmark's CPU legs may import
this package; the product package ``runit_mac_b200`` never does.  Parity for the quantized
operators is UNPINNED (the reference holds no golden vectors for them); see the header of
``runit_oracle.h``.
"""
from .binding import *  # noqa: F401,F403
from .packing import *  # noqa: F401,F403
