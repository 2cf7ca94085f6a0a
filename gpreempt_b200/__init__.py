"""gpreempt_b200 — Python binding of libgpx, the B200 (sm_100a) preemptive inference executor.

The product is the C-ABI library (include/gpx.h) and the C++ classes above it
(include/gpx/*.h) that mirror thustorage/GPreempt's model/executor interfaces.  This package
binds the C ABI with ctypes for tests and benchmarks; there is no CPU fallback: importing
`gpreempt_b200.api` without a built library raises.
"""
from .binding import LIB_PATH, GpxError, load  # noqa: F401
