"""B200 (sm_100a) fused layer kernels of dl-cuda behind a C ABI.

The product is ``libdlcuda_b200.so`` (sources in ``csrc/``, interface in
``include/dlcuda_b200.h``) and the C++ layer classes in ``src/`` that mirror the
reference's API on top of it.  The Python here is plumbing for tests and
benchmarks: ``capi`` binds the C ABI through ctypes, ``ops`` wraps it for torch
tensors, ``build`` compiles it.
"""
from . import capi  # noqa: F401

__all__ = ["capi"]
