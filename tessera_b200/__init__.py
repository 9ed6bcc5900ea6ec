"""tessera_b200: sm_100a CUDA backend for Tessera's quantized projection path.

The product is the shared library ``tessera_b200/lib/libtessera_b200.so`` (C ABI
in ``include/tessera_b200.h``) and the C++ ``CudaBackend`` built on it.  This
Python package is the thin host layer used by the tests and the benchmark: a
ctypes binding (:mod:`tessera_b200.capi`), a mirror of the reference's
``tessera::Backend`` interface (:mod:`tessera_b200.backend`), the projection
planner (:mod:`tessera_b200.project`) and seeded synthetic inputs
(:mod:`tessera_b200.synth`).  There is no CPU fallback anywhere in it.
"""

from .capi import StatusCode, StatusError, library_path, load_library  # noqa: F401

__all__ = ["StatusCode", "StatusError", "library_path", "load_library"]
