"""eddl_b200: B200 (sm_100a) backend for EDDL's data-parallel convnet training step.

The product is native: ``eddl_b200/lib/libeddl_b200.so`` (CUDA kernels + the C ABI of
``include/eddl_b200.h``) and the C++ shim in ``eddl_b200/shim`` that defines EDDL's ``gpu_*``
functions on top of it.  This Python package only binds the C ABI (``capi``) and the net
harness (``harness``) for tests and benchmarks.
"""
from . import capi  # noqa: F401

__all__ = ["capi"]
