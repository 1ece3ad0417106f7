"""B200 (sm_100a) packed polynomial transcendentals.

Layout:
  ``_lib``            ctypes binding of the C ABI (``include/fpt_b200.h``)
  ``spline_ops``      the reference's op names and signatures on torch CUDA tensors
  ``build``           in-tree nvcc build of ``libfpt_b200.so``
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
