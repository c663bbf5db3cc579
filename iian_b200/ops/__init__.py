"""The kernel layer.  Parts call ``ops.kernels()`` and nothing else to compute.

The product has one kernel set, :class:`~iian_b200.ops.cuda_backend.CudaKernels` (hand-written
CUDA for sm_100a, CUDA tensors only).  ``use_kernels`` exists so that tests of the host logic
(batch building, block tables, scheduling) can put a stand-in underneath the parts; the engine
never installs one itself.
"""
from __future__ import annotations

from contextlib import contextmanager

_active = None


def kernels():
    global _active
    if _active is None:
        from .cuda_backend import CudaKernels
        _active = CudaKernels()
    return _active


@contextmanager
def use_kernels(backend):
    global _active
    prev = _active
    _active = backend
    try:
        yield backend
    finally:
        _active = prev
