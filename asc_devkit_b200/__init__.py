"""B200 (sm_100a) implementation of the Ascend C quantized-inference operators.

``ops`` mirrors the reference's operator interface on CUDA tensors; ``_lib`` is the raw ctypes view of the
C ABI declared in ``include/ascq.h``; ``build`` compiles ``libascq.so`` in-tree with nvcc."""
from . import _lib  # noqa: F401
from ._lib import AscqError  # noqa: F401

__all__ = ["_lib", "AscqError"]
