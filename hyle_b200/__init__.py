"""hyle_b200: B200 (sm_100a) kernels for HYLE's elementwise, broadcast and reduction operators.

``hyle_b200.abi``   ctypes binding of the C ABI (include/hyle_b200.h)
``hyle_b200.ops``   the operators on torch CUDA tensors (device memory and streams only)
``hyle_b200.build`` in-tree build of libhyle_b200.so
"""
from . import abi  # noqa: F401

__all__ = ["abi"]
