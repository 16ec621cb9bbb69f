"""deers_b200: B200 (sm_100a) causal self-attention for deers behind a C ABI.

``deers_b200._lib`` binds ``libdeers_b200.so`` (built in-tree by
``python -m deers_b200.build``); ``deers_b200.ops`` mirrors the deers operator
interface (``TensorOp``: forward / backward / dependencies) on top of it.  There
is no CPU or PyTorch fallback: if the library is missing or the device is not a
B200 the calls raise.
"""
from . import _lib  # noqa: F401
from .errors import CudaError, DeersError, DeviceMismatch, DTypeMismatch, LayoutMismatch  # noqa: F401

__all__ = ["_lib", "ops", "shard", "DeersError", "CudaError", "DeviceMismatch", "DTypeMismatch",
           "LayoutMismatch"]
