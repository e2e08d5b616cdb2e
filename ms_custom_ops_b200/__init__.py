"""B200-native paged-KV decode operators: reshape_and_cache and paged_attention.

Drop-in for the two operators of the same names in `ms_custom_ops`
(python/ms_custom_ops/__init__.py:76 re-exports them from the plugin module):
same argument names, order, defaults, layouts, dtypes and attribute values.
Underneath: hand-written CUDA kernels for sm_100a behind a thin C ABI
(libmsco_b200.so).  There is no CPU or PyTorch fallback; importing the
operators without the built library raises.
"""
from . import _abi  # noqa: F401
from ._abi import MscoError  # noqa: F401

__all__ = ["MscoError"]
