"""smartkv_b200: B200 (sm_100a) implementation of SmartKV's quantized-KV decode path.

The compute lives in ``libsmartkv_b200.so`` (hand-written CUDA, C ABI declared in
``include/smartkv_b200.h``); this package is the host-side mirror of the
reference's Python interface for that path.  There is no CPU fallback.
"""
from ._lib import SmartKVLibraryError, lib  # noqa: F401

__version__ = "0.1.0"
