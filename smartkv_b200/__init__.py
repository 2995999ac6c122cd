"""smartkv_b200: B200 (sm_100a) implementation of SmartKV's quantized-KV decode path.

The compute lives in ``libsmartkv_b200.so`` (hand-written CUDA, C ABI declared in
``include/smartkv_b200.h``); this package is the host-side mirror of the
reference's Python interface for that path (``smartkv.core``, ``smartkv.kernels``,
``smartkv.models`` keep their names under ``smartkv_b200``).  There is no CPU fallback.
"""
from ._lib import SmartKVLibraryError, lib  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    # the reference exports these from its top-level package (smartkv/__init__.py); resolved lazily so
    # that importing the package does not pull in torch.nn or transformers
    if name == "SmartKVCache":
        from .core.cache import SmartKVCache
        return SmartKVCache
    if name == "BatchedSmartKVCache":
        from .core.batched_cache import BatchedSmartKVCache
        return BatchedSmartKVCache
    if name in ("SmartKVConfig", "LlamaSmartKV", "LlamaSmartKVAttention"):
        from .models import llama_smartkv
        return getattr(llama_smartkv, name)
    if name == "PackedKVStore":
        from .store import PackedKVStore
        return PackedKVStore
    raise AttributeError(f"module 'smartkv_b200' has no attribute {name!r}")
