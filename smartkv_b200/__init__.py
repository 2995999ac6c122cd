"""smartkv_b200: B200 (sm_100a) implementation of SmartKV's quantized-KV decode path.

The compute lives in ``libsmartkv_b200.so`` (hand-written CUDA, C ABI declared in
``include/smartkv_b200.h``); this package is the host-side mirror of the
reference's Python interface for that path (``smartkv.core``, ``smartkv.kernels``,
``smartkv.models`` keep their names under ``smartkv_b200``).  There is no CPU fallback.
"""
from ._lib import SmartKVLibraryError, lib  # noqa: F401

__version__ = "0.1.0"


def alias_as_smartkv() -> None:
    """Registers this package under the reference's import name, so that code written against
    ``smartkv`` (``from smartkv.models.llama_smartkv import LlamaSmartKV, SmartKVConfig``,
    ``from smartkv.core.cache import SmartKVCache``, ``from smartkv.kernels import quantized_attention`` ...)
    runs on the B200 library unchanged.  Opt-in, and refused when another ``smartkv`` is already imported: the two
    must never be mixed up silently."""
    import importlib
    import sys
    other = sys.modules.get("smartkv")
    this = sys.modules[__name__]
    if other is not None and other is not this:
        raise ImportError(f"a different 'smartkv' is already imported from {getattr(other, '__file__', '?')}")
    sys.modules["smartkv"] = this
    for sub in ("core", "core.cache", "core.importance", "core._quant_cuda", "core.batched_cache", "kernels",
                "kernels.bit_packing", "models", "models.llama_smartkv"):
        sys.modules[f"smartkv.{sub}"] = importlib.import_module(f"{__name__}.{sub}")


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
