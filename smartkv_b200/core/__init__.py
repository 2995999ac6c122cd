"""Mirror of ``smartkv.core``: the cache and the quantiser entry points, over the B200 library."""
from .cache import SmartKVCache  # noqa: F401
from .batched_cache import BatchedSmartKVCache  # noqa: F401
