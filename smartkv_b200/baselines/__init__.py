"""Mirror of ``smartkv.baselines``: the comparison caches, on the packed store and its decode kernels."""
from .kivi import KIVICache, KIVIConfig, create_kivi_baseline  # noqa: F401
from .uniform_quant import UniformQuantCache, UniformQuantConfig, create_uniform_baseline  # noqa: F401
