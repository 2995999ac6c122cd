"""Mirror of ``smartkv.models``."""
from .llama_smartkv import LlamaSmartKV, LlamaSmartKVAttention, SmartKVConfig  # noqa: F401
