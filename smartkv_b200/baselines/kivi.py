"""Mirror of ``smartkv.baselines.kivi`` (smartkv/baselines/kivi.py:30-336): keys and values at different
widths (2-bit keys, 4-bit values by default), one scale per token tensor, kept in the packed store.

Keys and values of a token share one bucket of the packed store, so both are packed at the wider of the two
widths; the codes themselves are those of the narrower quantiser, so ``retrieve`` returns exactly what the
reference returns and ``get_memory_stats`` reports the reference's accounting (key_bits + value_bits), not the
bytes of this layout.

``per_channel_keys=True`` (the reference's default: every channel of a key gets its own scale across the
heads, kivi.py:130-168) cannot be expressed in rows that carry one scale per (token, head), which is what the
packed kernels read; it raises.  Construct with ``per_channel_keys=False``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Sequence

import torch

from ._packed import PackedBaselineCache, quantize_per_tensor


@dataclass
class KIVIConfig:
    """smartkv/baselines/kivi.py:20-27."""
    key_bits: int = 2
    value_bits: int = 4
    enabled: bool = True
    device: str = "cpu"
    per_channel_keys: bool = True


class KIVICache(PackedBaselineCache):
    def __init__(self, num_layers: int, num_heads: int, head_dim: int, key_bits: int = 2, value_bits: int = 4,
                 per_channel_keys: bool = True, device: str = "cuda", max_tokens: int = 4096,
                 num_query_heads: Optional[int] = None):
        if key_bits not in (2, 4):
            raise ValueError(f"Unsupported key_bits: {key_bits}")
        if value_bits not in (2, 4):
            raise ValueError(f"Unsupported value_bits: {value_bits}")
        if per_channel_keys:
            raise NotImplementedError(
                "per-channel key scales do not fit rows with one scale per (token, head), which the packed decode "
                "kernels read; construct KIVICache(..., per_channel_keys=False)")
        self.key_bits, self.value_bits, self.per_channel_keys = key_bits, value_bits, False
        super().__init__(num_layers, num_heads, head_dim, max(key_bits, value_bits), device, max_tokens, num_query_heads)

    def quantize_and_store(self, layer_idx: int, token_id: int, k_vec: torch.Tensor, v_vec: torch.Tensor) -> None:
        """k_vec, v_vec [num_heads, head_dim] (smartkv/baselines/kivi.py:91-128)."""
        self.quantize_and_store_batch(layer_idx, [int(token_id)], k_vec.unsqueeze(0), v_vec.unsqueeze(0))

    def quantize_and_store_batch(self, layer_idx: int, token_ids: Sequence[int], k: torch.Tensor, v: torch.Tensor) -> None:
        k, v = k.to(self._dev), v.to(self._dev)
        kq, ks = quantize_per_tensor(k, self.key_bits)
        vq, vs = quantize_per_tensor(v, self.value_bits)
        H = self.num_heads
        self._store_codes(layer_idx, token_ids, kq, ks[:, None].expand(-1, H).contiguous(), vq,
                          vs[:, None].expand(-1, H).contiguous())

    def get_memory_stats(self) -> Dict[str, Any]:
        """smartkv/baselines/kivi.py:282-312."""
        key_bytes = self.num_heads * self.head_dim * self.key_bits / 8
        value_bytes = self.num_heads * self.head_dim * self.value_bits / 8
        fp16_bytes = self.num_heads * self.head_dim * 2 * 2
        return {"key_bits": self.key_bits, "value_bits": self.value_bits, "num_tokens": len(self),
                "num_cache_entries": self.num_cache_entries, "total_tokens_stored": self.total_tokens_stored,
                "memory_ratio": (key_bytes + value_bytes) / fp16_bytes, "per_channel_keys": self.per_channel_keys,
                "quantizer": "kivi"}

    def __repr__(self) -> str:
        return (f"KIVICache(layers={self.num_layers}, key_bits={self.key_bits}, value_bits={self.value_bits}, "
                f"cached={self.num_cache_entries})")


def create_kivi_baseline(key_bits: int = 2, value_bits: int = 4, name: Optional[str] = None) -> Dict[str, Any]:
    """smartkv/baselines/kivi.py:494-521."""
    return {"name": name or f"KIVI-K{key_bits}V{value_bits}", "key_bits": key_bits, "value_bits": value_bits, "type": "kivi",
            "cache_class": KIVICache, "config": KIVIConfig(key_bits=key_bits, value_bits=value_bits, per_channel_keys=False)}
