"""Mirror of ``smartkv.baselines.uniform_quant`` (smartkv/baselines/uniform_quant.py): the uniform INT8 / INT4
comparison cache, kept in the packed store and attended by the packed decode kernels.

Same quantiser as the reference's (one scale per token tensor, smartkv/core/quantizers.py:69-91, :114-133), so
``retrieve`` / ``retrieve_all`` return bit-identical values.  ``bits=16`` (the reference's FP16 pass-through) has no
packed representation and raises."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Sequence

import torch

from ._packed import PackedBaselineCache, quantize_per_tensor


@dataclass
class UniformQuantConfig:
    """smartkv/baselines/uniform_quant.py:15-21."""
    bits: int = 8
    enabled: bool = True
    device: str = "cpu"


class UniformQuantCache(PackedBaselineCache):
    """smartkv/baselines/uniform_quant.py:24-245."""

    def __init__(self, num_layers: int, num_heads: int, head_dim: int, bits: int = 8, device: str = "cuda",
                 max_tokens: int = 4096, num_query_heads: Optional[int] = None):
        if bits == 16:
            raise NotImplementedError("the FP16 pass-through cache has no packed representation; use the model's own cache")
        if bits not in (4, 8):
            raise ValueError(f"Unsupported bits: {bits}. Use 4, 8, or 16.")
        self.bits = bits
        super().__init__(num_layers, num_heads, head_dim, bits, device, max_tokens, num_query_heads)

    def quantize_and_store(self, layer_idx: int, token_id: int, k_vec: torch.Tensor, v_vec: torch.Tensor) -> None:
        """k_vec, v_vec [num_heads, head_dim] (smartkv/baselines/uniform_quant.py:73-110)."""
        self.quantize_and_store_batch(layer_idx, [int(token_id)], k_vec.unsqueeze(0), v_vec.unsqueeze(0))

    def quantize_and_store_batch(self, layer_idx: int, token_ids: Sequence[int], k: torch.Tensor, v: torch.Tensor) -> None:
        """Several tokens at once: k, v [n, num_heads, head_dim] (each token quantised on its own)."""
        k, v = k.to(self._dev), v.to(self._dev)
        kq, ks = quantize_per_tensor(k, self.bits)
        vq, vs = quantize_per_tensor(v, self.bits)
        H = self.num_heads
        self._store_codes(layer_idx, token_ids, kq, ks[:, None].expand(-1, H).contiguous(), vq,
                          vs[:, None].expand(-1, H).contiguous())

    def get_memory_stats(self) -> Dict[str, Any]:
        """smartkv/baselines/uniform_quant.py:192-220 (payload bytes only, as there)."""
        bytes_per_token = self.num_heads * self.head_dim * self.bits / 8 * 2
        fp16_bytes = self.num_heads * self.head_dim * 2 * 2
        return {"bits": self.bits, "num_tokens": len(self), "num_cache_entries": self.num_cache_entries,
                "total_tokens_stored": self.total_tokens_stored, "memory_ratio": bytes_per_token / fp16_bytes,
                "quantizer": f"int{self.bits}"}

    def __repr__(self) -> str:
        return f"UniformQuantCache(layers={self.num_layers}, bits={self.bits}, cached={self.num_cache_entries})"


def create_uniform_baseline(bits: int = 8, name: Optional[str] = None) -> Dict[str, Any]:
    """smartkv/baselines/uniform_quant.py:397-422."""
    if name is None:
        name = "FP16-Baseline" if bits == 16 else f"Uniform-INT{bits}"
    return {"name": name, "bits": bits, "type": "uniform", "cache_class": UniformQuantCache,
            "config": UniformQuantConfig(bits=bits)}
