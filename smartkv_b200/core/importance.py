"""Mirror of ``smartkv.core.importance.ImportanceTracker`` (smartkv/core/importance.py:9-250):
the dict-keyed view of token importance that callers and tests of the reference read.

The decode path itself never goes through these dicts: the attention kernel leaves logits, the
importance kernel folds the per-key mass into device arrays in storage order, and
``SmartKVCache`` pulls what accumulated there into this tracker whenever somebody asks.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch


class ImportanceTracker:
    def __init__(self, num_layers: int, decay: float = 0.9, device: str = "cuda"):
        self.num_layers = num_layers
        self.decay = decay
        self.device = device
        self.token_importance: Dict[int, float] = {}            # token id -> cumulative score
        self.layer_importance: Dict[Tuple[int, int], float] = {}  # (layer, token id) -> EMA
        self.importance_history: List[Dict[int, float]] = []
        self.update_count = 0

    def update_attention(self, layer_idx: int, attention_weights: Optional[torch.Tensor], token_ids) -> None:
        """attention_weights [batch, heads, queries, keys]; token_ids: ids of the keys
        (smartkv/core/importance.py:44-101)."""
        if attention_weights is None:
            return
        w = attention_weights
        if w.ndim != 4:
            raise ValueError(f"attention_weights must be [batch, heads, queries, keys]; got {tuple(w.shape)}")
        key_importance = w.detach().float().sum(dim=(0, 1, 2)).tolist()
        ids = [int(t) for t in (token_ids.tolist() if isinstance(token_ids, torch.Tensor) else token_ids)]
        for i, tid in enumerate(ids):
            if i >= len(key_importance):
                break
            self.add_mass(layer_idx, tid, float(key_importance[i]))
        self.update_count += 1

    def add_mass(self, layer_idx: int, token_id: int, score: float) -> None:
        key = (layer_idx, token_id)
        if key in self.layer_importance:
            self.layer_importance[key] = self.decay * self.layer_importance[key] + (1 - self.decay) * score
        else:
            self.layer_importance[key] = score
        if token_id in self.token_importance:
            self.token_importance[token_id] += score
        else:
            self.token_importance[token_id] = score

    def get_importance(self, token_id: int) -> float:
        return self.token_importance.get(token_id, 0.0)

    def get_layer_importance(self, layer_idx: int, token_id: int) -> float:
        return self.layer_importance.get((layer_idx, token_id), 0.0)

    def get_top_k_tokens(self, k: int) -> List[Tuple[int, float]]:
        return sorted(self.token_importance.items(), key=lambda x: x[1], reverse=True)[:k]

    def get_bottom_k_tokens(self, k: int) -> List[Tuple[int, float]]:
        return sorted(self.token_importance.items(), key=lambda x: x[1])[:k]

    def get_importance_statistics(self) -> Dict[str, float]:
        if not self.token_importance:
            return {"mean": 0.0, "std": 0.0, "min": 0.0, "max": 0.0, "total": 0.0, "num_tokens": 0}
        t = torch.tensor(list(self.token_importance.values()), dtype=torch.float64)
        return {"mean": float(t.mean()), "std": float(t.std(unbiased=False)), "min": float(t.min()),
                "max": float(t.max()), "total": float(t.sum()), "num_tokens": int(t.numel())}

    def reset(self) -> None:
        self.token_importance.clear()
        self.layer_importance.clear()
        self.importance_history.clear()
        self.update_count = 0
