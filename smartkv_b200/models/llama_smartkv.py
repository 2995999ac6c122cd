"""Mirror of ``smartkv.models.llama_smartkv`` (smartkv/models/llama_smartkv.py): ``SmartKVConfig``,
``LlamaSmartKVAttention`` and ``LlamaSmartKV`` with the reference's names, arguments and attributes,
driving the B200 library.

Decode steps (one query token against a non-empty cache) go through the fused packed attention
kernel with the current token in full precision, the way the reference's fused CPU path does
(smartkv/models/llama_smartkv.py:264-305); the importance update and the reallocation trigger run
inside ``SmartKVCache.fused_decode_attention``.  Prefill (more than one query token) computes
ordinary causal attention over the prompt with torch, hands the probabilities to
``update_attention`` with the ids of the keys, and bulk-stores the prompt, as the reference does
(:392-427).  Projections, rotary embedding and everything outside attention stay with the wrapped
Hugging Face module.

With one batch row the cache is ``SmartKVCache``; like the reference it keeps ONE sequence (:457-466).
With more than one row (or ``SmartKVConfig.batched=True``) the wrapper builds a ``BatchedSmartKVCache``
instead: every batch row is an independent sequence of the same packed store, and a decode step costs two
kernel launches per layer for the whole batch.  ``batched=False`` restores the reference's behaviour for a
batch (every row attends to row 0's cache).
"""
from __future__ import annotations

import warnings
import weakref
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..core.batched_cache import BatchedSmartKVCache
from ..core.cache import SmartKVCache


@dataclass
class SmartKVConfig:
    """smartkv/models/llama_smartkv.py:39-57, same fields and defaults (``device`` defaults to "cpu" there
    too; this library has no CPU path, so a cache is only built with device="cuda").  The three fields after
    ``forecast_lr`` have no counterpart in the reference: ``batched`` (None: a batch of more than one row gets
    a multi-sequence cache), ``max_tokens`` (capacity per sequence of that cache) and ``key_attribution``
    ("keys": attention mass is credited to the key it falls on; "wrapper": what the reference's wrapper does
    in a decode step, see BatchedSmartKVCache)."""
    enabled: bool = False
    memory_budget: float = 0.5
    decay: float = 0.9
    realloc_freq: int = 16
    available_bits: Optional[List[int]] = None
    device: str = "cpu"
    enable_forecast: bool = False
    forecast_history: int = 2048
    forecast_update_interval: int = 32
    forecast_blend: float = 0.5
    forecast_lr: float = 0.05
    batched: Optional[bool] = None
    max_tokens: int = 4096
    key_attribution: str = "keys"

    def __post_init__(self):
        if self.available_bits is None:
            self.available_bits = [2, 3, 4, 8]


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


class LlamaSmartKVAttention(nn.Module):
    """Wraps one Hugging Face Llama attention module (smartkv/models/llama_smartkv.py:60-439)."""

    def __init__(self, original_attention: nn.Module, layer_idx: int, smartkv_config: SmartKVConfig):
        super().__init__()
        self.original_attention = original_attention
        self.layer_idx = layer_idx
        self.smartkv_config = smartkv_config
        cfg = getattr(original_attention, "config", None)
        self.q_proj, self.k_proj = original_attention.q_proj, original_attention.k_proj
        self.v_proj, self.o_proj = original_attention.v_proj, original_attention.o_proj
        self.head_dim = getattr(original_attention, "head_dim", None) or (cfg.hidden_size // cfg.num_attention_heads)
        self.num_heads = getattr(original_attention, "num_heads", None) or self.q_proj.out_features // self.head_dim
        self.num_key_value_heads = (getattr(original_attention, "num_key_value_heads", None)
                                    or self.k_proj.out_features // self.head_dim)
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.hidden_size = self.q_proj.in_features
        self.rotary_emb = getattr(original_attention, "rotary_emb", None)
        self.smartkv_cache: Optional[SmartKVCache] = None
        self.use_smartkv = False
        self.use_fused_cpu = False
        self.use_fused_gpu = True
        self.token_counter = 0

    def enable_smartkv(self, shared_cache: SmartKVCache):
        self.smartkv_cache = shared_cache
        self.use_smartkv = True

    def disable_smartkv(self):
        self.use_smartkv = False

    def _apply_rotary_pos_emb(self, q, k, position_embeddings=None, position_ids=None):
        if position_embeddings is not None:
            cos, sin = position_embeddings
        elif self.rotary_emb is not None:
            cos, sin = self.rotary_emb(k, position_ids)
        else:
            raise ValueError("no rotary embedding available: pass position_embeddings or set rotary_emb")
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
        return (q * cos) + (_rotate_half(q) * sin), (k * cos) + (_rotate_half(k) * sin)

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.LongTensor] = None, past_key_value: Any = None,
                output_attentions: bool = False, use_cache: bool = False, token_ids: Optional[List[int]] = None,
                position_embeddings: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                cache_position: Optional[torch.LongTensor] = None, **kwargs):
        if not self.use_smartkv or self.smartkv_cache is None:
            if past_key_value is not None:
                kwargs.setdefault("past_key_values", past_key_value)
            return self.original_attention(hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                                           position_embeddings=position_embeddings, cache_position=cache_position,
                                           **kwargs)
        kwargs.pop("past_key_values", None)
        bsz, q_len, _ = hidden_states.size()
        owner = getattr(self, "_owner", None)
        if owner is not None:
            owner()._select_cache(bsz)
        cache = self.smartkv_cache
        if isinstance(cache, BatchedSmartKVCache):
            return self._forward_batched(cache, hidden_states, position_embeddings, position_ids, output_attentions)
        q = self.q_proj(hidden_states).view(bsz, q_len, self.num_heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(hidden_states).view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(hidden_states).view(bsz, q_len, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        q, k = self._apply_rotary_pos_emb(q, k, position_embeddings=position_embeddings, position_ids=position_ids)
        if token_ids is None:
            token_ids = list(range(self.token_counter, self.token_counter + q_len))
            self.token_counter += q_len
        token_ids = [int(t) for t in token_ids]
        past_ids = sorted(cache._layer_tokens[self.layer_idx])
        attn_weights = None
        if q_len == 1 and past_ids and not output_attentions and self.use_fused_gpu:
            rows = []
            for b in range(bsz):
                rows.append(cache.fused_decode_attention(self.layer_idx, q[b, :, 0], k[b, :, 0], v[b, :, 0], token_ids[0],
                                                         update_importance=(b == 0)))
            attn_output = torch.stack(rows).to(hidden_states.dtype).reshape(bsz, 1, self.num_heads * self.head_dim)
        else:
            key_states, value_states = k, v
            if past_ids:
                pk, pv = cache.retrieve_all(self.layer_idx)          # [n, Hkv, D] fp32, ascending token id
                pk = pk.to(k.dtype).permute(1, 0, 2).unsqueeze(0).expand(bsz, -1, -1, -1)
                pv = pv.to(v.dtype).permute(1, 0, 2).unsqueeze(0).expand(bsz, -1, -1, -1)
                key_states, value_states = torch.cat([pk, k], dim=2), torch.cat([pv, v], dim=2)
            if self.num_key_value_groups > 1:
                key_states = key_states.repeat_interleave(self.num_key_value_groups, dim=1)
                value_states = value_states.repeat_interleave(self.num_key_value_groups, dim=1)
            scores = torch.matmul(q, key_states.transpose(2, 3)) / (self.head_dim ** 0.5)
            kv_len, past_len = scores.shape[-1], len(past_ids)
            qi = torch.arange(q_len, device=scores.device)[:, None] + past_len
            ki = torch.arange(kv_len, device=scores.device)[None, :]
            scores = scores.masked_fill(ki > qi, float("-inf"))
            attn_weights = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
            attn_output = torch.matmul(attn_weights, value_states).transpose(1, 2).contiguous()
            attn_output = attn_output.reshape(bsz, q_len, self.num_heads * self.head_dim)
            cache.update_attention(self.layer_idx, attn_weights[:1], past_ids + token_ids)   # ids of the keys
        if bsz > 1 and not getattr(self, "_smartkv_multi_batch_warned", False):
            warnings.warn("SmartKV cache currently stores KV from the first batch item only; ensure sequences are "
                          "aligned when using multi-batch fused generation.", UserWarning)
            self._smartkv_multi_batch_warned = True
        cache.quantize_and_store_batch(self.layer_idx, token_ids, k[0].transpose(0, 1).contiguous(),
                                       v[0].transpose(0, 1).contiguous())
        attn_output = self.o_proj(attn_output)
        return (attn_output, attn_weights) if output_attentions else (attn_output, None)


    def _forward_batched(self, cache: BatchedSmartKVCache, hidden_states, position_embeddings, position_ids,
                         output_attentions):
        """Every batch row is its own sequence of ``cache``.  One query token: the fused packed kernels for the
        whole batch.  More: causal attention over the unquantised prompt with torch, whose probabilities feed
        the importance update before the prompt is stored (smartkv/models/llama_smartkv.py:392-427)."""
        bsz, q_len, _ = hidden_states.size()
        H, Hkv, D = self.num_heads, self.num_key_value_heads, self.head_dim
        q = self.q_proj(hidden_states).view(bsz, q_len, H, D).transpose(1, 2)
        k = self.k_proj(hidden_states).view(bsz, q_len, Hkv, D).transpose(1, 2)
        v = self.v_proj(hidden_states).view(bsz, q_len, Hkv, D).transpose(1, 2)
        q, k = self._apply_rotary_pos_emb(q, k, position_embeddings=position_embeddings, position_ids=position_ids)
        self.token_counter += q_len
        attn_weights = None
        if q_len == 1:
            out = cache.decode_layer(self.layer_idx, q[:, :, 0], k[:, :, 0], v[:, :, 0])
            attn_output = out.to(hidden_states.dtype).reshape(bsz, 1, H * D)
        elif q.dtype == torch.float16 and not output_attentions and D in (64, 128):
            # the prompt-pass kernel: attention output and per-key mass without the [B, Hq, n, n] probabilities
            from ..prefill import causal_prefill_attention
            w = cache.prefill_head_weights(q_len)
            out, mass = causal_prefill_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), w)
            attn_output = out.reshape(bsz, q_len, H * D)
            cache.prefill_layer(self.layer_idx, k.transpose(1, 2), v.transpose(1, 2), key_mass=mass)
        else:
            kk = k.repeat_interleave(self.num_key_value_groups, dim=1)
            vv = v.repeat_interleave(self.num_key_value_groups, dim=1)
            scores = torch.matmul(q, kk.transpose(2, 3)) / (D ** 0.5)
            idx = torch.arange(q_len, device=scores.device)
            scores = scores.masked_fill(idx[None, :] > idx[:, None], float("-inf"))
            probs = torch.softmax(scores, dim=-1, dtype=torch.float32)
            attn_weights = probs.to(q.dtype)
            attn_output = torch.matmul(attn_weights, vv).transpose(1, 2).reshape(bsz, q_len, H * D)
            cache.prefill_layer(self.layer_idx, k.transpose(1, 2), v.transpose(1, 2), attn_weights.float())
        attn_output = self.o_proj(attn_output)
        return (attn_output, attn_weights) if output_attentions else (attn_output, None)


class LlamaSmartKV(nn.Module):
    """Wraps a Hugging Face Llama model (smartkv/models/llama_smartkv.py:596-792)."""

    def __init__(self, model: nn.Module, smartkv_config: Optional[SmartKVConfig] = None):
        super().__init__()
        self.model = model
        self.smartkv_config = smartkv_config or SmartKVConfig()
        self.smartkv_cache: Optional[SmartKVCache] = None
        self.use_fused_cpu = False
        self.use_fused_gpu = True
        if self.smartkv_config.enabled:
            self._replace_attention_layers()

    def _layers(self):
        if not (hasattr(self.model, "model") and hasattr(self.model.model, "layers")):
            raise ValueError("Model structure not compatible with SmartKV")
        return self.model.model.layers

    def _replace_attention_layers(self):
        layers = self._layers()
        cfg = getattr(self.model, "config", None)
        first = layers[0].self_attn
        if isinstance(first, LlamaSmartKVAttention):
            first = first.original_attention
        head_dim = getattr(first, "head_dim", None) or (cfg.hidden_size // cfg.num_attention_heads)
        num_kv = getattr(first, "num_key_value_heads", None) or first.k_proj.out_features // head_dim
        num_q = first.q_proj.out_features // head_dim
        special = [t for t in (getattr(cfg, "bos_token_id", None), getattr(cfg, "eos_token_id", None),
                               getattr(cfg, "pad_token_id", None)) if isinstance(t, int)] if cfg is not None else []
        c = self.smartkv_config
        self._geometry = dict(num_layers=len(layers), num_heads=num_kv, head_dim=head_dim, num_query_heads=num_q,
                              special_token_ids=special)
        self._batched_cache = None
        self._single_cache = SmartKVCache(
            num_layers=len(layers), num_heads=num_kv, head_dim=head_dim, memory_budget=c.memory_budget, decay=c.decay,
            realloc_freq=c.realloc_freq, available_bits=c.available_bits, device=c.device, special_token_ids=special,
            enable_forecast=c.enable_forecast, forecast_history=c.forecast_history,
            forecast_update_interval=c.forecast_update_interval, forecast_blend=c.forecast_blend,
            forecast_lr=c.forecast_lr, num_query_heads=num_q, max_tokens=c.max_tokens)
        self.smartkv_cache = self._single_cache
        shared_rotary = getattr(self.model.model, "rotary_emb", None)
        for idx, layer in enumerate(layers):
            if not hasattr(layer, "self_attn"):
                continue
            original = layer.self_attn
            if isinstance(original, LlamaSmartKVAttention):
                original = original.original_attention
            attn = LlamaSmartKVAttention(original, idx, c)
            attn.use_fused_cpu, attn.use_fused_gpu = self.use_fused_cpu, self.use_fused_gpu
            if attn.rotary_emb is None and shared_rotary is not None:
                attn.rotary_emb = shared_rotary
            attn.enable_smartkv(self.smartkv_cache)
            object.__setattr__(attn, "_owner", weakref.ref(self))      # not a submodule: no reference cycle in nn.Module
            layer.self_attn = attn

    def _select_cache(self, batch_size: int):
        """The cache for a forward pass over ``batch_size`` rows: the multi-sequence one when asked for (or,
        by default, whenever there is more than one row), built on first use."""
        c = self.smartkv_config
        batched = c.batched if c.batched is not None else batch_size > 1
        want = self._single_cache
        if batched:
            bc = self._batched_cache
            if bc is None or bc.batch_size != batch_size:
                g = self._geometry
                bc = BatchedSmartKVCache(
                    num_layers=g["num_layers"], num_heads=g["num_heads"], head_dim=g["head_dim"],
                    num_query_heads=g["num_query_heads"], batch_size=batch_size, max_tokens=c.max_tokens,
                    memory_budget=c.memory_budget, decay=c.decay, realloc_freq=c.realloc_freq,
                    available_bits=c.available_bits, device=c.device, special_token_ids=g["special_token_ids"],
                    key_attribution=c.key_attribution)
                self._batched_cache = bc
            want = bc
        if want is not self.smartkv_cache:
            self.smartkv_cache = want
            for layer in self._layers():
                if isinstance(layer.self_attn, LlamaSmartKVAttention):
                    layer.self_attn.smartkv_cache = want

    def enable_smartkv(self, memory_budget: Optional[float] = None, decay: Optional[float] = None,
                       realloc_freq: Optional[int] = None):
        if memory_budget is not None:
            self.smartkv_config.memory_budget = memory_budget
        if decay is not None:
            self.smartkv_config.decay = decay
        if realloc_freq is not None:
            self.smartkv_config.realloc_freq = realloc_freq
        self.smartkv_config.enabled = True
        self._replace_attention_layers()

    def disable_smartkv(self):
        self.smartkv_config.enabled = False
        for layer in self._layers():
            if isinstance(layer.self_attn, LlamaSmartKVAttention):
                layer.self_attn = layer.self_attn.original_attention

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)

    def generate(self, *args, **kwargs):
        return self.model.generate(*args, **kwargs)

    def get_smartkv_stats(self) -> Dict[str, Any]:
        return {} if self.smartkv_cache is None else self.smartkv_cache.get_memory_stats()

    def reset_cache(self):
        for cache in (getattr(self, "_single_cache", None), getattr(self, "_batched_cache", None)):
            if cache is not None:
                cache.clear()
        for layer in self._layers():
            if hasattr(layer.self_attn, "token_counter"):
                layer.self_attn.token_counter = 0

    def set_use_fused_cpu(self, enabled: bool) -> None:
        """Kept for interface parity; there is no CPU path, the flag is only recorded."""
        self.use_fused_cpu = enabled
        for layer in self._layers():
            if isinstance(layer.self_attn, LlamaSmartKVAttention):
                layer.self_attn.use_fused_cpu = enabled

    def set_use_fused_gpu(self, enabled: bool) -> None:
        """False sends decode steps through the dequantise-and-concatenate path used for prefill."""
        self.use_fused_gpu = enabled
        for layer in self._layers():
            if isinstance(layer.self_attn, LlamaSmartKVAttention):
                layer.self_attn.use_fused_gpu = enabled

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.model, name)
