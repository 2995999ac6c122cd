"""Mirror of ``smartkv.core.cache.SmartKVCache`` (smartkv/core/cache.py:34-1705) over the packed
device store: the same constructor arguments, methods, return layouts and public attributes, with
every numeric step done by ``libsmartkv_b200.so``.

What differs from the reference, on purpose:
  * CUDA only.  ``device="cpu"`` raises; there is no INT8 / CPU storage mode, so ``use_packing`` is
    always True and the memory accounting is the packed one.
  * One sequence per cache, like the reference (it stores batch row 0 only,
    smartkv/models/llama_smartkv.py:457-466).  Batched decode uses ``PackedKVStore`` directly.
  * A token becomes visible to attention once every layer has stored it, and a reallocation that
    falls due while some layer still lacks the newest token is applied as soon as all layers have it
    (the reference requantises layer by layer in the middle of a step).
  * ``enable_forecast`` runs the reference's predictor on the host (``core/forecast.py``); with it every
    fused decode step pulls the device importance of the step's token (a synchronisation the default path
    does not have).
  * Capacity is ``max_tokens`` (grown by doubling when exceeded), not an amortised ``torch.cat``.
"""
from __future__ import annotations

import ctypes
import math
import os
import warnings
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from .. import _lib
from .._lib import BITS_TO_BUCKET, BUCKET_BITS, NUM_BUCKETS, StoreDesc, check, ptr
from ..kernels.bit_packing import compute_packed_size  # noqa: F401  (re-exported like the reference, cache.py:30)
from ..store import PackedKVStore, round_up
from .importance import ImportanceTracker


def compute_minimum_budget(num_heads: int = 8, head_dim: int = 128, scale_dtype: str = "fp32",
                           use_packing: bool = False) -> float:
    """smartkv/core/allocation.py:401-441 (counts four scale slots per head)."""
    scale_bits = 32 if scale_dtype == "fp32" else 16
    payload_bits = 2 * num_heads * head_dim * (2 if use_packing else 8)
    return (payload_bits + 4 * num_heads * scale_bits) / (2 * num_heads * head_dim * 16)


def compute_memory_usage(allocation: Dict[int, int], fp16_baseline: bool = True, num_heads: Optional[int] = None,
                         head_dim: Optional[int] = None, scale_dtype: str = "fp32",
                         use_packing: bool = False) -> Dict[str, Any]:
    """smartkv/core/allocation.py:444-531."""
    mode = "packed" if use_packing else "int8"
    if not allocation:
        return {"total_bits": 0, "total_bits_with_scales": 0, "avg_bits": 0.0, "memory_ratio": 0.0,
                "memory_ratio_true": 0.0, "num_tokens": 0, "scale_overhead_pct": 0.0, "storage_mode": mode,
                "scale_dtype": scale_dtype}
    n = len(allocation)
    sbits = 32 if scale_dtype == "fp32" else 16
    if num_heads is None or head_dim is None:
        theoretical = sum(b * 2 for b in allocation.values())
        actual = theoretical if use_packing else n * 2 * 8
        s_theory = s_actual = 0
        fp16_bits = n * 32 if fp16_baseline else n
    else:
        elements = 2 * num_heads * head_dim
        theoretical = sum(b * elements for b in allocation.values())
        actual = theoretical if use_packing else n * elements * 8
        s_theory = n * 4 * num_heads * sbits
        s_actual = n * 2 * num_heads * sbits
        fp16_bits = n * elements * 16 if fp16_baseline else n
    total_theory, total_actual = theoretical + s_theory, actual + s_actual
    return {
        "total_bits": total_theory, "total_bits_actual": total_actual, "total_bits_with_scales": total_actual,
        "payload_bits": actual, "scale_bits": s_actual, "avg_bits": sum(allocation.values()) / n,
        "memory_ratio": (total_theory / fp16_bits if fp16_bits > 0 else 0.0) if fp16_baseline else 1.0,
        "memory_ratio_true": (total_actual / fp16_bits if fp16_bits > 0 else 0.0) if fp16_baseline else 1.0,
        "num_tokens": n, "scale_overhead_pct": (s_actual / total_actual * 100) if total_actual > 0 else 0.0,
        "storage_mode": mode, "scale_dtype": scale_dtype,
    }


class SmartKVCache:
    def __init__(self, num_layers: int, num_heads: int, head_dim: int, memory_budget: float = 0.5, decay: float = 0.9,
                 realloc_freq: int = 16, available_bits: Sequence[int] = (2, 3, 4, 8), device: str = "cuda",
                 special_token_ids: Optional[Sequence[int]] = None, use_bit_packing: bool = True,
                 enable_forecast: bool = False, forecast_history: int = 2048, forecast_update_interval: int = 32,
                 forecast_blend: float = 0.5, forecast_lr: float = 0.05, utility_alpha: float = 0.5,
                 importance_floor: float = 1e-6, hysteresis_rank_threshold: float = 0.05,
                 hysteresis_intervals: int = 2, use_bucketed_layout: bool = False,
                 high_precision_fraction: float = 0.02, high_precision_boost: float = 1.5,
                 min_high_precision_tokens: int = 0, max_tokens: int = 4096, num_query_heads: Optional[int] = None):
        dev = torch.device(device)
        if dev.type != "cuda":
            raise _lib.SmartKVLibraryError("SmartKVCache on the B200 library needs a CUDA device; there is no CPU path")
        if head_dim not in (64, 128):
            raise ValueError(f"head_dim must be 64 or 128 on the B200 path; got {head_dim}")
        self.num_layers, self.num_heads, self.head_dim = num_layers, num_heads, head_dim
        self.num_query_heads = int(num_query_heads or num_heads)
        self.decay, self.realloc_freq = decay, realloc_freq
        self.available_bits = sorted(available_bits, reverse=True)
        for b in self.available_bits:
            if b not in BITS_TO_BUCKET:
                raise ValueError(f"available_bits must be drawn from 2, 3, 4, 8; got {b}")
        self.device = device
        if not use_bit_packing:
            warnings.warn("the B200 store is always bit-packed; use_bit_packing=False is ignored")
        self.use_packing = True
        self.scale_dtype = "fp32"
        # the optional importance forecast (smartkv/core/cache.py:111-133)
        self.enable_forecast = bool(enable_forecast and forecast_history > 0)
        self.forecast_history = max(1, forecast_history)
        self.forecast_update_interval = max(1, forecast_update_interval)
        self.forecast_blend = float(max(0.0, min(1.0, forecast_blend)))
        self.forecast_lr = float(max(forecast_lr, 1e-5))
        self.forecast_pending: Dict[int, Tuple[torch.Tensor, int]] = {}
        self.forecast_last_importance: Dict[int, float] = {}
        self.forecast_last_loss: Optional[float] = None
        if self.enable_forecast:
            from collections import deque
            from .forecast import ForecastPredictor
            self.forecast_feature_buffer = deque(maxlen=self.forecast_history)
            self.forecast_target_buffer = deque(maxlen=self.forecast_history)
            self.forecast_predictor = ForecastPredictor(feature_dim=6, lr=self.forecast_lr, device="cpu")
        else:
            self.forecast_feature_buffer = self.forecast_target_buffer = self.forecast_predictor = None
        self.utility_alpha = float(utility_alpha) if utility_alpha > 0 else 1.0
        self.importance_floor = float(max(importance_floor, 0.0))
        self.hysteresis_rank_threshold = float(max(hysteresis_rank_threshold, 0.0))
        self.hysteresis_intervals = max(int(hysteresis_intervals), 1)
        self.use_bucketed_layout = bool(use_bucketed_layout)
        self.min_budget = compute_minimum_budget(num_heads, head_dim, self.scale_dtype, self.use_packing)
        if memory_budget < self.min_budget:
            warnings.warn(f"memory_budget {memory_budget:.3f} is below the minimum {self.min_budget:.3f} achievable "
                          "with packed storage; clamping")
            self.memory_budget = self.min_budget
        else:
            self.memory_budget = memory_budget
        self.special_token_ids = set(special_token_ids or [])
        self.protected_tokens = set([0, 1, 2])
        self.head_importance = torch.ones(self.num_query_heads, dtype=torch.float32)
        self.head_importance_decay = 0.9
        self.recency_temperature = 512.0
        self.global_step = 0
        self.critical_token_window = 4
        self.critical_min_bits = max(self.available_bits)
        self.min_general_bits = min(self.available_bits)
        self.high_precision_fraction = float(max(0.0, min(high_precision_fraction, 0.5)))
        self.high_precision_boost = float(max(1.0, high_precision_boost))
        self.min_high_precision_tokens = int(max(0, min_high_precision_tokens))
        self.importance_tracker = ImportanceTracker(num_layers, decay=decay, device=device)
        self.precision_map: Dict[int, int] = {}
        self.k_cache: Dict[Tuple[int, int], Dict[str, Any]] = {}
        self.v_cache: Dict[Tuple[int, int], Dict[str, Any]] = {}
        self.last_seen: Dict[int, int] = {}
        self.token_counter = 0
        self.realloc_counter = 0
        self.total_tokens_stored = 0
        self._rank_state: Dict[int, Tuple[float, int]] = {}   # token id -> (percentile, streak), cache.py:423-450
        self._dev = dev
        self._max_tokens = 0
        self._alloc_ctx = None
        self._init_store(int(max_tokens))

    # ------------------------------------------------------------------ storage bookkeeping
    def _init_store(self, max_tokens: int):
        cap = round_up(max_tokens + 1, 128)
        self.store = PackedKVStore(self.num_layers, 1, self.num_heads, self.head_dim, self.num_query_heads,
                                   (cap, cap, cap, cap), device=self._dev, decay=self.decay,
                                   head_decay=self.head_importance_decay)
        self._max_tokens = cap - 1
        self._slot: Dict[int, Tuple[int, int]] = {}                      # token id -> (bucket, position)
        self._bucket_tokens: List[List[int]] = [[] for _ in range(NUM_BUCKETS)]   # token ids by position
        self._committed = [0] * NUM_BUCKETS                              # positions attention may read
        self._layers_of: Dict[int, set] = {}                             # token id -> layers that stored it
        self._layer_tokens: List[set] = [set() for _ in range(self.num_layers)]
        self._realloc_due = False
        self._dev_base = torch.zeros_like(self.store.cumulative)        # device importance already in the tracker

    def _pending_tokens(self) -> bool:
        return any(self._committed[b] < len(self._bucket_tokens[b]) for b in range(NUM_BUCKETS))

    def _advance_commits(self):
        changed = False
        for b in range(NUM_BUCKETS):
            toks = self._bucket_tokens[b]
            c = self._committed[b]
            while c < len(toks) and len(self._layers_of.get(toks[c], ())) == self.num_layers:
                c += 1
            if c != self._committed[b]:
                self._committed[b] = c
                changed = True
        if changed:
            self.store.counts.copy_(torch.tensor([self._committed], dtype=torch.int32))
            self.store._plan_valid = False
            if self._realloc_due and not self._pending_tokens():
                self._apply_allocation()

    def _assign_slot(self, token_id: int, bits: int) -> Tuple[int, int]:
        bucket = BITS_TO_BUCKET[bits]
        pos = len(self._bucket_tokens[bucket])
        if pos >= self.store.caps[bucket] - 1:
            self._grow()
            pos = len(self._bucket_tokens[bucket])
        self._bucket_tokens[bucket].append(token_id)
        self._slot[token_id] = (bucket, pos)
        self._layers_of[token_id] = set()
        return bucket, pos

    def _grow(self):
        """Doubles the capacity: a new store, every stored row copied across as codes + scales."""
        old = self.store
        old_slot, old_bucket_tokens = dict(self._slot), [list(t) for t in self._bucket_tokens]
        old_layers, old_committed = {t: set(s) for t, s in self._layers_of.items()}, list(self._committed)
        realloc_due = self._realloc_due         # a reallocation waiting for the step's token must survive the move
        self._pull_device_importance()
        self._init_store(2 * (self._max_tokens + 1))
        new = self.store
        self._slot, self._bucket_tokens, self._layers_of = old_slot, old_bucket_tokens, old_layers
        self._committed = old_committed
        for layer in range(self.num_layers):
            self._layer_tokens[layer] = {t for t, ls in old_layers.items() if layer in ls}
        dev = self._dev
        st = new._stream()
        for b in range(NUM_BUCKETS):
            n = len(old_bucket_tokens[b])
            if n == 0:
                continue
            seq = torch.zeros(n, dtype=torch.int32, device=dev)
            bk = torch.full((n,), b, dtype=torch.int32, device=dev)
            pos = torch.arange(n, dtype=torch.int32, device=dev)
            ids = torch.tensor(old_bucket_tokens[b], dtype=torch.int32, device=dev)
            new.slot_token[0, new.bucket_base[b]: new.bucket_base[b] + n] = ids
            for name in ("cumulative", "rank_pct", "rank_streak"):
                getattr(new, name)[0, new.bucket_base[b]: new.bucket_base[b] + n] = \
                    getattr(old, name)[0, old.bucket_base[b]: old.bucket_base[b] + n]
            new.layer_ema[:, 0, new.bucket_base[b]: new.bucket_base[b] + n] = \
                old.layer_ema[:, 0, old.bucket_base[b]: old.bucket_base[b] + n]
            new.touched[:, 0, new.bucket_base[b]: new.bucket_base[b] + n] = \
                old.touched[:, 0, old.bucket_base[b]: old.bucket_base[b] + n]
            kc = torch.empty((n, self.num_heads, self.head_dim), dtype=torch.int8, device=dev)
            vc = torch.empty_like(kc)
            ks = torch.empty((n, self.num_heads), dtype=torch.float32, device=dev)
            vs = torch.empty_like(ks)
            for layer in range(self.num_layers):
                check(old.lib.skv_export_rows(ctypes.byref(old.desc), ptr(old.arena), layer, n, ptr(seq), ptr(bk), ptr(pos),
                                              ptr(kc), ptr(vc), ptr(ks), ptr(vs), st), "skv_export_rows")
                check(new.lib.skv_import_rows(ctypes.byref(new.desc), ptr(new.arena), layer, n, ptr(seq), ptr(bk), ptr(pos),
                                              ptr(kc), ptr(vc), ptr(ks), ptr(vs), ptr(new.err), st), "skv_import_rows")
        new.counts.copy_(torch.tensor([self._committed], dtype=torch.int32))
        new.head_state.copy_(old.head_state)
        new.head_parity = old.head_parity
        new.appended_total = old.appended_total
        new.max_seq_tokens = old.max_seq_tokens
        self._realloc_due = realloc_due
        self._dev_base = new.cumulative.clone()
        torch.cuda.synchronize(dev)

    # ------------------------------------------------------------------ store
    def quantize_and_store(self, layer_idx: int, token_id: int, k_vec: torch.Tensor, v_vec: torch.Tensor) -> None:
        """One token: k_vec, v_vec [num_heads, head_dim] (smartkv/core/cache.py:1163-1185)."""
        self.quantize_and_store_batch(layer_idx, [int(token_id)], k_vec.unsqueeze(0), v_vec.unsqueeze(0))

    def quantize_and_store_batch(self, layer_idx: int, token_ids: Sequence[int], k_batch: torch.Tensor,
                                 v_batch: torch.Tensor) -> None:
        """token_ids [n]; k_batch, v_batch [n, num_heads, head_dim] (smartkv/core/cache.py:1187-1355).
        A token not yet in ``precision_map`` is stored at 4 bits and entered into the map."""
        if isinstance(token_ids, torch.Tensor):
            token_ids = token_ids.tolist()
        ids = [int(t) for t in token_ids]
        n = len(ids)
        if n == 0:
            return
        if k_batch.shape != (n, self.num_heads, self.head_dim) or v_batch.shape != k_batch.shape:
            raise ValueError(f"expected k/v of shape {(n, self.num_heads, self.head_dim)}; got {tuple(k_batch.shape)} "
                             f"and {tuple(v_batch.shape)}")
        k = k_batch.to(self._dev)
        v = v_batch.to(self._dev)
        if k.dtype not in (torch.float32, torch.float16):
            k, v = k.float(), v.float()
        elif v.dtype != k.dtype:
            v = v.to(k.dtype)
        buckets, poss = [], []
        for tid in ids:
            if tid not in self._slot:
                bits = self.precision_map.get(tid, 4)
                if bits not in BITS_TO_BUCKET:
                    raise ValueError(f"token {tid} has width {bits}; the store holds 2, 3, 4 or 8 bits")
                self.precision_map.setdefault(tid, bits)
                bucket, pos = self._assign_slot(tid, bits)
                self.store.slot_token[0, self.store.bucket_base[bucket] + pos] = tid
                seed = self.importance_tracker.token_importance.get(tid)
                if seed is not None:   # importance gathered before the token had a place in the store
                    idx = self.store.bucket_base[bucket] + pos
                    self.store.cumulative[0, idx] = seed
                    self._dev_base[0, idx] = seed
            bucket, pos = self._slot[tid]
            buckets.append(bucket)
            poss.append(pos)
        dev = self._dev
        seq = torch.zeros(n, dtype=torch.int32, device=dev)
        self.store.append(layer_idx, k, v, seq, torch.tensor(buckets, dtype=torch.int32, device=dev),
                          torch.tensor(poss, dtype=torch.int32, device=dev))
        for tid, bucket in zip(ids, buckets):
            meta = {"bits": BUCKET_BITS[bucket], "token_id": tid, "layer": layer_idx}
            self.k_cache[(layer_idx, tid)] = meta
            self.v_cache[(layer_idx, tid)] = meta
            self._layers_of[tid].add(layer_idx)
            self._layer_tokens[layer_idx].add(tid)
        self.total_tokens_stored += n
        self.token_counter += n
        self._advance_commits()

    # ------------------------------------------------------------------ read back
    def _rows_of(self, layer_idx: int, ids: List[int]):
        n = len(ids)
        dev = self._dev
        H, D = self.num_heads, self.head_dim
        kc = torch.empty((n, H, D), dtype=torch.int8, device=dev)
        vc = torch.empty_like(kc)
        ks = torch.empty((n, H), dtype=torch.float32, device=dev)
        vs = torch.empty_like(ks)
        if n:
            seq = torch.zeros(n, dtype=torch.int32, device=dev)
            bk = torch.tensor([self._slot[t][0] for t in ids], dtype=torch.int32, device=dev)
            pos = torch.tensor([self._slot[t][1] for t in ids], dtype=torch.int32, device=dev)
            st = self.store
            check(st.lib.skv_export_rows(ctypes.byref(st.desc), ptr(st.arena), layer_idx, n, ptr(seq), ptr(bk), ptr(pos),
                                         ptr(kc), ptr(vc), ptr(ks), ptr(vs), st._stream()), "skv_export_rows")
        return kc, vc, ks, vs

    def _values_of(self, layer_idx: int, ids: List[int]):
        """Dequantised (keys, values) fp32 [n, num_heads, head_dim] of the given tokens of one layer."""
        n = len(ids)
        dev = self._dev
        keys = torch.empty((n, self.num_heads, self.head_dim), dtype=torch.float32, device=dev)
        values = torch.empty_like(keys)
        if n:
            seq = torch.zeros(n, dtype=torch.int32, device=dev)
            bk = torch.tensor([self._slot[t][0] for t in ids], dtype=torch.int32, device=dev)
            pos = torch.tensor([self._slot[t][1] for t in ids], dtype=torch.int32, device=dev)
            st = self.store
            check(st.lib.skv_dequant_rows(ctypes.byref(st.desc), ptr(st.arena), layer_idx, n, ptr(seq), ptr(bk), ptr(pos),
                                          _lib.DTYPE_F32, ptr(keys), ptr(values), st._stream()), "skv_dequant_rows")
        return keys, values

    def _select(self, layer_idx: int, token_ids: Optional[Sequence[int]]) -> List[int]:
        have = self._layer_tokens[layer_idx]
        if token_ids is None:
            return sorted(have)
        return [int(t) for t in token_ids if int(t) in have]

    def retrieve(self, layer_idx: int, token_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dequantised (key, value) [num_heads, head_dim]; KeyError if the layer does not hold the token."""
        if int(token_id) not in self._layer_tokens[layer_idx]:
            raise KeyError(f"Token {token_id} not found in cache for layer {layer_idx}")
        keys, values = self._values_of(layer_idx, [int(token_id)])
        return keys[0], values[0]

    def retrieve_all(self, layer_idx: int, token_ids: Optional[List[int]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dequantised keys, values [n, num_heads, head_dim] (ascending token id, or the order asked for)."""
        ids = self._select(layer_idx, token_ids)
        if not ids:
            empty = torch.empty(0, self.num_heads, self.head_dim, device=self._dev)
            return empty, empty.clone()
        return self._values_of(layer_idx, ids)

    def retrieve_all_quantized(self, layer_idx: int, token_ids: Optional[List[int]] = None) -> Dict[str, torch.Tensor]:
        """Codes and scales as the reference hands them to its kernels (cache.py:1441-1491)."""
        ids = sorted(self._select(layer_idx, token_ids))
        kc, vc, ks, vs = self._rows_of(layer_idx, ids)
        result = {"token_ids": torch.tensor(ids, dtype=torch.long, device=self._dev), "k_qx": kc, "k_scale": ks,
                  "v_qx": vc, "v_scale": vs}
        if self.use_bucketed_layout:
            result["buckets"] = self.get_bucket_views(layer_idx)
        return result

    def get_bucket_views(self, layer_idx: int) -> Dict[int, Dict[str, torch.Tensor]]:
        """Per bit-width: token ids, their position in the layer's id-sorted token list ('global_slots'),
        packed rows [n, num_heads, packed_dim] and scales [n, num_heads] (cache.py:671-744)."""
        dev = self._dev
        have = sorted(self._layer_tokens[layer_idx])
        rank = {t: i for i, t in enumerate(have)}
        views: Dict[int, Dict[str, torch.Tensor]] = {}
        for b, bits in enumerate(BUCKET_BITS):
            toks = [t for t in self._bucket_tokens[b] if t in rank]
            if not toks:
                continue
            n_all = len(self._bucket_tokens[b])
            sel = torch.tensor([self._slot[t][1] for t in toks], dtype=torch.long, device=dev)
            d = self.store.desc
            base = layer_idx * int(d.arena_bytes)
            H, cap, rb = self.num_heads, self.store.caps[b], int(d.row_bytes[b])

            def region(off, row_bytes, dtype):
                raw = self.store.arena[base + off: base + off + H * cap * row_bytes]
                return raw.view(dtype).view(H, cap, -1)[:, :n_all]
            k = region(int(d.k_off[b]), rb, torch.uint8)[:, sel].permute(1, 0, 2).contiguous()
            v = region(int(d.v_off[b]), rb, torch.uint8)[:, sel].permute(1, 0, 2).contiguous()
            sc = region(int(d.sc_off[b]), 8, torch.float32)[:, sel]
            views[bits] = {
                "token_ids": torch.tensor(toks, dtype=torch.long, device=dev),
                "global_slots": torch.tensor([rank[t] for t in toks], dtype=torch.long, device=dev),
                "k_qx": k if bits < 8 else k.view(torch.int8), "v_qx": v if bits < 8 else v.view(torch.int8),
                "k_scale": sc[..., 0].transpose(0, 1).contiguous(), "v_scale": sc[..., 1].transpose(0, 1).contiguous(),
                "packed": torch.tensor(1 if bits < 8 else 0, device=dev), "packed_dim": torch.tensor(rb, device=dev),
            }
        return views

    # ------------------------------------------------------------------ importance
    def _pull_device_importance(self):
        """Adds what the importance kernel accumulated on the device since the last pull to the tracker."""
        if not self._slot:
            return
        delta = (self.store.cumulative[0] - self._dev_base[0]).cpu()
        if not bool((delta != 0).any()):
            return
        imp = self.importance_tracker.token_importance
        base = self.store.bucket_base
        dl = delta.tolist()
        for tid, (bucket, pos) in self._slot.items():
            x = dl[base[bucket] + pos]
            if x != 0.0:
                imp[tid] = imp.get(tid, 0.0) + x
        self._dev_base.copy_(self.store.cumulative)

    def update_attention(self, layer_idx: int, attention_weights: Optional[torch.Tensor], token_ids: List[int]) -> None:
        """attention_weights [batch, heads, queries, keys]; token_ids: the ids of the keys
        (smartkv/core/cache.py:216-279)."""
        if isinstance(token_ids, torch.Tensor):
            token_ids = token_ids.tolist()
        if attention_weights is not None:
            heads = attention_weights.size(1)
            if self.head_importance.numel() != heads:
                self.head_importance = torch.ones(heads, dtype=torch.float32)
            head_mean = attention_weights.detach().float().mean(dim=(0, 2, 3)).cpu()
            self.head_importance = (self.head_importance * self.head_importance_decay
                                    + head_mean * (1.0 - self.head_importance_decay))
            normalized = self.head_importance / (self.head_importance.mean() + 1e-6)
            attention_weights = attention_weights * normalized.view(1, -1, 1, 1).to(attention_weights.device)
        self.importance_tracker.update_attention(layer_idx, attention_weights, token_ids)
        self.global_step += 1
        for tid in token_ids:
            self.last_seen[int(tid)] = self.global_step
            if self.enable_forecast:
                self._record_forecast_target(int(tid), self.importance_tracker.get_importance(int(tid)))
        self._maybe_reallocate(layer_idx, [int(t) for t in token_ids])

    def _maybe_reallocate(self, layer_idx: int, token_ids: List[int]):
        total_tokens = len(self.precision_map) + len(token_ids)
        adaptive_freq = max(self.realloc_freq * (1 + layer_idx // 4), max(32, total_tokens // 8))
        if self.token_counter % adaptive_freq == 0:
            self.allocate_precision(layer_idx, token_ids)
            self.realloc_counter += 1

    # ------------------------------------------------------------------ allocation
    def _protected_ids(self, candidates) -> List[int]:
        prot = sorted((self.protected_tokens | self.special_token_ids) & set(candidates))
        if len(prot) > _lib.ALLOC_MAX_PROTECTED:
            raise ValueError(f"more than {_lib.ALLOC_MAX_PROTECTED} protected token ids are cached")
        return prot

    def _solve_allocation(self, tokens, importance_scores: Dict[int, float],
                          protected_tokens: Optional[set] = None) -> Dict[int, int]:
        """The budgeted allocator (smartkv/core/cache.py:353-601) run on the device.  ``importance_scores``
        are the scores after the recency factor; ids in ``protected_tokens`` or below the critical
        window get the widest width."""
        cand = sorted(int(t) for t in set(tokens))
        n = len(cand)
        if n == 0:
            return {}
        lib, dev = self.store.lib, self._dev
        T_need = round_up(n + 1, 128)
        ctx = self._alloc_ctx
        if ctx is None or ctx["cap"] < T_need:
            cap = max(T_need, 2 * (ctx["cap"] if ctx else 0))
            d = StoreDesc()
            d.num_layers, d.num_seqs, d.num_kv_heads, d.head_dim = 1, 1, self.num_heads, self.head_dim
            for i, c in enumerate((128, 128, cap, 128)):
                d.cap[i] = c
            check(lib.skv_store_layout(ctypes.byref(d)), "skv_store_layout")
            T = int(d.slots)
            ctx = {"cap": cap, "desc": d, "T": T, "base": int(d.bucket_base[2]),
                   "ws": torch.empty(int(lib.skv_alloc_workspace_bytes(ctypes.byref(d))), dtype=torch.uint8, device=dev),
                   "new_bits": torch.zeros(T, dtype=torch.uint8, device=dev),
                   "new_counts": torch.zeros(NUM_BUCKETS, dtype=torch.int32, device=dev),
                   "changed": torch.zeros(1, dtype=torch.int32, device=dev)}
            self._alloc_ctx = ctx
        T, base, d = ctx["T"], ctx["base"], ctx["desc"]
        prot_all = set(protected_tokens) if protected_tokens is not None else (self.protected_tokens | self.special_token_ids)
        prot = sorted(prot_all & set(cand))
        if len(prot) > _lib.ALLOC_MAX_PROTECTED:
            raise ValueError(f"more than {_lib.ALLOC_MAX_PROTECTED} protected token ids are cached")
        cfg = self.store.make_alloc_config(
            self.memory_budget, self.available_bits, utility_alpha=self.utility_alpha,
            importance_floor=self.importance_floor, hysteresis_rank_threshold=self.hysteresis_rank_threshold,
            hysteresis_intervals=self.hysteresis_intervals, high_precision_fraction=self.high_precision_fraction,
            high_precision_boost=self.high_precision_boost, min_high_precision_tokens=self.min_high_precision_tokens,
            protected=prot, critical_window=self.critical_token_window, scale_bits=32 if self.scale_dtype == "fp32" else 16)
        counts = torch.tensor([0, 0, n, 0], dtype=torch.int32, device=dev)
        slot_token = torch.full((T,), -1, dtype=torch.int32)
        slot_token[base: base + n] = torch.tensor(cand, dtype=torch.int32)
        scores = torch.zeros(T, dtype=torch.float64)
        sc = [float(importance_scores.get(t, 0.0)) for t in cand]
        scores[base: base + n] = torch.tensor([0.0 if math.isinf(x) else x for x in sc], dtype=torch.float64)
        pct = torch.zeros(T, dtype=torch.float64)
        streak = torch.full((T,), -1, dtype=torch.int8)
        st = [self._rank_state.get(t) for t in cand]
        pct[base: base + n] = torch.tensor([s[0] if s else 0.0 for s in st], dtype=torch.float64)
        streak[base: base + n] = torch.tensor([s[1] if s else -1 for s in st], dtype=torch.int8)
        slot_token, scores, pct, streak = (x.to(dev) for x in (slot_token, scores, pct, streak))
        check(lib.skv_alloc_bits(ctypes.byref(d), ctypes.byref(cfg), ptr(counts), ptr(slot_token), ptr(scores), None,
                                 ptr(pct), ptr(streak), ptr(ctx["new_bits"]), ptr(ctx["new_counts"]), ptr(ctx["changed"]),
                                 ptr(ctx["ws"]), self.store._stream()), "skv_alloc_bits")
        bits = ctx["new_bits"][base: base + n].tolist()
        pct_l, streak_l = pct[base: base + n].tolist(), streak[base: base + n].tolist()
        for t, p_, s_ in zip(cand, pct_l, streak_l):
            self._rank_state[t] = (p_, int(s_))
        return {t: int(b) for t, b in zip(cand, bits)}

    def allocate_precision(self, layer_idx: int, token_ids: List[int]) -> Dict[int, int]:
        """smartkv/core/cache.py:281-351: scores = importance x recency (+inf for protected ids), allocation
        over every known token, changed tokens requantised from their stored codes in every layer."""
        if isinstance(token_ids, torch.Tensor):
            token_ids = token_ids.tolist()
        token_ids = [int(t) for t in token_ids]
        if not token_ids:
            return {}
        self._pull_device_importance()
        candidates = set(token_ids) | set(self.precision_map.keys()) | set(self._slot.keys())
        fused_seen = getattr(self, "_fused_seen_step", None)
        scores: Dict[int, float] = {}
        for tid in candidates:
            score = self.importance_tracker.get_importance(tid)
            if self.recency_temperature > 0:
                seen = self.last_seen.get(tid, self.global_step)
                if fused_seen is not None and tid in self._slot:
                    seen = max(seen, fused_seen)
                score *= math.exp(-(self.global_step - seen) / self.recency_temperature)
            scores[tid] = score
        if self.enable_forecast:
            self._blend_forecast(scores)
        allocation = self._solve_allocation(candidates, scores)
        previous = self.precision_map
        self.precision_map = allocation
        changed = {t for t, b in allocation.items() if previous.get(t) != b}
        if changed:
            self._requantize_tokens(changed)
        return {t: allocation[t] for t in token_ids if t in allocation}

    # ------------------------------------------------------------------ importance forecast
    def _blend_forecast(self, scores: Dict[int, float]) -> None:
        """smartkv/core/cache.py:313-336: every token with a finite positive score (protected ids carry +inf in
        the reference and are skipped) gets (1 - blend) * score + blend * max(prediction, 0); the feature row is
        kept until the token's next update supplies the training target."""
        protected = self.protected_tokens | self.special_token_ids
        rows, toks, raws = [], [], []
        for tid, score in scores.items():
            if tid in protected or tid < self.critical_token_window or not math.isfinite(score) or score <= 0.0:
                continue
            feature = self._build_forecast_feature(tid, score)
            rows.append(feature)
            toks.append(tid)
            raws.append(score)
            self.forecast_pending[tid] = (feature, self.global_step)
        if rows:
            preds = self.forecast_predictor.predict(torch.stack(rows)).tolist()
            for tid, raw, pred in zip(toks, raws, preds):
                scores[tid] = (1.0 - self.forecast_blend) * raw + self.forecast_blend * max(pred, 0.0)
                self.forecast_last_importance[tid] = raw
        for tid, score in scores.items():
            if math.isfinite(score) and not (tid in protected or tid < self.critical_token_window):
                self.forecast_last_importance[tid] = score

    def _build_forecast_feature(self, token_id: int, raw_importance: float) -> torch.Tensor:
        """The six inputs of the predictor (smartkv/core/cache.py:746-773)."""
        if not self.enable_forecast:
            raise RuntimeError("Forecasting disabled")
        delta = raw_importance - self.forecast_last_importance.get(token_id, 0.0)
        age = self.global_step - self.last_seen.get(token_id, self.global_step)
        bits_now = float(self.precision_map.get(token_id, self.min_general_bits))
        head_mean = float(self.head_importance.mean().item())
        position = math.tanh(token_id / max(1.0, self.total_tokens_stored + 1))
        step = math.tanh(self.global_step / max(1.0, self.recency_temperature * 10.0))
        return torch.tensor([math.log1p(max(raw_importance, 0.0)), math.log1p(abs(delta)),
                             math.tanh(age / max(self.recency_temperature, 1.0)), bits_now / max(self.available_bits),
                             math.tanh(head_mean), position + step], dtype=torch.float32)

    def _record_forecast_target(self, token_id: int, actual_importance: float) -> None:
        """smartkv/core/cache.py:775-791: a token that was scored at the last allocation now shows what its
        importance became; enough such pairs trigger one training step."""
        if not self.enable_forecast:
            return
        pending = self.forecast_pending.pop(token_id, None)
        if pending is None or not math.isfinite(actual_importance):
            return
        self.forecast_feature_buffer.append(pending[0].detach().cpu())
        self.forecast_target_buffer.append(math.log1p(max(actual_importance, 0.0)))
        if len(self.forecast_feature_buffer) >= self.forecast_update_interval:
            self._update_forecast_predictor()

    def _update_forecast_predictor(self) -> None:
        """smartkv/core/cache.py:793-804."""
        if not self.enable_forecast or self.forecast_predictor is None or not self.forecast_feature_buffer:
            return
        features = torch.stack(list(self.forecast_feature_buffer))
        targets = torch.tensor(list(self.forecast_target_buffer), dtype=torch.float32)
        self.forecast_last_loss = self.forecast_predictor.update(features, targets)
        self.forecast_feature_buffer.clear()
        self.forecast_target_buffer.clear()

    def _requantize_tokens(self, tokens: set) -> None:
        """smartkv/core/cache.py:806-844: stored tokens whose width changed move to the bucket of the new
        width in every layer, requantised from their dequantised codes."""
        if not any(t in self._slot for t in tokens):
            return
        self._realloc_due = True
        if not self._pending_tokens():
            self._apply_allocation()

    def _apply_allocation(self):
        self._realloc_due = False
        st = self.store
        self._pull_device_importance()
        new_bits = torch.zeros(st.slots, dtype=torch.uint8)
        moved = False
        for tid, (bucket, pos) in self._slot.items():
            bits = self.precision_map.get(tid, BUCKET_BITS[bucket])
            new_bits[st.bucket_base[bucket] + pos] = bits
            moved |= bits != BUCKET_BITS[bucket]
        if not moved:
            return
        st.repack(new_bits.view(1, -1).to(self._dev), max_moves=len(self._slot))
        st.check_errors()
        counts = st.counts[0].tolist()
        slot_token = st.slot_token[0].cpu().tolist()
        self._slot.clear()
        for b in range(NUM_BUCKETS):
            toks = slot_token[st.bucket_base[b]: st.bucket_base[b] + counts[b]]
            self._bucket_tokens[b] = [int(t) for t in toks]
            self._committed[b] = counts[b]
            for pos, t in enumerate(toks):
                self._slot[int(t)] = (b, pos)
        for (layer, tid), meta in self.k_cache.items():
            if tid in self._slot:
                meta["bits"] = BUCKET_BITS[self._slot[tid][0]]
        self._dev_base = st.cumulative.clone()

    # ------------------------------------------------------------------ fused decode step (used by the Llama wrapper)
    def fused_decode_attention(self, layer_idx: int, query: torch.Tensor, cur_k: torch.Tensor, cur_v: torch.Tensor,
                               token_id: int, update_importance: bool = True) -> torch.Tensor:
        """One decode query against this layer's cache plus the current token in full precision
        (the reference's fused CPU path, smartkv/models/llama_smartkv.py:264-305): query
        [num_query_heads, head_dim], cur_k / cur_v [num_heads, head_dim].  Returns fp32
        [num_query_heads, head_dim].  With ``update_importance`` the per-key attention mass of every cached
        token and of the current one is folded into the importance arrays on the device (the
        cache-level contract of update_attention: token_ids are the ids of the keys)."""
        tid = int(token_id)
        st = self.store
        if tid not in self._slot:
            bits = self.precision_map.get(tid, 4)
            self.precision_map.setdefault(tid, bits)
            bucket, pos = self._assign_slot(tid, bits)
            st.slot_token[0, st.bucket_base[bucket] + pos] = tid
        bucket, pos = self._slot[tid]
        cur_storage = torch.tensor([st.bucket_base[bucket] + pos], dtype=torch.int32, device=self._dev)
        q = query.reshape(1, self.num_query_heads, self.head_dim)
        if q.dtype not in (torch.float32, torch.float16):
            q = q.float()
        kv_dtype = torch.float16 if cur_k.dtype == torch.float16 else torch.float32
        out = st.attention(layer_idx, q.contiguous(), cur_k.reshape(1, self.num_heads, self.head_dim).to(kv_dtype),
                           cur_v.reshape(1, self.num_heads, self.head_dim).to(kv_dtype),
                           update_importance=update_importance, cur_storage=cur_storage)
        if update_importance:
            self.global_step += 1
            self._fused_seen_step = self.global_step
            self.last_seen[tid] = self.global_step
            if self.enable_forecast and self.forecast_pending:
                # every cached key took part in this update: the tokens scored at the last allocation now have
                # their training target
                self._pull_device_importance()
                for t in [t for t in self.forecast_pending if t in self._slot]:
                    self._record_forecast_target(t, self.importance_tracker.get_importance(t))
            self._maybe_reallocate(layer_idx, [tid])
        return out[0].clone()

    # ------------------------------------------------------------------ stats and misc
    def get_memory_stats(self) -> Dict[str, Any]:
        if self.precision_map:
            a = compute_memory_usage(self.precision_map, num_heads=self.num_heads, head_dim=self.head_dim,
                                     scale_dtype=self.scale_dtype, use_packing=self.use_packing)
        else:
            a = {"total_bits": 0, "avg_bits": 0.0, "memory_ratio": 0.0, "memory_ratio_true": 0.0, "num_tokens": 0,
                 "storage_mode": "packed", "scale_dtype": self.scale_dtype}
        try:
            import psutil
            system_memory_mb = psutil.Process(os.getpid()).memory_info().rss / 1024 / 1024
        except Exception:
            system_memory_mb = None
        return {
            "memory_budget": self.memory_budget, "memory_ratio": a["memory_ratio"],
            "memory_ratio_true": a.get("memory_ratio_true", a["memory_ratio"]), "avg_bits": a["avg_bits"],
            "num_tokens": a["num_tokens"], "num_cache_entries": sum(len(s) for s in self._layer_tokens),
            "precision_distribution": {f"{b}-bit": sum(1 for x in self.precision_map.values() if x == b)
                                       for b in self.available_bits},
            "total_tokens_stored": self.total_tokens_stored, "realloc_count": self.realloc_counter,
            "system_memory_mb": system_memory_mb, "storage_mode": a.get("storage_mode"),
            "scale_dtype": a.get("scale_dtype"),
        }

    def get_precision(self, token_id: int) -> int:
        return self.precision_map.get(token_id, 4)

    def get_importance(self, token_id: int) -> float:
        self._pull_device_importance()
        return self.importance_tracker.get_importance(token_id)

    def get_top_k_important_tokens(self, k: int) -> List[Tuple[int, float]]:
        self._pull_device_importance()
        return self.importance_tracker.get_top_k_tokens(k)

    def get_bottom_k_important_tokens(self, k: int) -> List[Tuple[int, float]]:
        self._pull_device_importance()
        return self.importance_tracker.get_bottom_k_tokens(k)

    def clear(self) -> None:
        """Empties the cache (smartkv/core/cache.py:1627-1639; the allocator's rank record survives, as there)."""
        self.k_cache.clear()
        self.v_cache.clear()
        self.precision_map.clear()
        self.importance_tracker.reset()
        self.token_counter = 0
        self.realloc_counter = 0
        self.total_tokens_stored = 0
        self.global_step = 0
        self.last_seen.clear()
        self._fused_seen_step = None
        self.head_importance = torch.ones(self.num_query_heads, dtype=torch.float32)
        st = self.store
        st.counts.zero_()
        st.slot_token.fill_(-1)
        st.next_token.zero_()
        st.cumulative.zero_()
        st.layer_ema.zero_()
        st.touched.zero_()
        st.rank_pct.zero_()
        st.rank_streak.fill_(-1)
        st.head_state.fill_(1.0)
        st.head_parity = 0
        st._plan_valid = False
        self._slot.clear()
        self._bucket_tokens = [[] for _ in range(NUM_BUCKETS)]
        self._committed = [0] * NUM_BUCKETS
        self._layers_of.clear()
        self._layer_tokens = [set() for _ in range(self.num_layers)]
        self._realloc_due = False
        self._dev_base.zero_()

    def reset(self) -> None:
        self.clear()

    def export_state(self) -> Dict[str, Any]:
        return {
            "config": {"num_layers": self.num_layers, "num_heads": self.num_heads, "head_dim": self.head_dim,
                       "memory_budget": self.memory_budget, "decay": self.decay, "realloc_freq": self.realloc_freq,
                       "available_bits": self.available_bits},
            "precision_map": self.precision_map.copy(), "token_counter": self.token_counter,
            "realloc_counter": self.realloc_counter, "total_tokens_stored": self.total_tokens_stored,
        }

    def __repr__(self) -> str:
        return (f"SmartKVCache(layers={self.num_layers}, budget={self.memory_budget:.1%}, "
                f"tokens={len(self.precision_map)}, cached={sum(len(s) for s in self._layer_tokens)})")

    def __len__(self) -> int:
        return len(self.precision_map)
