"""Several independent sequences behind one packed store: the cache the Llama wrapper uses for a batch.

``SmartKVCache`` (smartkv/core/cache.py) holds one sequence and does its bookkeeping in host
dictionaries, token by token.  ``BatchedSmartKVCache`` keeps B sequences of equal length in one
``PackedKVStore`` and keeps the policy state (importance, hysteresis record, widths) on the device, so that
one decode step costs two kernel launches per layer for the whole batch, and a reallocation is a fixed
handful of launches.  What it mirrors from the reference, per sequence:

* the head-weighted importance update of ``update_attention`` (smartkv/core/cache.py:232-264,
  smartkv/core/importance.py:44-101);
* the reallocation trigger ``token_counter % adaptive_freq == 0`` evaluated at every layer's update
  (cache.py:266-279), with the same counters, so that reallocations fall on the same layer of the same
  step as in the reference -- including in the middle of a decode step, when the step's token is among the
  candidates although only the layers before the trigger have stored it (cache.py:291-293, :806-844);
* the allocator with recency factor, protected ids, rank hysteresis and budget (cache.py:281-601), run on
  the device for all sequences at once, and the requantisation of changed tokens from their stored codes;
* new tokens enter at the width the last allocation gave them, 4 bits otherwise (cache.py:1214).

``key_attribution`` selects whose importance an attention row feeds.  ``"keys"`` (default) is the contract
``update_attention`` documents: the mass on a key is credited to that key's token.  ``"wrapper"`` reproduces
what the reference's Llama wrapper does in a decode step: it passes the id of the NEW token only
(smartkv/models/llama_smartkv.py:416-426), so the tracker credits the mass on the first cached key to the
new token, and only the new token's last-seen step is refreshed.  Parity runs against the reference wrapper
need it; nothing else should use it.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Sequence

import torch

from .. import _lib
from ..store import BUCKET_BITS, NUM_BUCKETS, PackedKVStore, round_up


class BatchedSmartKVCache:
    def __init__(self, num_layers: int, num_heads: int, head_dim: int, num_query_heads: int, batch_size: int,
                 max_tokens: int = 4096, memory_budget: float = 0.5, decay: float = 0.9, realloc_freq: int = 16,
                 available_bits: Sequence[int] = (2, 3, 4, 8), device: str = "cuda",
                 special_token_ids: Optional[Sequence[int]] = None, key_attribution: str = "keys",
                 utility_alpha: float = 0.5, importance_floor: float = 1e-6, hysteresis_rank_threshold: float = 0.05,
                 hysteresis_intervals: int = 2, high_precision_fraction: float = 0.02,
                 high_precision_boost: float = 1.5, min_high_precision_tokens: int = 0):
        if key_attribution not in ("keys", "wrapper"):
            raise ValueError("key_attribution must be 'keys' or 'wrapper'")
        dev = torch.device(device)
        if dev.type != "cuda":
            raise _lib.SmartKVLibraryError("BatchedSmartKVCache needs a CUDA device; there is no CPU path")
        self.num_layers, self.num_heads, self.head_dim = num_layers, num_heads, head_dim
        self.num_query_heads, self.batch_size = int(num_query_heads), int(batch_size)
        self.decay, self.realloc_freq = decay, int(realloc_freq)
        self.available_bits = sorted(int(b) for b in available_bits)
        self.key_attribution = key_attribution
        self.memory_budget = float(memory_budget)
        self.head_importance_decay = 0.9
        self.recency_temperature = 512.0
        self.max_tokens = round_up(int(max_tokens) + 1, 128)
        self._dev = dev
        cap = self.max_tokens
        self.store = PackedKVStore(num_layers, self.batch_size, num_heads, head_dim, self.num_query_heads,
                                   (cap, cap, cap, cap), device=dev, decay=decay,
                                   head_decay=self.head_importance_decay)
        self.store.token_capacity = self.max_tokens
        self.store.capture_check = "caller"      # a step that commits early ends twice; GraphedDecoder checks the total
        protected = sorted({0, 1, 2} | set(int(t) for t in (special_token_ids or [])))
        self._cfg = self.store.make_alloc_config(
            self.memory_budget, self.available_bits, utility_alpha=utility_alpha, importance_floor=importance_floor,
            hysteresis_rank_threshold=hysteresis_rank_threshold, hysteresis_intervals=hysteresis_intervals,
            high_precision_fraction=high_precision_fraction, high_precision_boost=high_precision_boost,
            min_high_precision_tokens=min_high_precision_tokens, protected=protected, critical_window=4)
        st = self.store
        slots = st.slots
        sb = torch.zeros(slots, dtype=torch.int32)
        sp = torch.zeros(slots, dtype=torch.int32)
        for b in range(NUM_BUCKETS):
            lo = st.bucket_base[b]
            hi = st.bucket_base[b + 1] if b + 1 < NUM_BUCKETS else slots
            sb[lo:hi] = b
            sp[lo:hi] = torch.arange(hi - lo, dtype=torch.int32)
        self._slot_bucket, self._slot_pos = sb.to(dev), sp.to(dev)
        self._slot_index = torch.arange(slots, dtype=torch.int64, device=dev)
        self._rows = torch.arange(self.batch_size, dtype=torch.int64, device=dev)
        self._mask = torch.zeros((self.batch_size, self.max_tokens), dtype=torch.float32, device=dev)
        self._staging_budget = 256 << 20
        # id of the token the next decode step appends, as a device scalar: everything a decode step does with it
        # (mask column, look-up of its storage index) reads this tensor, so a captured step stays valid on replay
        self._tok_dev = torch.zeros(1, dtype=torch.int64, device=dev)
        self.clear()

    # ------------------------------------------------------------------ bookkeeping
    def clear(self) -> None:
        st = self.store
        st.flush_importance()
        for t in (st.counts, st.next_token, st.cumulative, st.layer_ema, st.touched, st.rank_pct, st.err):
            t.zero_()
        st.slot_token.fill_(-1)
        st.rank_streak.fill_(-1)
        st.head_state.fill_(1.0)
        st.head_parity = 0
        st.appended_total = st.max_seq_tokens = 0
        st._plan_valid = False
        if getattr(st, "_pipe", None) is not None:
            st._pipe["calls"], st._pipe["pending"], st._pipe["post_events"] = 0, None, []
        self._mask.zero_()
        self._tok_dev.zero_()
        self.head_importance = torch.ones((self.batch_size, self.num_query_heads), dtype=torch.float32, device=self._dev)
        self.last_seen = torch.zeros(self.max_tokens, dtype=torch.float64, device=self._dev)
        self.num_cached = 0          # tokens every layer has stored, per sequence
        self.num_known = 0           # tokens with a width (len(precision_map) of the reference)
        self.token_counter = 0       # rows stored over all layers, per sequence (cache.py:1355)
        self.global_step = 0
        self.realloc_counter = 0
        self._step = None

    reset = clear

    def __len__(self) -> int:
        return self.num_cached

    def _token_storage(self) -> torch.Tensor:
        """int64 [B, max_tokens]: storage index of every cached token id (-1 where absent)."""
        st = self.store
        live = self._slot_pos[None, :] < st.counts.gather(1, self._slot_bucket[None].expand(self.batch_size, -1).long())
        dump = self.max_tokens                     # column that collects the unused storage indices
        tok = torch.where(live, st.slot_token.long(), torch.full_like(st.slot_token, dump, dtype=torch.int64))
        where = torch.full((self.batch_size, self.max_tokens + 1), -1, dtype=torch.int64, device=self._dev)
        where.scatter_(1, tok, self._slot_index[None].expand(self.batch_size, -1))
        where[:, dump] = -1
        return where[:, : self.max_tokens]

    def _plan_for(self, storage: torch.Tensor):
        storage = storage.to(torch.int32)
        flat = storage.reshape(-1).long()
        n = storage.numel() // self.batch_size
        seq = self.store._seq_ids[:, None].expand(self.batch_size, n).contiguous().view(-1)
        return seq, self._slot_bucket[flat].contiguous(), self._slot_pos[flat].contiguous(), storage.contiguous()

    def _trigger(self, layer: int, new_tokens: int) -> bool:
        total = self.num_known + new_tokens
        adaptive = max(self.realloc_freq * (1 + layer // 4), max(32, total // 8))
        return self.token_counter % adaptive == 0

    def _reallocate(self):
        st = self.store
        st.flush_importance()
        recency = None
        if self.key_attribution == "wrapper" and self.recency_temperature > 0:
            tok = st.slot_token.long().clamp(min=0)
            age = float(self.global_step) - self.last_seen[tok]
            recency = torch.exp(-age / self.recency_temperature).contiguous()
        if recency is None and torch.cuda.is_current_stream_capturing():
            # inside a captured decode step the launches become part of that graph; buffers sized for the capacity
            st.reallocate(self._cfg, max_moves=self.batch_size * st.slots, staging_budget=self._staging_budget)
        elif recency is None:
            # allocator + repack are some seventy small launches; replayed as one CUDA graph after the first time
            st.reallocate_graphed(self._cfg, staging_budget=self._staging_budget)
        else:
            new_bits, _, _ = st.allocate_bits(self._cfg, recency=recency)
            st.repack(new_bits, max_moves=self.batch_size * max(self.num_known, 1))
        self.realloc_counter += 1

    def _weights(self, head_mean: torch.Tensor) -> torch.Tensor:
        """Head-importance EMA and the normalised head weights (cache.py:243-250); fp32 [B, Hq]."""
        d = self.head_importance_decay
        st = self.store
        if self.key_attribution == "keys":       # the decode kernels keep this state on the device, double buffered
            st.flush_importance()
            self.head_importance = st.head_state[:, st.head_parity].clone()
        self.head_importance = self.head_importance * d + head_mean * (1.0 - d)
        if self.key_attribution == "keys":
            st.head_state[:, 0] = self.head_importance
            st.head_state[:, 1] = self.head_importance
        return self.head_importance / (self.head_importance.mean(dim=1, keepdim=True) + 1e-6)

    # ------------------------------------------------------------------ prefill
    def prefill_head_weights(self, num_tokens: int) -> torch.Tensor:
        """Advances the head-importance EMA by one prompt pass over ``num_tokens`` tokens and returns the
        normalised head weights fp32 [B, Hq] (cache.py:243-250).  Every causal row sums to one, so the mean
        probability of a head over (queries, keys) is 1 / num_tokens whatever the data: the weights can be had
        before the attention runs, which lets the prompt-pass kernel apply them while it sums the key mass."""
        mean = torch.full((self.batch_size, self.num_query_heads), 1.0 / num_tokens, dtype=torch.float32, device=self._dev)
        return self._weights(mean)

    def prefill_layer(self, layer: int, k: torch.Tensor, v: torch.Tensor, probs: Optional[torch.Tensor] = None,
                      key_mass: Optional[torch.Tensor] = None) -> None:
        """The prompt of every sequence for one layer: k, v [B, n, num_heads, head_dim]; either probs fp32
        [B, Hq, n, n], the causal attention probabilities the layer computed over the unquantised prompt
        (smartkv/models/llama_smartkv.py:392-427), or key_mass fp32 [B, n], their head-weighted sum over heads
        and queries computed with the weights of prefill_head_weights (the prompt-pass kernel's output).
        Importance update, reallocation trigger, then the rows are quantised at the widths in force and stored."""
        st = self.store
        B, n = k.shape[0], k.shape[1]
        if B != self.batch_size:
            raise ValueError(f"the cache was built for {self.batch_size} sequences; got {B}")
        if layer == 0:
            if self.num_cached:
                raise NotImplementedError("a second multi-token call on a non-empty batched cache (chunked prefill)")
            if n + 1 > self.max_tokens:
                raise _lib.SmartKVLibraryError(f"{n} prompt tokens exceed the cache capacity of {self.max_tokens - 1}")
        if key_mass is not None:
            mass = key_mass.double()
        else:
            w = self._weights(probs.float().mean(dim=(2, 3)))
            mass = (probs.float() * w[:, :, None, None]).sum(dim=(1, 2)).double()      # [B, n] per key
        ids = torch.arange(n, device=self._dev)
        if layer == 0:
            bits = torch.full((B, n), 4, dtype=torch.int32, device=self._dev)
            storage = st.plan_bulk(bits)[3].long()
            st.cumulative.scatter_(1, storage, mass)
            self.num_known = n
            first_known = 0
        else:
            storage = self._token_storage()[:, :n]
            st.cumulative.scatter_add_(1, storage, mass)
            first_known = n
        old = st.layer_ema[layer].gather(1, storage)
        seen = st.touched[layer].gather(1, storage).bool()
        st.layer_ema[layer].scatter_(1, storage, torch.where(seen, self.decay * old + (1 - self.decay) * mass.float(),
                                                             mass.float()))
        st.touched[layer].scatter_(1, storage, torch.ones_like(storage, dtype=torch.uint8))
        self.global_step += 1
        self.last_seen[ids] = float(self.global_step)
        # the reference counts len(precision_map) + len(token_ids); at layer 0 the map is still empty
        known = self.num_known
        self.num_known = first_known
        fire = self._trigger(layer, n)
        self.num_known = known
        if fire:
            self._reallocate()
            storage = self._token_storage()[:, :n]
        seq, bucket, pos, _ = self._plan_for(storage)
        st.append(layer, k.reshape(B * n, self.num_heads, self.head_dim), v.reshape(B * n, self.num_heads, self.head_dim),
                  seq, bucket, pos)
        self.token_counter += n
        if layer == self.num_layers - 1:
            self.num_cached = n
            self._tok_dev.fill_(n)

    # ------------------------------------------------------------------ decode
    def decode_layer(self, layer: int, query: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """One decode step of one layer for the whole batch: query [B, Hq, head_dim], k / v [B, num_heads,
        head_dim] of the step's token (attended in full precision, smartkv/models/llama_smartkv.py:264-305).
        Returns fp32 [B, Hq, head_dim] (a buffer the store reuses).  Layers must be called in order 0..L-1."""
        st = self.store
        if layer == 0:
            if self.num_cached + 2 > self.max_tokens:
                raise _lib.SmartKVLibraryError(f"the cache holds {self.num_cached} tokens per sequence; capacity "
                                               f"{self.max_tokens - 1} (max_tokens)")
            plan = st.plan_step(None)
            self._step = {"plan": plan, "early": False, "token": self.num_cached, "token0": None}
        step = self._step
        if step is None:
            raise RuntimeError("decode_layer(0, ...) starts a step")
        wrapper = self.key_attribution == "wrapper"
        kv_dtype = torch.float16 if k.dtype == torch.float16 else torch.float32
        k, v = k.to(kv_dtype).contiguous(), v.to(kv_dtype).contiguous()
        q = query if query.dtype in (torch.float16, torch.float32) else query.float()
        out = st.decode_layer(layer, q, k, v, step["plan"], update_importance=True,
                              mask=self._mask if step["early"] else None)
        self.global_step += 1
        if wrapper:
            logits, lmax, lsum, _cur = st.take_pending_logits()
            if step["token0"] is None:
                step["token0"] = self._token_storage()[:, 0]
            p0 = torch.exp2(logits[self._rows, :, step["token0"]] - lmax) / lsum              # [B, Hq]
            # every head's probabilities sum to one over the cached keys and the new token
            w = self._weights(torch.full_like(p0, 1.0 / (self.num_cached + 1)))
            score = (p0 * w).sum(dim=1).double()
            st.cumulative[self._rows, step["plan"][3].long()] += score
            self.last_seen[step["token"]] = float(self.global_step)
        new_known = self.num_cached + (1 if (layer > 0 or step["early"]) else 0)
        self.num_known = new_known
        if self._trigger(layer, 1):
            if not step["early"]:
                st.commit_step(step["plan"])             # the step's token becomes a candidate of the allocation
                step["early"] = True
                self._mask.index_fill_(1, self._tok_dev, -1e30)   # ... but stays out of the cached keys of this step
            self._reallocate()
            where = self._token_storage()
            step["plan"] = self._plan_for(where.index_select(1, self._tok_dev)[:, 0])
            step["token0"] = where[:, 0]
            # this layer's row at the width just decided, from the full-precision values (cache.py:1214)
            st.append(layer, k, v, *step["plan"][:3])
        self.num_known = self.num_cached + 1
        self.token_counter += 1
        if layer == self.num_layers - 1:
            if step["early"]:
                st.end_step()
                self._mask.index_fill_(1, self._tok_dev, 0.0)
            else:
                st.commit_step(step["plan"])
            self._tok_dev += 1
            self.num_cached += 1
            self._step = None
        return out

    # ------------------------------------------------------------------ captured decode steps
    def next_step_triggers(self) -> tuple:
        """The layers at which the NEXT decode step will reallocate (a function of the counters only): the key
        under which a captured step can be replayed."""
        out, tc, early = [], self.token_counter, False
        for layer in range(self.num_layers):
            known = self.num_cached + (1 if (layer > 0 or early) else 0)
            total = known + 1
            adaptive = max(self.realloc_freq * (1 + layer // 4), max(32, total // 8))
            if tc % adaptive == 0:
                out.append(layer)
                early = True
            tc += 1
        return tuple(out)

    def advance_after_replay(self, triggers: tuple) -> None:
        """Host-side bookkeeping of one decode step that ran as a graph replay (the device did the rest)."""
        L = self.num_layers
        self.token_counter += L
        self.global_step += L
        self.realloc_counter += len(triggers)
        self.num_cached += 1
        self.num_known = self.num_cached
        st = self.store
        st.max_seq_tokens += 1
        st.appended_total += self.batch_size
        st._plan_valid = False

    # ------------------------------------------------------------------ stats
    def token_bits(self) -> torch.Tensor:
        """uint8 [B, tokens]: the width of every cached token (syncs)."""
        where = self._token_storage()[:, : self.num_cached]
        bits = torch.tensor(BUCKET_BITS, dtype=torch.uint8, device=self._dev)
        return bits[self._slot_bucket[where.clamp(min=0)].long()]

    def get_memory_stats(self) -> Dict[str, Any]:
        from .cache import compute_memory_usage
        bits = self.token_bits().cpu()
        per_seq = []
        for b in range(self.batch_size):
            alloc = {t: int(x) for t, x in enumerate(bits[b].tolist())}
            per_seq.append(compute_memory_usage(alloc, num_heads=self.num_heads, head_dim=self.head_dim,
                                                scale_dtype="fp32", use_packing=True) if alloc else {})
        a = dict(per_seq[0]) if per_seq and per_seq[0] else {"num_tokens": 0, "avg_bits": 0.0, "memory_ratio": 0.0,
                                                              "memory_ratio_true": 0.0}
        a["memory_ratio_true_max"] = max((p.get("memory_ratio_true", 0.0) for p in per_seq), default=0.0)
        a["memory_budget"] = self.memory_budget
        a["num_sequences"] = self.batch_size
        a["precision_distribution"] = {f"{w}-bit": int((bits == w).sum()) for w in (8, 4, 3, 2)}
        a["realloc_count"] = self.realloc_counter
        a["storage_mode"] = "packed"
        a["scale_dtype"] = "fp32"
        return a

    def check_errors(self):
        self.store.check_errors()

    def __repr__(self) -> str:
        return (f"BatchedSmartKVCache(layers={self.num_layers}, sequences={self.batch_size}, tokens={self.num_cached}, "
                f"budget={self.memory_budget}, attribution={self.key_attribution})")
