"""Common part of the comparison caches (uniform INT8 / INT4, KIVI): one sequence in a ``PackedKVStore``,
rows entered as already quantised codes + scales (skv_import_rows), read back through the same export /
dequantise entry points and attended by the same packed decode kernels as the SmartKV cache."""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _lib
from .._lib import check, ptr
from ..store import BITS_TO_BUCKET, NUM_BUCKETS, PackedKVStore, round_up


def quantize_per_tensor(x: torch.Tensor, bits: int):
    """The reference quantizers (smartkv/core/quantizers.py:69-91, :114-133, :191-210): ONE scale per token
    tensor, ``max|x| / qmax`` (1 for an all-zero tensor), codes ``clamp(round(x / scale), -2^(b-1), 2^(b-1)-1)``.
    x [n, heads, head_dim] fp32 -> (codes int8 [n, heads, head_dim], scale fp32 [n])."""
    x = x.float()
    # a device tensor as divisor: dividing a CUDA tensor by a Python number multiplies by the rounded reciprocal,
    # which is not the reference's (CPU) true division in the last bit
    qmax = torch.tensor(float(2 ** (bits - 1) - 1), dtype=torch.float32, device=x.device)
    scale = x.abs().amax(dim=(1, 2)) / qmax
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = torch.clamp(torch.round(x / scale[:, None, None]), -(2 ** (bits - 1)), 2 ** (bits - 1) - 1).to(torch.int8)
    return q, scale


class PackedBaselineCache:
    """Token bookkeeping over a one-sequence packed store whose rows all sit in the bucket of ``store_bits``."""

    def __init__(self, num_layers: int, num_heads: int, head_dim: int, store_bits: int, device: str = "cuda",
                 max_tokens: int = 4096, num_query_heads: Optional[int] = None):
        dev = torch.device(device)
        if dev.type != "cuda":
            raise _lib.SmartKVLibraryError("the comparison caches of the B200 library need a CUDA device; there is no CPU path")
        if head_dim not in (64, 128):
            raise ValueError(f"head_dim must be 64 or 128 on the B200 path; got {head_dim}")
        self.num_layers, self.num_heads, self.head_dim = num_layers, num_heads, head_dim
        self.num_query_heads = int(num_query_heads or num_heads)
        self.device = device
        self._dev = dev
        self._bucket = BITS_TO_BUCKET[store_bits]
        self._max_tokens = int(max_tokens)
        self._init_store()
        self.total_tokens_stored = 0

    def _init_store(self):
        cap = round_up(self._max_tokens + 1, 128)
        caps = [128] * NUM_BUCKETS
        caps[self._bucket] = cap
        self.store = PackedKVStore(self.num_layers, 1, self.num_heads, self.head_dim, self.num_query_heads, tuple(caps),
                                   device=self._dev, track_importance=False)
        self._pos: Dict[int, int] = {}                                     # token id -> position in the bucket
        self._layer_tokens: List[set] = [set() for _ in range(self.num_layers)]

    # ---------------------------------------------------------------- storing
    def _store_codes(self, layer_idx: int, token_ids: Sequence[int], kq, ks, vq, vs):
        """kq, vq int8 [n, H, D]; ks, vs fp32 [n, H]."""
        st = self.store
        ids = [int(t) for t in token_ids]
        for t in ids:
            if t not in self._pos:
                if len(self._pos) >= self._max_tokens:
                    raise _lib.SmartKVLibraryError(f"the cache holds {len(self._pos)} tokens; capacity {self._max_tokens} "
                                                   "(max_tokens)")
                p = len(self._pos)
                self._pos[t] = p
                st.slot_token[0, st.bucket_base[self._bucket] + p] = t
        n = len(ids)
        dev = self._dev
        seq = torch.zeros(n, dtype=torch.int32, device=dev)
        bk = torch.full((n,), self._bucket, dtype=torch.int32, device=dev)
        pos = torch.tensor([self._pos[t] for t in ids], dtype=torch.int32, device=dev)
        check(st.lib.skv_import_rows(ctypes.byref(st.desc), ptr(st.arena), layer_idx, n, ptr(seq), ptr(bk), ptr(pos),
                                     ptr(kq.contiguous()), ptr(vq.contiguous()), ptr(ks.contiguous()), ptr(vs.contiguous()),
                                     ptr(st.err), st._stream()), "skv_import_rows")
        self._layer_tokens[layer_idx].update(ids)
        self.total_tokens_stored += n
        # a token becomes visible to attention once every layer holds it
        full = sum(1 for t in self._pos if all(t in s for s in self._layer_tokens))
        if full != int(getattr(self, "_visible", 0)):
            self._visible = full
            counts = [0] * NUM_BUCKETS
            counts[self._bucket] = full
            st.counts.copy_(torch.tensor([counts], dtype=torch.int32))
            st._plan_valid = False
            st.max_seq_tokens = full

    # ---------------------------------------------------------------- reading
    def _rows(self, layer_idx: int, ids: List[int], dequant: bool):
        n, dev, st = len(ids), self._dev, self.store
        seq = torch.zeros(n, dtype=torch.int32, device=dev)
        bk = torch.full((n,), self._bucket, dtype=torch.int32, device=dev)
        pos = torch.tensor([self._pos[t] for t in ids], dtype=torch.int32, device=dev)
        H, D = self.num_heads, self.head_dim
        if dequant:
            k = torch.empty((n, H, D), dtype=torch.float32, device=dev)
            v = torch.empty_like(k)
            check(st.lib.skv_dequant_rows(ctypes.byref(st.desc), ptr(st.arena), layer_idx, n, ptr(seq), ptr(bk), ptr(pos),
                                          _lib.DTYPE_F32, ptr(k), ptr(v), st._stream()), "skv_dequant_rows")
            return k, v
        kc = torch.empty((n, H, D), dtype=torch.int8, device=dev)
        vc = torch.empty_like(kc)
        ks = torch.empty((n, H), dtype=torch.float32, device=dev)
        vs = torch.empty_like(ks)
        check(st.lib.skv_export_rows(ctypes.byref(st.desc), ptr(st.arena), layer_idx, n, ptr(seq), ptr(bk), ptr(pos),
                                     ptr(kc), ptr(vc), ptr(ks), ptr(vs), st._stream()), "skv_export_rows")
        return kc, vc, ks, vs

    def retrieve(self, layer_idx: int, token_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dequantised (key, value) [num_heads, head_dim]; KeyError if the layer does not hold the token."""
        if int(token_id) not in self._layer_tokens[layer_idx]:
            raise KeyError(f"Token {token_id} not found in layer {layer_idx}")
        k, v = self._rows(layer_idx, [int(token_id)], True)
        return k[0], v[0]

    def retrieve_all(self, layer_idx: int, token_ids: Optional[list] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dequantised keys, values [n, num_heads, head_dim] in ascending token id (or the order asked for;
        ids the layer does not hold are skipped, as the reference skips them)."""
        have = self._layer_tokens[layer_idx]
        ids = sorted(have) if token_ids is None else [int(t) for t in token_ids if int(t) in have]
        if not ids:
            return torch.empty(0), torch.empty(0)
        return self._rows(layer_idx, ids, True)

    def decode_attention(self, layer_idx: int, query: torch.Tensor, cur_k: Optional[torch.Tensor] = None,
                         cur_v: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode query [num_query_heads, head_dim] against the layer's cache (every token all layers hold),
        optionally with the step's own token [num_heads, head_dim] in full precision: the packed decode kernels
        of the SmartKV path on this cache's rows.  Returns fp32 [num_query_heads, head_dim]."""
        q = query.reshape(1, self.num_query_heads, self.head_dim)
        if q.dtype not in (torch.float16, torch.float32):
            q = q.float()
        ck = None if cur_k is None else cur_k.reshape(1, self.num_heads, self.head_dim).float()
        cv = None if cur_v is None else cur_v.reshape(1, self.num_heads, self.head_dim).float()
        return self.store.attention(layer_idx, q.contiguous(), ck, cv)[0].clone()

    # ---------------------------------------------------------------- misc
    def clear(self) -> None:
        st = self.store
        st.counts.zero_()
        st.slot_token.fill_(-1)
        st._plan_valid = False
        st.max_seq_tokens = 0
        self._pos.clear()
        self._layer_tokens = [set() for _ in range(self.num_layers)]
        self._visible = 0
        self.total_tokens_stored = 0

    def reset(self) -> None:
        self.clear()

    def __len__(self) -> int:
        return len(self._pos)

    @property
    def num_cache_entries(self) -> int:
        return sum(len(s) for s in self._layer_tokens)
