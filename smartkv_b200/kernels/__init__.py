"""Mirror of ``smartkv.kernels`` (smartkv/kernels/__init__.py): ``quantized_attention``,
``quantized_attention_bucketed``, ``CUDA_AVAILABLE``, ``check_cuda_availability``.

Same names, argument layouts and error messages as the reference; the work is done by the packed
decode-attention kernels of ``libsmartkv_b200.so`` (the int8 codes the caller hands over are packed
into a scratch store first).  Differences, all deliberate:
  * there is no PyTorch fallback: a CPU tensor or a missing library is an error;
  * an additive attention mask is one row per (sequence, query position), shared by the heads
    ([B, 1, q, k], as the reference's kernels index it); a mask that differs between heads raises;
  * ``quantized_attention_bucketed`` accepts batch 1 only, like the reference (:278).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from .. import _lib
from .._lib import check, ptr
from ..store import PackedKVStore, round_up
from .bit_packing import (compute_packed_size, get_compression_ratio, get_memory_savings_vs_fp16,  # noqa: F401
                          pack_tensor, unpack_tensor)

CUDA_AVAILABLE = True
LEGACY_TILE_SIZE = 128


def check_cuda_availability() -> bool:
    """True when the B200 library loads and a CUDA device is present."""
    try:
        _lib.lib()
    except _lib.SmartKVLibraryError:
        return False
    return torch.cuda.is_available()


# ---- layout helpers: the reference accepts a few layouts and normalises them (:17-85) ------------
def _ensure_query_layout(query: torch.Tensor) -> torch.Tensor:
    if query.ndim != 4:
        raise ValueError(f"query must be 4D [B, H, q_len, d]; got shape {query.shape}")
    return query


def _ensure_kv_layout(tensor: torch.Tensor, num_heads: int, name: str) -> torch.Tensor:
    if tensor.ndim != 4:
        raise ValueError(f"{name} must be 4D; got shape {tensor.shape}")
    if tensor.size(1) == num_heads:
        return tensor
    if tensor.size(2) == num_heads:
        return tensor.permute(0, 2, 1, 3).contiguous()
    raise ValueError(f"{name} has incompatible shape {tensor.shape}; cannot infer head dimension")


def _ensure_scale_layout(scale: torch.Tensor, num_heads: int, k_len: int, name: str) -> torch.Tensor:
    if scale.ndim == 3 and scale.size(1) == num_heads:
        return scale
    if scale.ndim == 3 and scale.size(2) == num_heads:
        return scale.permute(0, 2, 1).contiguous()
    if scale.ndim == 2 and scale.size(1) == k_len:
        return scale.unsqueeze(1).expand(-1, num_heads, -1)
    raise ValueError(f"{name} must broadcast to [B, H, k_len]; got shape {scale.shape}")


def _mask_rows(attention_mask: Optional[torch.Tensor], batch: int, q_len: int, k_len: int) -> Optional[torch.Tensor]:
    """The reference's additive mask [B, 1, q, k] (smartkv/csrc/quantized_attention.cu:213-216, 570-575) as
    fp32 [B, q, k]; None stays None."""
    if attention_mask is None:
        return None
    m = attention_mask
    if m.dim() == 4:
        if m.size(1) != 1:
            if bool((m != m[:, :1]).any()):
                raise NotImplementedError("per-head attention masks are not supported: the kernels take one mask row "
                                          "per sequence and query position, like the reference's")
            m = m[:, :1]
        m = m[:, 0]
    if m.dim() == 2:
        m = m[:, None, :]
    if m.dim() != 3:
        raise ValueError(f"attention_mask must be [B, 1, q_len, k_len]; got shape {tuple(attention_mask.shape)}")
    m = m.to(torch.float32).expand(batch, q_len, m.size(-1))
    if m.size(-1) < k_len:
        raise ValueError(f"attention_mask covers {m.size(-1)} keys, the cache holds {k_len}")
    return m.contiguous()


def _need_cuda(t: torch.Tensor, what: str):
    if t.device.type != "cuda":
        raise _lib.SmartKVLibraryError(f"{what}: tensor is on {t.device}; the B200 library has no CPU path")


def _attend(query: torch.Tensor, per_seq_rows, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """query [B, H, q, D]; per_seq_rows[b] = list of (bits, k_codes [n, H, D] int8, v_codes, k_scale [n, H], v_scale,
    key positions int [n] or None = 0..n-1).  mask fp32 [B, q, k] or None, indexed by key position.
    Packs the rows into a scratch store (every query head its own KV head) and runs the decode kernels
    once per query position."""
    B, H, q_len, D = query.shape
    dev = query.device
    if D not in (64, 128):
        raise ValueError(f"head_dim must be 64 or 128 on the B200 path; got {D}")
    need = [128, 128, 128, 128]
    for rows in per_seq_rows:
        tot = {2: 0, 3: 0, 4: 0, 8: 0}
        for bits, kq, *_rest in rows:
            tot[bits] += kq.shape[0]
        for i, w in enumerate(_lib.BUCKET_BITS):
            need[i] = max(need[i], round_up(tot[w] + 1, 128))
    out = torch.empty((B, H, q_len, D), dtype=torch.float32, device=dev)
    # group size <= 8: query heads are processed in chunks of KV heads of the same count (group 1)
    store = PackedKVStore(1, B, H, D, H, tuple(need), device=dev, track_importance=False)
    st = store._stream()
    for b, rows in enumerate(per_seq_rows):
        seen = 0
        for bits, kq, vq, ks, vs, positions in rows:
            n = kq.shape[0]
            if n == 0:
                continue
            bucket = _lib.BITS_TO_BUCKET[bits]
            base = int(store.counts[b, bucket])
            if positions is None:
                positions = torch.arange(seen, seen + n, dtype=torch.int32, device=dev)
            seen += n
            store.slot_token[b, store.bucket_base[bucket] + base: store.bucket_base[bucket] + base + n] = \
                positions.to(device=dev, dtype=torch.int32)
            seq = torch.full((n,), b, dtype=torch.int32, device=dev)
            bk = torch.full((n,), bucket, dtype=torch.int32, device=dev)
            pos = torch.arange(base, base + n, dtype=torch.int32, device=dev)
            check(store.lib.skv_import_rows(ctypes.byref(store.desc), ptr(store.arena), 0, n, ptr(seq), ptr(bk), ptr(pos),
                                            ptr(kq.contiguous()), ptr(vq.contiguous()),
                                            ptr(ks.contiguous().float()), ptr(vs.contiguous().float()), ptr(store.err),
                                            st), "skv_import_rows")
            store.counts[b, bucket] += n
    store._plan_valid = False
    qf = query.float() if query.dtype not in (torch.float32, torch.float16) else query
    for i in range(q_len):
        out[:, :, i] = store.attention(0, qf[:, :, i].contiguous(), mask=None if mask is None else mask[:, i])
    store.check_errors()
    return out.to(query.dtype) if query.dtype in (torch.float16, torch.bfloat16) else out


def quantized_attention(query: torch.Tensor, key_int8: torch.Tensor, key_scale: torch.Tensor,
                        value_int8: torch.Tensor, value_scale: torch.Tensor,
                        attention_mask: Optional[torch.Tensor] = None, use_cuda: bool = True) -> torch.Tensor:
    """softmax(Q K^T / sqrt(d)) V with K, V given as int8 codes and per-(head, key) scales
    (smartkv/kernels/__init__.py:103-186).  query [B, H, q_len, d]; key_int8 / value_int8
    [B, H, k_len, d]; scales [B, H, k_len].  Returns [B, H, q_len, d]."""
    query = _ensure_query_layout(query)
    _need_cuda(query, "quantized_attention")
    batch, num_heads, q_len, d = query.shape
    key_int8 = _ensure_kv_layout(key_int8, num_heads, "key_int8")
    value_int8 = _ensure_kv_layout(value_int8, num_heads, "value_int8")
    k_len = key_int8.shape[2]
    key_scale = _ensure_scale_layout(key_scale, num_heads, k_len, "key_scale")
    value_scale = _ensure_scale_layout(value_scale, num_heads, k_len, "value_scale")
    mask = _mask_rows(attention_mask, batch, q_len, k_len)
    if k_len == 0:
        return torch.zeros_like(query)
    rows = []
    for b in range(batch):
        rows.append([(8, key_int8[b].permute(1, 0, 2).contiguous().to(torch.int8),
                      value_int8[b].permute(1, 0, 2).contiguous().to(torch.int8),
                      key_scale[b].transpose(0, 1).contiguous(), value_scale[b].transpose(0, 1).contiguous(), None)])
    return _attend(query, rows, mask)


def quantized_attention_bucketed(query: torch.Tensor, bucket_views: Dict[int, Dict[str, torch.Tensor]],
                                 attention_mask: Optional[torch.Tensor] = None, use_cuda: bool = True) -> torch.Tensor:
    """Attention over the per-bit-width views ``SmartKVCache.get_bucket_views`` returns
    (smartkv/kernels/__init__.py:269-386): bucket_views[bits] = {'token_ids', 'global_slots',
    'k_qx', 'v_qx' (packed uint8 [n, H, packed_dim] or int8 [n, H, d]), 'k_scale', 'v_scale' [n, H],
    'packed', 'packed_dim'}."""
    query = _ensure_query_layout(query)
    _need_cuda(query, "quantized_attention_bucketed")
    batch, num_heads, q_len, head_dim = query.shape
    if batch != 1:
        raise ValueError("Bucketed attention currently supports batch=1")
    rows = []
    k_total = 0
    for bits in sorted(bucket_views.keys()):
        view = bucket_views[bits]
        n = int(view["token_ids"].numel())
        if n == 0:
            continue
        if bits not in _lib.BITS_TO_BUCKET:
            raise ValueError(f"bits must be 2, 3, 4, or 8, got {bits}")
        k, v = view["k_qx"], view["v_qx"]
        packed = int(view["packed"].item()) if "packed" in view else 0
        if packed:
            shape = (n, num_heads, head_dim)
            k = unpack_tensor(k.reshape(n, num_heads, -1).contiguous().reshape(-1), bits, shape)
            v = unpack_tensor(v.reshape(n, num_heads, -1).contiguous().reshape(-1), bits, shape)
        # the mask is indexed by the key's global slot (smartkv/kernels/__init__.py:292-296)
        slots = view["global_slots"].reshape(n) if "global_slots" in view else None
        rows.append((bits, k.to(torch.int8), v.to(torch.int8), view["k_scale"].reshape(n, num_heads),
                     view["v_scale"].reshape(n, num_heads), slots))
        k_total = max(k_total + n, int(slots.max()) + 1 if slots is not None else 0)
    if not rows:
        return torch.zeros_like(query)
    return _attend(query, [rows], _mask_rows(attention_mask, batch, q_len, k_total))


__all__ = ["quantized_attention", "quantized_attention_bucketed", "CUDA_AVAILABLE", "check_cuda_availability",
           "pack_tensor", "unpack_tensor", "compute_packed_size", "get_compression_ratio",
           "get_memory_savings_vs_fp16"]
