"""The prompt pass: causal attention over the unquantised prompt with the per-key attention mass of the
importance update (skv_prefill_attention), for fp16 queries, keys and values on the device."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import check, ptr


def _strides(t: torch.Tensor):
    """Element strides (batch, token, head) of a [B, n, H, D] view; head_dim must be contiguous."""
    if t.stride(3) != 1:
        raise ValueError("head_dim must be the contiguous dimension")
    return (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def causal_prefill_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                             head_weights: Optional[torch.Tensor] = None,
                             want_mass: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """q [B, n, Hq, D], k / v [B, n, Hkv, D]: fp16 CUDA tensors, any strides with D contiguous (the transposed
    views a Llama attention module holds are fine).  ``head_weights`` fp32 [B, Hq].  Returns
    (out fp16 [B, n, Hq, D], key_mass fp32 [B, n] or None): out is softmax(q k^T / sqrt(D) + causal) v, key_mass[b, j]
    the sum over heads h and queries i of head_weights[b, h] * probability[b, h, i, j]."""
    if q.dtype != torch.float16 or k.dtype != torch.float16 or v.dtype != torch.float16:
        raise TypeError("the prompt-pass kernel takes fp16 inputs")
    if not q.is_cuda:
        raise _lib.SmartKVLibraryError("the prompt-pass kernel needs CUDA tensors; there is no CPU path")
    B, n, Hq, D = q.shape
    Hkv = k.shape[2]
    assert k.shape == (B, n, Hkv, D) and v.shape == k.shape
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.stride(3) != 1 or any(s % 8 for s in t.stride()[:3]) or t.data_ptr() % 16:
            raise ValueError(f"{name}: head_dim must be contiguous, other strides multiples of 8, base 16-byte aligned")
    out = torch.empty((B, n, Hq, D), dtype=torch.float16, device=q.device)
    lse = torch.empty((B, Hq, n), dtype=torch.float32, device=q.device)
    mass = torch.empty((B, Hkv, n), dtype=torch.float32, device=q.device) if want_mass else None
    w = None if head_weights is None else head_weights.to(torch.float32).contiguous()
    st = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
    check(_lib.lib().skv_prefill_attention(ptr(q), ptr(k), ptr(v), _lib.DTYPE_F16, B, n, Hq, Hkv, D, _strides(q),
                                           _strides(k), _strides(v), ptr(w), ptr(out), ptr(lse), ptr(mass), st),
          "skv_prefill_attention")
    return out, (mass.sum(dim=1) if want_mass else None)
