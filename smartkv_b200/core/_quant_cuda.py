"""Mirror of ``smartkv.core._quant_cuda`` (smartkv/core/_quant_cuda.py:19-90) over the C ABI."""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from .. import _lib
from .._lib import check, ptr
from ..kernels.bit_packing import pack_tensor, unpack_tensor


def _quantize(x: torch.Tensor, bits: int):
    x = x.contiguous()
    if x.dtype not in (torch.float32, torch.float16):
        x = x.float()                       # the reference upcasts before quantising (cache.py:1201-1202)
    n, h, d = x.shape
    codes = torch.empty((n, h, d), dtype=torch.int8, device=x.device)
    scales = torch.empty((n, h), dtype=torch.float32, device=x.device)
    if n * h:
        stream = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
        check(_lib.lib().skv_quantize_per_head(ptr(x), _lib.DTYPE_F16 if x.dtype == torch.float16 else _lib.DTYPE_F32,
                                               n * h, d, bits, ptr(codes), ptr(scales), stream), "skv_quantize_per_head")
    return codes, scales


def quantize_per_head_cuda(k_subset: torch.Tensor, v_subset: torch.Tensor,
                           bits: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """k, v [N, H, D] on a CUDA device -> (k_q int8, v_q int8, k_scale fp32 [N, H], v_scale)."""
    if not k_subset.is_cuda or not v_subset.is_cuda:
        raise ValueError("Input tensors must be on CUDA device")
    k_q, k_scale = _quantize(k_subset, bits)
    v_q, v_scale = _quantize(v_subset, bits)
    return k_q, v_q, k_scale, v_scale


def pack_values(tensor: torch.Tensor, bits: int) -> torch.Tensor:
    return pack_tensor(tensor, bits)


def unpack_values(packed: torch.Tensor, bits: int, shape) -> torch.Tensor:
    return unpack_tensor(packed, bits, tuple(shape))


__all__ = ["quantize_per_head_cuda", "pack_values", "unpack_values"]
