"""Mirror of ``smartkv.kernels.bit_packing`` (pack_tensor / unpack_tensor and the size helpers,
smartkv/kernels/bit_packing.py:24-160) over ``skv_pack`` / ``skv_unpack``.

Same names, arguments, error messages and byte format (smartkv/csrc/bit_packing.cu).  The
reference falls back to an uncompressed uint8 cast when its extension is missing or the tensor is
on the CPU; here a non-CUDA tensor is an error: there is no CPU path.
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from .. import _lib
from .._lib import check, ptr

CUDA_AVAILABLE = True


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need_cuda(t: torch.Tensor, what: str):
    if t.device.type != "cuda":
        raise _lib.SmartKVLibraryError(f"{what}: tensor is on {t.device}; the B200 library has no CPU path")


_WIDTHS = (2, 3, 4, 8)
# values per group and bytes per group of every width: 4 crumbs, 8 three-bit fields, 2 nibbles or 1 byte
_GROUP = {2: (4, 1), 3: (8, 3), 4: (2, 1), 8: (1, 1)}


def _bad_width(bits) -> ValueError:
    return ValueError(f"bits must be 2, 3, 4, or 8, got {bits}")       # the reference's message


def compute_packed_size(num_elements: int, bits: int) -> int:
    """Bytes of ``num_elements`` packed values (smartkv/kernels/bit_packing.py:102-122)."""
    if bits not in _GROUP:
        raise _bad_width(bits)
    per_group, group_bytes = _GROUP[bits]
    return -(-num_elements // per_group) * group_bytes


def pack_tensor(tensor: torch.Tensor, bits: int) -> torch.Tensor:
    """int8 tensor -> flat packed uint8 tensor (8 bits: returned unchanged, contiguous)."""
    if tensor.dtype != torch.int8:
        raise ValueError(f"Input must be int8, got {tensor.dtype}")
    if bits not in _WIDTHS:
        raise _bad_width(bits)
    src = tensor.contiguous()
    if bits == 8:
        return src
    _need_cuda(src, "pack_tensor")
    n = src.numel()
    out = torch.empty(compute_packed_size(n, bits), dtype=torch.uint8, device=src.device)
    if n:
        check(_lib.lib().skv_pack(ptr(src), n, bits, ptr(out), _stream(src)), "skv_pack")
    return out


def unpack_tensor(packed: torch.Tensor, bits: int, shape: Tuple[int, ...]) -> torch.Tensor:
    """Packed uint8 tensor -> int8 tensor of ``shape``."""
    if bits not in _WIDTHS:
        raise _bad_width(bits)
    if bits == 8:
        if packed.dtype not in (torch.uint8, torch.int8):
            raise ValueError(f"Packed tensor must be uint8/int8 for 8-bit, got {packed.dtype}")
        return packed.view(shape).to(torch.int8)
    if packed.dtype != torch.uint8:
        raise ValueError(f"Packed tensor must be uint8, got {packed.dtype}")
    _need_cuda(packed, "unpack_tensor")
    n = 1
    for extent in shape:
        n *= int(extent)
    src = packed.contiguous()
    need = compute_packed_size(n, bits)
    if src.numel() < need:
        raise ValueError(f"packed tensor holds {src.numel()} bytes, shape {tuple(shape)} at {bits} bits needs {need}")
    out = torch.empty(n, dtype=torch.int8, device=src.device)
    if n:
        check(_lib.lib().skv_unpack(ptr(src), n, bits, ptr(out), _stream(src)), "skv_unpack")
    return out.view(tuple(shape))


def get_compression_ratio(bits: int) -> float:
    """Compression against int8 storage (smartkv/kernels/bit_packing.py:125-140)."""
    if bits not in _WIDTHS:
        raise _bad_width(bits)
    return 8.0 / bits


def get_memory_savings_vs_fp16(bits: int) -> float:
    """Memory as a fraction of fp16 storage, e.g. 0.125 for 2 bits (smartkv/kernels/bit_packing.py:143-160)."""
    if bits not in _WIDTHS:
        raise _bad_width(bits)
    return bits / 16.0
