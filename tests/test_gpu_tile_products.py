"""The tensor-core fragment path (register unpack + mma.sync) on integer inputs: exact.

The hooks that expose single tile products are not part of the product library: this file compiles
tests/csrc/tile_hooks.cu (which includes the kernel's own fragment header) into a test-only library."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def hooks():
    src = os.path.join(HERE, "csrc", "tile_hooks.cu")
    out_dir = os.path.join(HERE, "_build")
    lib = os.path.join(out_dir, "libskv_tile_hooks.so")
    os.makedirs(out_dir, exist_ok=True)
    deps = [src] + [os.path.join(HERE, "..", "smartkv_b200", "csrc", f) for f in ("attn_frag.cuh", "common.cuh")]
    if not os.path.exists(lib) or any(os.path.getmtime(d) > os.path.getmtime(lib) for d in deps):
        subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
                        "-shared", src, "-o", lib], check=True)
    h = ctypes.CDLL(lib)
    h.skv_test_tile_products.restype = ctypes.c_int
    h.skv_test_tile_products.argtypes = [ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 7
    h.skv_test_tile_scores_i8.restype = ctypes.c_int
    h.skv_test_tile_scores_i8.argtypes = [ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 4
    return h


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_tile_products_exact(d, bits, hooks):
    from smartkv_b200 import _lib as L
    lo, hi = orc.code_range(bits)
    for seed in range(3):
        rng = np.random.default_rng(seed * 10 + bits + d)
        kc = rng.integers(lo, hi + 1, size=(16, d)).astype(np.int8)
        vc = rng.integers(lo, hi + 1, size=(16, d)).astype(np.int8)
        if seed == 0:      # every code value appears, extremes included
            kc.reshape(-1)[: hi - lo + 1] = np.arange(lo, hi + 1)
            vc.reshape(-1)[-(hi - lo + 1):] = np.arange(lo, hi + 1)
        q = rng.integers(-3, 4, size=(16, d)).astype(np.float16)
        p = rng.integers(-2, 3, size=(16, 16)).astype(np.float16)
        kr = torch.from_numpy(orc.pack_rows(kc, bits)).cuda().contiguous()
        vr = torch.from_numpy(orc.pack_rows(vc, bits)).cuda().contiguous()
        qt, pt = torch.from_numpy(q).cuda(), torch.from_numpy(p).cuda()
        scores = torch.empty((8, 16), dtype=torch.float32, device="cuda")
        out = torch.empty((8, d), dtype=torch.float32, device="cuda")
        L.check(hooks.skv_test_tile_products(d, bits, L.ptr(kr), L.ptr(vr), L.ptr(qt), L.ptr(pt), L.ptr(scores),
                                                L.ptr(out), L.stream_ptr()))
        torch.cuda.synchronize()
        # rows 0..7 = heads of the group, rows 8..15 = the residual rows of the precise mode
        want_s = (q[:8].astype(np.float64) + q[8:].astype(np.float64)) @ kc.astype(np.float64).T
        want_o = (p[:8].astype(np.float64) + p[8:].astype(np.float64)) @ vc.astype(np.float64)
        assert np.array_equal(scores.cpu().numpy().astype(np.float64), want_s), (d, bits, "scores")
        assert np.array_equal(out.cpu().numpy().astype(np.float64), want_o), (d, bits, "out")


@pytest.mark.parametrize("d,bits", [(64, 2), (64, 4), (64, 8), (128, 2), (128, 3), (128, 4), (128, 8)])
def test_tile_scores_int8_exact(d, bits, hooks):
    """The int8 tensor-core path used for 2/4/8-bit keys (and 3-bit keys at head_dim 128): exact int32 dot products."""
    from smartkv_b200 import _lib as L
    lo, hi = orc.code_range(bits)
    for seed in range(3):
        rng = np.random.default_rng(seed * 7 + bits + d)
        kc = rng.integers(lo, hi + 1, size=(16, d)).astype(np.int8)
        if seed == 0:
            kc.reshape(-1)[: hi - lo + 1] = np.arange(lo, hi + 1)
        q = rng.integers(-128, 128, size=(8, d)).astype(np.int8)
        kr = torch.from_numpy(orc.pack_rows(kc, bits)).cuda().contiguous()
        qt = torch.from_numpy(q).cuda()
        scores = torch.empty((8, 16), dtype=torch.int32, device="cuda")
        L.check(hooks.skv_test_tile_scores_i8(d, bits, L.ptr(kr), L.ptr(qt), L.ptr(scores), L.stream_ptr()))
        torch.cuda.synchronize()
        stored = kc.astype(np.int64) + (0 if bits == 8 else (1 << (bits - 1)))
        want = q.astype(np.int64) @ stored.T
        assert np.array_equal(scores.cpu().numpy().astype(np.int64), want), (d, bits)
