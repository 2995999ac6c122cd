"""GPU parity of quantize / pack / append against the CPU oracle: bit-exact."""
import ctypes
import hashlib

import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc

pytestmark = pytest.mark.gpu


def _lib():
    from smartkv_b200 import _lib
    return _lib


def _quantize_gpu(x, bits):
    L = _lib()
    xt = torch.from_numpy(x).cuda().contiguous()
    rows = xt.numel() // xt.shape[-1]
    codes = torch.empty(xt.shape, dtype=torch.int8, device="cuda")
    scales = torch.empty(xt.shape[:-1], dtype=torch.float32, device="cuda")
    code = L.DTYPE_F32 if xt.dtype == torch.float32 else L.DTYPE_F16
    L.check(L.lib().skv_quantize_per_head(L.ptr(xt), code, rows, xt.shape[-1], bits, L.ptr(codes), L.ptr(scales),
                                          L.stream_ptr()))
    torch.cuda.synchronize()
    return codes.cpu().numpy(), scales.cpu().numpy()


@pytest.mark.parametrize("tag", ["a", "b"])
@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_quantize_golden_bit_exact(golden, tag, bits):
    g = golden("quant")
    for name in ("k", "v"):
        q, s = _quantize_gpu(g[f"quant_{tag}_{name}"], bits)
        assert np.array_equal(q, g[f"quant_{tag}_{name}q{bits}"])
        assert np.array_equal(s.view(np.uint32), g[f"quant_{tag}_{name}s{bits}"].view(np.uint32))


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("d", [64, 128, 80])
def test_quantize_random_vs_oracle(bits, d):
    rng = np.random.default_rng(bits * 100 + d)
    x = (rng.standard_normal((777, d)) * rng.choice([1e-3, 1.0, 50.0], size=(777, 1))).astype(np.float32)
    x[5] = 0
    x[6, :] = np.round(x[6] * 4) / 4
    q, s = _quantize_gpu(x, bits)
    qo, so = orc.quantize_rows(x, bits)
    assert np.array_equal(q, qo)
    assert np.array_equal(s.view(np.uint32), so.view(np.uint32))


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("d", [64, 128])
def test_quantize_near_ties_and_extreme_scales(bits, d):
    """Values whose quotient x / scale sits on or next to a half-integer, and rows whose scale is
    tiny, huge or subnormal: the kernel's reciprocal-multiply shortcut must fall back to the IEEE
    division exactly where the two could round differently."""
    rng = np.random.default_rng(900 + bits + d)
    levels = max(2 ** (bits - 1) - 1, 1)
    rows = []
    for amax in (1.0, 3.0, 0.7310585, 127.0, 1e-3, 6.1e-5, 2.5e7, 1e-33, 1e33, 3e-39, 1e-44):
        amax = np.float32(amax)
        s = np.float32(amax / np.float32(levels))
        for _ in range(24):
            k = rng.integers(-levels, levels, size=d).astype(np.float32)
            delta = rng.choice([0.0, 1e-7, -1e-7, 1e-6, -1e-6, 3e-5, -3e-5, 1.2e-4, -1.2e-4, 1.3e-4, -1.3e-4, 4e-4],
                               size=d).astype(np.float32)
            x = ((k + np.float32(0.5) + delta) * s).astype(np.float32)
            x = np.clip(x, -amax, amax)
            x[rng.integers(0, d)] = amax * rng.choice([-1.0, 1.0])   # pins the row's absolute maximum
            rows.append(x.astype(np.float32))
    x = np.stack(rows)
    q, s = _quantize_gpu(x, bits)
    with np.errstate(all="ignore"):
        qo, so = orc.quantize_rows(x, bits)
    assert np.array_equal(s.view(np.uint32), so.view(np.uint32))
    assert np.array_equal(q, qo)


def test_quantize_fp16_input():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((300, 128)).astype(np.float16)
    q, s = _quantize_gpu(x, 4)
    qo, so = orc.quantize_rows(x.astype(np.float32), 4)
    assert np.array_equal(q, qo) and np.array_equal(s, so)


def test_quantize_bulk_digest_matches_reference(golden):
    g = golden("quant")
    k, _ = orc.synth_kv(512, 8, 128, seed=3)
    for bits in (2, 3, 4, 8):
        q, s = _quantize_gpu(k, bits)
        sha = lambda a: np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8)
        assert np.array_equal(sha(q), g[f"quant_bulk_sha_kq{bits}"])
        assert np.array_equal(sha(s), g[f"quant_bulk_sha_ks{bits}"])


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("n", [1, 3, 8, 17, 100, 1000, 4096 + 5])
def test_pack_unpack_vs_oracle(bits, n):
    L = _lib()
    lo, hi = orc.code_range(bits)
    rng = np.random.default_rng(n + bits)
    codes = rng.integers(lo, hi + 1, size=n).astype(np.int8)
    ct = torch.from_numpy(codes).cuda()
    packed = torch.zeros(orc.packed_size(n, bits), dtype=torch.uint8, device="cuda")
    L.check(L.lib().skv_pack(L.ptr(ct), n, bits, L.ptr(packed), L.stream_ptr()))
    assert np.array_equal(packed.cpu().numpy(), orc.pack_codes(codes, bits))
    back = torch.empty(n, dtype=torch.int8, device="cuda")
    L.check(L.lib().skv_unpack(L.ptr(packed), n, bits, L.ptr(back), L.stream_ptr()))
    assert np.array_equal(back.cpu().numpy(), codes)


def test_pack_empty_and_bad_args():
    L = _lib()
    t = torch.zeros(4, dtype=torch.int8, device="cuda")
    p = torch.zeros(4, dtype=torch.uint8, device="cuda")
    assert L.lib().skv_pack(L.ptr(t), 0, 2, L.ptr(p), L.stream_ptr()) == 0
    assert L.lib().skv_pack(L.ptr(t), 4, 5, L.ptr(p), L.stream_ptr()) < 0
    assert L.lib().skv_pack(None, 4, 2, L.ptr(p), L.stream_ptr()) < 0


@pytest.mark.parametrize("hkv,d", [(4, 64), (8, 128)])
def test_append_then_export_bit_exact(hkv, d):
    from tests.gpu_util import fill_store, make_store, oracle_quantized
    B, n, Lyr = 2, 333, 2
    rng = np.random.default_rng(7)
    bits = rng.choice([2, 3, 4, 8], size=(B, n))
    store = make_store(Lyr, B, hkv, d, hkv * 4, n)
    kv = []
    for layer in range(Lyr):
        ks, vs = zip(*[orc.synth_kv(n, hkv, d, seed=10 * layer + b) for b in range(B)])
        kv.append((np.stack(ks), np.stack(vs)))
    fill_store(store, kv, bits)
    torch.cuda.synchronize()
    assert store.counts.cpu().numpy().tolist() == [[int((bits[b] == w).sum()) for w in (2, 3, 4, 8)] for b in range(B)]
    for layer in range(Lyr):
        for b in range(B):
            ids, wb, kc, vc, ksc, vsc = store.export_sequence(layer, b)
            assert np.array_equal(ids.cpu().numpy(), np.arange(n))
            assert np.array_equal(wb.cpu().numpy(), bits[b])
            kq, vq, kso, vso = oracle_quantized(kv[layer][0][b], kv[layer][1][b], bits[b])
            assert np.array_equal(kc.cpu().numpy(), kq)
            assert np.array_equal(vc.cpu().numpy(), vq)
            assert np.array_equal(ksc.cpu().numpy().view(np.uint32), kso.view(np.uint32))
            assert np.array_equal(vsc.cpu().numpy().view(np.uint32), vso.view(np.uint32))
            # raw packed bytes of every bucket equal the oracle's row packing
            for bi, w in enumerate((2, 3, 4, 8)):
                sel = np.nonzero(bits[b] == w)[0]
                kr, vr, _, _ = store.bucket_rows(layer, b, bi)
                want_k = orc.pack_rows(kq[sel], w).transpose(1, 0, 2)
                want_v = orc.pack_rows(vq[sel], w).transpose(1, 0, 2)
                assert np.array_equal(kr.cpu().numpy(), want_k)
                assert np.array_equal(vr.cpu().numpy(), want_v)
