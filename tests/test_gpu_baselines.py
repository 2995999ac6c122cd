"""The comparison caches (uniform INT8 / INT4, KIVI with per-token scales) on the packed store: values read
back must equal the reference's bit for bit (fixture tests/golden/baselines.npz, produced by the reference's own
classes), and the packed decode kernels over those rows must match the oracle's dequantise-then-attend."""
import os

import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu
Z = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "baselines.npz")


def make(tag, L, H, D, hq):
    from smartkv_b200.baselines import KIVICache, UniformQuantCache
    if tag == "u8":
        return UniformQuantCache(L, H, D, bits=8, max_tokens=100, num_query_heads=hq)
    if tag == "u4":
        return UniformQuantCache(L, H, D, bits=4, max_tokens=100, num_query_heads=hq)
    kb, vb = (2, 4) if tag == "kivi24" else (4, 2)
    return KIVICache(L, H, D, key_bits=kb, value_bits=vb, per_channel_keys=False, max_tokens=100, num_query_heads=hq)


@pytest.mark.parametrize("tag", ["u8", "u4", "kivi24", "kivi42"])
def test_baseline_cache_matches_reference_and_attends_on_packed_kernels(tag):
    z = np.load(Z)
    k, v = z["b_k"], z["b_v"]
    L, n, H, D = k.shape
    hq = 4 * H
    c = make(tag, L, H, D, hq)
    for l in range(L):
        if l == 0:      # token by token, as the reference is driven
            for t in range(n):
                c.quantize_and_store(l, t, torch.from_numpy(k[l, t]).cuda(), torch.from_numpy(v[l, t]).cuda())
        else:
            c.quantize_and_store_batch(l, list(range(n)), torch.from_numpy(k[l]).cuda(), torch.from_numpy(v[l]).cuda())
    assert len(c) == n and c.get_memory_stats()["memory_ratio"] == float(z[f"b_{tag}_ratio"])
    rng = np.random.default_rng(2)
    for l in range(L):
        kk, vv = c.retrieve_all(l)
        assert np.array_equal(kk.cpu().numpy(), z[f"b_{tag}_k{l}"]), (tag, l)
        assert np.array_equal(vv.cpu().numpy(), z[f"b_{tag}_v{l}"]), (tag, l)
        one_k, one_v = c.retrieve(l, 7)
        assert np.array_equal(one_k.cpu().numpy(), z[f"b_{tag}_k{l}"][7])
        q = rng.standard_normal((hq, D)).astype(np.float32)
        ck = rng.standard_normal((H, D)).astype(np.float32)
        cv = rng.standard_normal((H, D)).astype(np.float32)
        out = c.decode_attention(l, torch.from_numpy(q).cuda(), torch.from_numpy(ck).cuda(), torch.from_numpy(cv).cuda())
        c.store.check_errors()
        kd = np.concatenate([z[f"b_{tag}_k{l}"], ck[None]]).repeat(4, axis=1)
        vd = np.concatenate([z[f"b_{tag}_v{l}"], cv[None]]).repeat(4, axis=1)
        s = np.einsum("hd,nhd->hn", q, kd) / np.sqrt(D)
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        ref = np.einsum("hn,nhd->hd", p, vd)
        assert_close(out.cpu().numpy(), ref, 2e-3, 1e-3, f"{tag} layer {l}")
    with pytest.raises(KeyError):
        c.retrieve(0, n + 3)
    c.clear()
    assert len(c) == 0 and c.store.counts.sum().item() == 0


def test_unsupported_modes_say_so():
    from smartkv_b200.baselines import KIVICache, UniformQuantCache
    with pytest.raises(NotImplementedError):
        KIVICache(1, 4, 64)                       # per-channel key scales
    with pytest.raises(NotImplementedError):
        UniformQuantCache(1, 4, 64, bits=16)      # FP16 pass-through
    with pytest.raises(ValueError):
        UniformQuantCache(1, 4, 64, bits=3)
