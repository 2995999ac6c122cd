"""Helpers shared by the GPU parity tests (all compute goes through the C ABI)."""
import numpy as np
import torch

from oracle import smartkv_oracle as orc
from smartkv_b200.store import PackedKVStore, round_up


def make_store(num_layers, num_seqs, hkv, d, hq, max_tokens, **kw):
    cap = round_up(max_tokens + 1, 128)
    return PackedKVStore(num_layers, num_seqs, hkv, d, hq, (cap, cap, cap, cap), device="cuda", **kw)


def fill_store(store, layer_kv, bits):
    """layer_kv: list over layers of (k, v) numpy [B, n, Hkv, D]; bits numpy int [B, n]."""
    B, n = bits.shape
    bt = torch.from_numpy(bits.astype(np.int64)).cuda()
    dst_seq, dst_bucket, dst_pos, storage = store.plan_bulk(bt)
    for layer, (k, v) in enumerate(layer_kv):
        kt = torch.from_numpy(k).cuda().reshape(B * n, store.num_kv_heads, store.head_dim)
        vt = torch.from_numpy(v).cuda().reshape(B * n, store.num_kv_heads, store.head_dim)
        store.append(layer, kt, vt, dst_seq, dst_bucket, dst_pos)
    return storage


def oracle_quantized(k, v, bits):
    """Per-token widths -> (kq, vq, ks, vs) numpy in token order for one sequence [n,Hkv,D]."""
    kq = np.empty(k.shape, np.int8)
    vq = np.empty(v.shape, np.int8)
    ks = np.empty(k.shape[:2], np.float32)
    vs = np.empty(k.shape[:2], np.float32)
    for w in (2, 3, 4, 8):
        sel = bits == w
        if sel.any():
            kq[sel], ks[sel] = orc.quantize_rows(k[sel], w)
            vq[sel], vs[sel] = orc.quantize_rows(v[sel], w)
    return kq, vq, ks, vs


def oracle_attention(q, kq, vq, ks, vs, group, cur_k=None, cur_v=None):
    """q [Hq, D]; quantized cache of one sequence; returns (out [Hq, D], probs [Hq, n(+1)])."""
    e = lambda x: orc.expand_gqa(x, group)
    o, p = orc.streaming_attention(q[None, :, None, :], e(kq), e(ks), e(vq), e(vs), tile_size=2048,
                                   current_k=None if cur_k is None else e(cur_k[None]),
                                   current_v=None if cur_v is None else e(cur_v[None]))
    return o[0, :, 0], p[0, :, 0]


def assert_close(got, ref, atol=2e-3, rtol=1e-3, what=""):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    err = np.abs(got - ref)
    tol = atol + rtol * np.abs(ref)
    assert np.all(err <= tol), f"{what}: max abs err {err.max():.3e}, worst excess {(err - tol).max():.3e}"
