"""The benchmark's configurations (8B-shape batch 16 x 8192, long context 131072, 70B shape) at their full sizes (one layer each), checked through properties that
do not need the oracle to walk the whole input, plus the oracle itself on a slice it finishes in seconds:
  * the fp16-query kernel and the fp32-query ("precise") kernel are two different instruction paths; their
    outputs must agree within the attention tolerance;
  * splitting the keys of a sequence into two stores and folding the two (max, sum, out) results with the
    log-sum-exp rule must reproduce the single-store output (split-KV invariance);
  * a round trip through requantise/repack with unchanged widths leaves every byte in place;
  * the oracle on one (sequence, KV head) of the full-size input.
"""
import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc
from smartkv_b200 import sharding
from smartkv_b200.store import PackedKVStore, bucket_capacities
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu


def _fill(store, B, n, hkv, d, bits, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    dst = store.plan_bulk(bits)
    k = torch.randn((B * n, hkv, d), generator=gen, device="cuda")
    v = torch.randn((B * n, hkv, d), generator=gen, device="cuda")
    k[:, :, :4] *= 8.0
    v[:, :, 4:8] *= 8.0
    store.append(0, k, v, dst[0], dst[1], dst[2])
    return k.view(B, n, hkv, d), v.view(B, n, hkv, d)


def _bits(B, n, seed, probs=(0.08, 0.37, 0.08, 0.47)):
    g = torch.Generator(device="cuda").manual_seed(seed)
    idx = torch.multinomial(torch.tensor(probs, device="cuda"), B * n, replacement=True, generator=g).view(B, n)
    lut = torch.tensor([2, 3, 4, 8], device="cuda")
    bits = lut[idx]
    bits[:, :4] = 8
    return bits


def _attend(store, q, ck=None, cv=None):
    out = store.attention(0, q, ck, cv).clone()
    store.check_errors()
    return out, store.lse_max.clone(), store.lse_sum.clone()


@pytest.mark.parametrize("name,B,n,hq,hkv,d", [("config1", 16, 8192, 32, 8, 128), ("config3", 1, 131072, 32, 8, 128),
                                               ("config4_per_gpu", 64, 16384, 8, 1, 128)])
def test_full_size_properties(name, B, n, hq, hkv, d):
    caps = bucket_capacities(n, None, d)
    store = PackedKVStore(1, B, hkv, d, hq, caps, device="cuda", track_importance=False)
    bits = _bits(B, n, seed=len(name))
    k, v = _fill(store, B, n, hkv, d, bits, seed=7)
    gen = torch.Generator(device="cuda").manual_seed(11)
    q32 = torch.randn((B, hq, d), generator=gen, device="cuda")
    q16 = q32.half()
    ck = torch.randn((B, hkv, d), generator=gen, device="cuda")
    cv = torch.randn((B, hkv, d), generator=gen, device="cuda")
    out16, m16, l16 = _attend(store, q16, ck, cv)
    out32, m32, l32 = _attend(store, q16.float(), ck, cv)        # same values, the other kernel
    assert_close(out16.cpu().numpy(), out32.cpu().numpy(), what=f"{name}: fp16-query vs fp32-query kernel")
    assert torch.isfinite(out16).all()

    # the oracle on sequence 0, KV head 0 of the full-size input
    g = hq // hkv
    kb, vb, bb = k[0, :, :1].cpu().numpy(), v[0, :, :1].cpu().numpy(), bits[0].cpu().numpy()
    kq = np.empty(kb.shape, np.int8); vq = np.empty(kb.shape, np.int8)
    ks = np.empty(kb.shape[:2], np.float32); vs = np.empty(kb.shape[:2], np.float32)
    for w in (2, 3, 4, 8):
        sel = bb == w
        kq[sel], ks[sel] = orc.quantize_rows(kb[sel], w)
        vq[sel], vs[sel] = orc.quantize_rows(vb[sel], w)
    e = lambda x: orc.expand_gqa(x, g)
    ref, _ = orc.streaming_attention(q32[0, :g].cpu().numpy()[None, :, None, :], e(kq), e(ks), e(vq), e(vs),
                                     tile_size=8192, current_k=e(ck[0, :1].cpu().numpy()[None]),
                                     current_v=e(cv[0, :1].cpu().numpy()[None]))
    assert_close(out32[0, :g].cpu().numpy(), ref[0, :, 0], what=f"{name}: oracle on (sequence 0, head 0)")

    # split-KV invariance: first and second half of every sequence in separate stores
    half = n // 2
    parts = []
    for lo, hi in ((0, half), (half, n)):
        s2 = PackedKVStore(1, B, hkv, d, hq, bucket_capacities(hi - lo, None, d), device="cuda", track_importance=False)
        dst = s2.plan_bulk(bits[:, lo:hi].contiguous())
        s2.append(0, k[:, lo:hi].reshape(-1, hkv, d).contiguous(), v[:, lo:hi].reshape(-1, hkv, d).contiguous(),
                  dst[0], dst[1], dst[2])
        o, m, l = _attend(s2, q16)                  # no current token: it would be counted twice
        parts.append((m, l, o * l[..., None]))
        del s2
    ms, ls, os_ = (torch.stack([p[i] for p in parts]) for i in range(3))
    M = ms.max(0).values
    w = torch.exp2(ms - M)
    folded = (os_ * w[..., None]).sum(0) / (ls * w).sum(0)[..., None]
    whole, _, _ = _attend(store, q16)
    assert_close(folded.cpu().numpy(), whole.cpu().numpy(), what=f"{name}: split-KV fold")
    single, M1, L1 = sharding.combine_partials(ms[0], ls[0], os_[0])
    assert torch.allclose(single, parts[0][2] / parts[0][1][..., None])

    # repack with unchanged widths: nothing moves
    before = store.arena.clone()
    new_bits = torch.zeros((B, store.slots), dtype=torch.uint8, device="cuda")
    for i, w in enumerate((2, 3, 4, 8)):
        cnt = store.counts[:, i]
        pos = torch.arange(store.caps[i], device="cuda")[None, :] < cnt[:, None]
        new_bits[:, store.bucket_base[i]: store.bucket_base[i] + store.caps[i]][pos] = w
    store.repack(new_bits)
    store.check_errors()
    assert int(store._realloc["n_moves"].sum()) == 0 and torch.equal(store.arena, before)
