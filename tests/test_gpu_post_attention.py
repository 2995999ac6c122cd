"""skv_post_attention (combine + importance + append in one launch) against the three separate calls."""
import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc
from tests.gpu_util import fill_store, make_store

pytestmark = pytest.mark.gpu


def _pair(B, hq, hkv, d, n, L, seed):
    stores = []
    rng = np.random.default_rng(seed)
    bits = rng.choice((2, 3, 4, 8), size=(B, n))
    kvs = []
    for l in range(L):
        k, v = orc.synth_kv(B * n, hkv, d, seed=seed * 10 + l)
        kvs.append((k.reshape(B, n, hkv, d), v.reshape(B, n, hkv, d)))
    for _ in range(3):
        s = make_store(L, B, hkv, d, hq, n + 8)
        fill_store(s, kvs, bits)
        stores.append(s)
    return stores, rng


@pytest.mark.parametrize("hq,hkv,d,q_dtype", [(32, 8, 128, np.float16), (8, 2, 64, np.float32), (6, 2, 128, np.float16),
                                              (4, 4, 64, np.float16)])
def test_fused_post_attention_equals_separate_calls(hq, hkv, d, q_dtype):
    _fused_equals_separate(3, hq, hkv, d, 700, q_dtype)


def test_fused_post_attention_large_batch_takes_the_wide_importance_blocks():
    """80 sequences x 18 live chunks exceed two waves of importance blocks, so the fused launch switches to blocks of four
    chunks (four keys per thread, their loads in flight together); the stand-alone importance kernel keeps one.  The
    per-key sums run in the same order either way, so every importance array must come out the same."""
    _fused_equals_separate(80, 4, 1, 64, 2000, np.float16)


def _fused_equals_separate(B, hq, hkv, d, n, q_dtype):
    L = 2
    (a, b, c), rng = _pair(B, hq, hkv, d, n, L, seed=hq + d)
    for step in range(3):
        plan_a, plan_b, plan_c = a.plan_step(), b.plan_step(), c.plan_step()
        outs_a, outs_c = [], [torch.empty((B, hq, d), dtype=torch.float32, device="cuda") for _ in range(L)]
        for l in range(L):
            q = torch.from_numpy(rng.standard_normal((B, hq, d)).astype(q_dtype)).cuda()
            ck = torch.from_numpy(rng.standard_normal((B, hkv, d)).astype(np.float32)).cuda()
            cv = torch.from_numpy(rng.standard_normal((B, hkv, d)).astype(np.float32)).cuda()
            out_a = a.attention(l, q, ck, cv, update_importance=True, cur_storage=plan_a[3]).clone()
            a.append(l, ck, cv, plan_a[0], plan_a[1], plan_a[2])
            out_b = b.decode_layer(l, q, ck, cv, plan_b, update_importance=True).clone()
            # third store: the post-attention launch on a side stream, overlapping the next layer's attention
            c.decode_layer(l, q, ck, cv, plan_c, update_importance=True, out=outs_c[l], overlap=True)
            outs_a.append(out_a)
            assert torch.equal(out_a, out_b), (step, l)
            assert torch.equal(a.lse_max, b.lse_max) and torch.equal(a.lse_sum, b.lse_sum)
            assert torch.equal(a.cur_prob, b.cur_prob)
        a.commit_step(plan_a)
        b.commit_step(plan_b)
        c.commit_step(plan_c)
        a.check_errors(); b.check_errors(); c.check_errors()
        for l in range(L):
            assert torch.equal(outs_a[l], outs_c[l]), (step, l, "overlap")
        assert torch.equal(a.cumulative, c.cumulative) or torch.allclose(a.cumulative, c.cumulative, rtol=1e-6, atol=1e-12)
        assert torch.allclose(a.layer_ema, c.layer_ema, rtol=1e-5, atol=1e-9) and torch.equal(a.touched, c.touched)
        assert torch.equal(a.counts, b.counts) and torch.equal(a.counts, c.counts)
        assert torch.allclose(a.cumulative, b.cumulative, rtol=1e-6, atol=1e-12)
        assert torch.allclose(a.layer_ema, b.layer_ema, rtol=1e-5, atol=1e-9)
        assert torch.equal(a.touched, b.touched)
        assert torch.allclose(a.head_state, b.head_state, rtol=1e-6)
    assert torch.equal(a.arena, b.arena) and torch.equal(a.arena, c.arena)   # the appended rows are byte-identical


def test_fused_post_attention_without_importance_or_append():
    (a, b, _), rng = _pair(2, 8, 2, 128, 300, 1, seed=3)
    q = torch.from_numpy(rng.standard_normal((2, 8, 128)).astype(np.float16)).cuda()
    ck = torch.from_numpy(rng.standard_normal((2, 2, 128)).astype(np.float32)).cuda()
    cv = torch.from_numpy(rng.standard_normal((2, 2, 128)).astype(np.float32)).cuda()
    out_a = a.attention(0, q, ck, cv).clone()
    out_b = b.decode_layer(0, q, ck, cv, b.plan_step(), update_importance=False).clone()
    assert torch.equal(out_a, out_b)
    assert float(b.cumulative.abs().sum()) == 0.0
