"""skv_decode_attention_static: attention whose partials live in the library's fixed device
array.  Collected last on purpose: it has to give the same answer as the caller-buffer entry
point whether it is the first attention launch of the process or runs after every other test."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc
from smartkv_b200 import _lib
from smartkv_b200._lib import check, ptr
from tests.gpu_util import fill_store, make_store

pytestmark = pytest.mark.gpu

STATIC_LIMIT = 16 << 20


def _filled_store(seed, B=3, n=700, hq=8, hkv=2, d=128):
    rng = np.random.default_rng(seed)
    store = make_store(1, B, hkv, d, hq, n)
    kv = [orc.synth_kv(B * n, hkv, d, seed=seed + 1)]
    k = kv[0][0].reshape(B, n, hkv, d)
    v = kv[0][1].reshape(B, n, hkv, d)
    bits = rng.choice((2, 3, 4, 8), size=(B, n))
    fill_store(store, [(k, v)], bits)
    store.build_plan()
    return store, rng


def _combine(store, q, partials_ptr, cur_k, cur_v):
    out = torch.empty((store.num_seqs, store.num_q_heads, store.head_dim), dtype=torch.float32, device="cuda")
    lmax = torch.empty((store.num_seqs, store.num_q_heads), dtype=torch.float32, device="cuda")
    lsum = torch.empty_like(lmax)
    cprob = torch.empty_like(lmax)
    check(store.lib.skv_lse_combine(ctypes.byref(store.desc), ptr(store.plan), ptr(q), _lib.DTYPE_F16,
                                    store.num_q_heads, partials_ptr, store.num_ctas, ptr(cur_k), ptr(cur_v),
                                    _lib.DTYPE_F32, ptr(out), ptr(lmax), ptr(lsum), ptr(cprob), store._stream()),
          "skv_lse_combine")
    return out, lmax, lsum, cprob


def _reference_call(store, q, logits, cur_k, cur_v):
    check(store.lib.skv_decode_attention(ctypes.byref(store.desc), ptr(store.arena), 0, ptr(store.plan), ptr(q),
                                         _lib.DTYPE_F16, store.num_q_heads, ptr(store.partials), store.num_ctas,
                                         ptr(logits), ptr(store.err), store._stream()), "skv_decode_attention")
    return _combine(store, q, ptr(store.partials), cur_k, cur_v)


def _static_call(store, q, logits, cur_k, cur_v):
    where = ctypes.c_void_p(0)
    check(store.lib.skv_decode_attention_static(ctypes.byref(store.desc), ptr(store.arena), 0, ptr(store.plan),
                                                ptr(q), _lib.DTYPE_F16, store.num_q_heads, store.num_ctas,
                                                ptr(logits), ptr(store.err), ctypes.byref(where), store._stream()),
          "skv_decode_attention_static")
    assert where.value, "the entry point must report where the partials are"
    return _combine(store, q, where, cur_k, cur_v), where.value


def test_static_scratch_matches_caller_buffer_twice_in_a_row():
    store, rng = _filled_store(seed=71)
    B, hq, hkv, d = store.num_seqs, store.num_q_heads, store.num_kv_heads, store.head_dim
    addresses = []
    for call in range(2):  # two calls in a row, different queries: leftovers of call 0 must not leak into call 1
        q = torch.from_numpy(rng.standard_normal((B, hq, d)).astype(np.float16)).cuda()
        ck = torch.from_numpy(rng.standard_normal((B, hkv, d)).astype(np.float32)).cuda()
        cv = torch.from_numpy(rng.standard_normal((B, hkv, d)).astype(np.float32)).cuda()
        logits_a = torch.zeros((B, hq, store.desc.slots), dtype=torch.float32, device="cuda")
        logits_b = torch.zeros_like(logits_a)
        got, where = _static_call(store, q, logits_b, ck, cv)
        want = _reference_call(store, q, logits_a, ck, cv)
        store.check_errors()
        addresses.append(where)
        for g, w, name in zip(got, want, ("out", "lse_max", "lse_sum", "cur_prob")):
            assert torch.equal(g, w), f"call {call}: {name} differs from the caller-buffer entry point"
        assert torch.equal(logits_a, logits_b), f"call {call}: logits differ"
        assert torch.isfinite(got[0]).all()
    assert addresses[0] == addresses[1], "one fixed array per device"


def test_static_scratch_after_a_smaller_shape():
    # a second store with fewer, shorter sequences reuses the same array: stale partials of the
    # larger launch above must not be read
    store, rng = _filled_store(seed=72, B=1, n=130, hq=4, hkv=1, d=64)
    B, hq, hkv, d = store.num_seqs, store.num_q_heads, store.num_kv_heads, store.head_dim
    q = torch.from_numpy(rng.standard_normal((B, hq, d)).astype(np.float16)).cuda()
    ck = torch.from_numpy(rng.standard_normal((B, hkv, d)).astype(np.float32)).cuda()
    cv = torch.from_numpy(rng.standard_normal((B, hkv, d)).astype(np.float32)).cuda()
    got, _ = _static_call(store, q, None, ck, cv)
    want = _reference_call(store, q, None, ck, cv)
    store.check_errors()
    for g, w in zip(got, want):
        assert torch.equal(g, w)


def test_static_scratch_rejects_shapes_beyond_its_limit():
    store, rng = _filled_store(seed=73, B=1, n=130, hq=4, hkv=1, d=64)
    big = _lib.StoreDesc()
    ctypes.memmove(ctypes.byref(big), ctypes.byref(store.desc), ctypes.sizeof(big))
    big.num_seqs = 1024
    big.num_kv_heads = 8
    hq = 64
    need = int(store.lib.skv_attn_partials_bytes(ctypes.byref(big), hq, store.num_ctas))
    assert need > STATIC_LIMIT
    q = torch.zeros((1, hq, 64), dtype=torch.float16, device="cuda")
    where = ctypes.c_void_p(123)
    rc = store.lib.skv_decode_attention_static(ctypes.byref(big), ptr(store.arena), 0, ptr(store.plan), ptr(q),
                                               _lib.DTYPE_F16, hq, store.num_ctas, None, ptr(store.err),
                                               ctypes.byref(where), store._stream())
    assert rc == -3  # SKV_ERR_CAPACITY: nothing was launched
    assert not where.value
    torch.cuda.synchronize()
    store.check_errors()
