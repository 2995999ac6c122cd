"""A decode step captured once as a CUDA graph and replayed many times must track the eager path: the cache
grows by one token per replay, so the launch scalars that depend on the token count (the number of
importance blocks) and on the step (the half of the double-buffered head state) must not be frozen at
their capture-time values."""
import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc
from smartkv_b200 import _lib
from tests.gpu_util import fill_store, make_store

pytestmark = pytest.mark.gpu


def build(L, B, hkv, d, hq, n, room):
    rng = np.random.default_rng(3)
    store = make_store(L, B, hkv, d, hq, n + room)
    kv = []
    for l in range(L):
        ks, vs = zip(*(orc.synth_kv(n, hkv, d, seed=10 * l + b) for b in range(B)))
        kv.append((np.stack(ks), np.stack(vs)))
    fill_store(store, kv, rng.choice([2, 3, 4, 8], size=(B, n)))
    return store


def decode_step(store, q, k, v, outs):
    plan = store.plan_step()
    for layer in range(store.num_layers):
        store.decode_layer(layer, q[layer], k[layer], v[layer], plan, update_importance=True, out=outs[layer])
    store.commit_step(plan)


def test_replayed_step_matches_eager_steps():
    L, B, hkv, d, hq, n, steps = 4, 3, 8, 128, 32, 300, 40       # 40 replays cross a 16-key tile and a 128-key block edge
    a, b = build(L, B, hkv, d, hq, n, steps + 8), build(L, B, hkv, d, hq, n, steps + 8)
    dev = "cuda"
    q = torch.zeros((L, B, hq, d), dtype=torch.float16, device=dev)
    k = torch.zeros((L, B, hkv, d), dtype=torch.float16, device=dev)
    v = torch.zeros_like(k)
    outs_a = torch.zeros((L, B, hq, d), dtype=torch.float32, device=dev)
    outs_b = torch.zeros_like(outs_a)
    gen = torch.Generator(device=dev).manual_seed(0)

    def new_inputs():
        q.copy_(torch.randn(q.shape, generator=gen, device=dev))
        k.copy_(torch.randn(k.shape, generator=gen, device=dev))
        v.copy_(torch.randn(v.shape, generator=gen, device=dev))

    # one eager step on both stores first (allocates the pipeline buffers outside the capture)
    new_inputs()
    decode_step(a, q, k, v, outs_a)
    decode_step(b, q, k, v, outs_b)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        decode_step(a, q, k, v, outs_a)
    # torch runs nothing while capturing: the captured step has not happened on store `a` yet
    for t in range(steps):
        new_inputs()
        graph.replay()
        a.max_seq_tokens += 1          # host-side mirror of what the replayed commit did on the device
        a.appended_total += B
        decode_step(b, q, k, v, outs_b)
        torch.cuda.synchronize()
        assert torch.equal(outs_a, outs_b), f"step {t}: max diff {float((outs_a - outs_b).abs().max())}"
    a.check_errors(); b.check_errors()
    assert torch.equal(a.counts, b.counts) and torch.equal(a.slot_token, b.slot_token)
    assert torch.equal(a.cumulative, b.cumulative)
    assert torch.equal(a.layer_ema, b.layer_ema)
    assert torch.equal(a.head_state[:, a.head_parity], b.head_state[:, b.head_parity])
    assert int(a.counts.sum()) == B * (n + 1 + steps)


def test_capture_of_an_odd_number_of_importance_updates_is_refused():
    L, B, hkv, d, hq, n = 3, 1, 8, 128, 32, 100
    store = build(L, B, hkv, d, hq, n, 16)
    q = torch.randn((L, B, hq, d), device="cuda").half()
    k = torch.randn((L, B, hkv, d), device="cuda").half()
    v = torch.randn((L, B, hkv, d), device="cuda").half()
    outs = torch.zeros((L, B, hq, d), dtype=torch.float32, device="cuda")
    decode_step(store, q, k, v, outs)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with pytest.raises(_lib.SmartKVLibraryError, match="even number"):
        with torch.cuda.graph(graph):
            decode_step(store, q, k, v, outs)
    torch.cuda.synchronize()
    # the store is still usable without a graph
    decode_step(store, q, k, v, outs)
    store.check_errors()
    assert int(store.counts.sum()) >= n + 2


def test_token_capacity_bounds_the_captured_importance_grid():
    """With ``token_capacity`` stated, a captured step launches importance blocks for that many tokens instead of
    every storage index; the replays must still match the eager steps while the cache grows towards the bound."""
    L, B, hkv, d, hq, n, steps = 2, 2, 8, 128, 32, 250, 20
    a, b = build(L, B, hkv, d, hq, n, steps + 8), build(L, B, hkv, d, hq, n, steps + 8)
    a.token_capacity = n + steps + 2
    q = torch.zeros((L, B, hq, d), dtype=torch.float16, device="cuda")
    k = torch.zeros((L, B, hkv, d), dtype=torch.float16, device="cuda")
    v = torch.zeros_like(k)
    oa = torch.zeros((L, B, hq, d), dtype=torch.float32, device="cuda")
    ob = torch.zeros_like(oa)
    gen = torch.Generator(device="cuda").manual_seed(1)
    fresh = lambda t: t.copy_(torch.randn(t.shape, generator=gen, device="cuda"))
    fresh(q); fresh(k); fresh(v)
    decode_step(a, q, k, v, oa)
    decode_step(b, q, k, v, ob)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        decode_step(a, q, k, v, oa)
    for t in range(steps):
        fresh(q); fresh(k); fresh(v)
        graph.replay()
        decode_step(b, q, k, v, ob)
        torch.cuda.synchronize()
        assert torch.equal(oa, ob), t
    a.check_errors(); b.check_errors()
    assert torch.equal(a.cumulative, b.cumulative) and torch.equal(a.layer_ema, b.layer_ema)
