"""BatchedSmartKVCache at the cache level: several independent sequences in one packed store, prompt
stored from causal attention probabilities, then decode steps whose reallocations fall in the middle
of a step.  After every layer call the kernel output is compared with the oracle's attention over the
rows the store holds at that moment (exported codes and scales, token order) plus the step's token in
full precision; tolerance 2e-3 absolute + 1e-3 relative."""
import numpy as np
import pytest
import torch

from tests.gpu_util import assert_close, oracle_attention

pytestmark = pytest.mark.gpu


def causal_probs(B, Hq, n, rng):
    s = rng.standard_normal((B, Hq, n, n)).astype(np.float32)
    s[..., np.triu_indices(n, 1)[0], np.triu_indices(n, 1)[1]] = -np.inf
    p = np.exp(s - s.max(-1, keepdims=True))
    return (p / p.sum(-1, keepdims=True)).astype(np.float32)


@pytest.mark.parametrize("attribution", ["keys", "wrapper"])
@pytest.mark.parametrize("q_dtype", [torch.float32, torch.float16])
def test_decode_matches_oracle_through_mid_step_reallocations(attribution, q_dtype):
    from smartkv_b200 import BatchedSmartKVCache
    L, B, Hq, Hkv, D, n, steps = 3, 2, 32, 4, 64, 70, 40
    rng = np.random.default_rng(5)
    cache = BatchedSmartKVCache(L, Hkv, D, Hq, B, max_tokens=n + steps + 4, memory_budget=0.45, realloc_freq=16,
                                key_attribution=attribution)
    st = cache.store
    for l in range(L):
        k = torch.from_numpy(rng.standard_normal((B, n, Hkv, D)).astype(np.float32)).cuda()
        v = torch.from_numpy(rng.standard_normal((B, n, Hkv, D)).astype(np.float32)).cuda()
        cache.prefill_layer(l, k, v, torch.from_numpy(causal_probs(B, Hq, n, rng)).cuda())
    cache.check_errors()
    assert len(cache) == n and st.counts.sum().item() == B * n
    assert cache.realloc_counter >= 1
    triggers_seen = set()
    for t in range(steps):
        for l in range(L):
            q = rng.standard_normal((B, Hq, D)).astype(np.float32)
            ck = rng.standard_normal((B, Hkv, D)).astype(np.float32)
            cv = rng.standard_normal((B, Hkv, D)).astype(np.float32)
            # what the layer holds before the call, in token order (the step's token is not among the cached keys)
            before = []
            for b in range(B):
                ids, bits, kc, vc, ks, vs = st.export_sequence(l, b)
                keep = (ids < n + t).cpu().numpy()
                before.append(tuple(x.cpu().numpy()[keep] for x in (kc, vc, ks, vs)))
            r0 = cache.realloc_counter
            qt = torch.from_numpy(q).cuda().to(q_dtype)
            out = cache.decode_layer(l, qt, torch.from_numpy(ck).cuda(), torch.from_numpy(cv).cuda()).cpu().numpy()
            if cache.realloc_counter != r0:
                triggers_seen.add(l)
            for b in range(B):
                kc, vc, ks, vs = before[b]
                ref, _ = oracle_attention(qt[b].float().cpu().numpy(), kc, vc, ks, vs, Hq // Hkv, ck[b], cv[b])
                assert_close(out[b], ref, 2e-3, 1e-3, f"step {t} layer {l} sequence {b}")
        cache.check_errors()
        assert len(cache) == n + t + 1 and st.counts.sum().item() == B * (n + t + 1)
    assert len(triggers_seen) >= 2, triggers_seen          # reallocations did fall on different layers of a step
    stats = cache.get_memory_stats()
    assert stats["memory_ratio_true_max"] <= 0.45 + 1e-6
    # every token id is cached exactly once per sequence
    where = cache._token_storage()[:, : n + steps]
    assert bool((where >= 0).all())


def test_reference_trigger_schedule():
    """The reallocation trigger follows the reference's counters (smartkv/core/cache.py:266-279): the same
    schedule as a host replay of token_counter, len(precision_map) and the per-layer adaptive frequency."""
    from smartkv_b200 import BatchedSmartKVCache
    L, B, Hq, Hkv, D, n, steps = 5, 1, 8, 2, 64, 50, 30
    rng = np.random.default_rng(1)
    cache = BatchedSmartKVCache(L, Hkv, D, Hq, B, max_tokens=n + steps + 4, memory_budget=0.5, realloc_freq=16)
    want, tc, known = [], 0, 0
    for l in range(L):
        total = known + n
        if tc % max(16 * (1 + l // 4), max(32, total // 8)) == 0:
            want.append(("prefill", l))
        known = n
        tc += n
    for t in range(steps):
        for l in range(L):
            fired_before = any(x == (t, j) for x in want for j in range(l))
            total = known + 1
            if tc % max(16 * (1 + l // 4), max(32, total // 8)) == 0:
                want.append((t, l))
                known = n + t + 1
            if l == 0:
                known = n + t + 1
            tc += 1
    got = []
    for l in range(L):
        r0 = cache.realloc_counter
        cache.prefill_layer(l, torch.randn(B, n, Hkv, D, device="cuda"), torch.randn(B, n, Hkv, D, device="cuda"),
                            torch.from_numpy(causal_probs(B, Hq, n, rng)).cuda())
        if cache.realloc_counter != r0:
            got.append(("prefill", l))
    for t in range(steps):
        for l in range(L):
            r0 = cache.realloc_counter
            cache.decode_layer(l, torch.randn(B, Hq, D, device="cuda"), torch.randn(B, Hkv, D, device="cuda"),
                               torch.randn(B, Hkv, D, device="cuda"))
            if cache.realloc_counter != r0:
                got.append((t, l))
    cache.check_errors()
    assert got == want, (got, want)


def test_graph_replayed_steps_are_bit_identical_to_eager_steps():
    """GraphedDecoder over a synthetic per-layer forward (queries, keys and values looked up from seeded tables by
    token id and position, no GEMM library in the way): every replayed step, including the ones whose graphs hold a
    reallocation in the middle of the step, must leave exactly the outputs and the cache state of the same step
    launched from Python."""
    from smartkv_b200 import BatchedSmartKVCache
    from smartkv_b200.models.graphed_decode import GraphedDecoder
    L, B, Hq, Hkv, D, n, steps, V = 6, 3, 32, 4, 64, 70, 48, 97      # 6 layers: triggers fall on several different layers
    g = torch.Generator(device="cuda").manual_seed(5)
    tq = torch.randn((L, V, Hq, D), generator=g, device="cuda").half()
    tk = torch.randn((L, V, Hkv, D), generator=g, device="cuda").half()
    tv = torch.randn((L, V, Hkv, D), generator=g, device="cuda").half()
    rng = np.random.default_rng(9)
    prompt_kv = [(torch.randn((B, n, Hkv, D), generator=g, device="cuda"), torch.randn((B, n, Hkv, D), generator=g, device="cuda"))
                 for _ in range(L)]
    probs = [torch.from_numpy(causal_probs(B, Hq, n, rng)).cuda() for _ in range(L)]
    feed = torch.randint(0, V, (steps, B), generator=g, device="cuda")
    results = []
    for graphed in (False, True):
        cache = BatchedSmartKVCache(L, Hkv, D, Hq, B, max_tokens=n + steps + 4, memory_budget=0.45, realloc_freq=16)
        for l in range(L):
            cache.prefill_layer(l, prompt_kv[l][0], prompt_kv[l][1], probs[l])

        def forward(ids, pos, cache=cache):
            outs = []
            idx = (ids[:, 0] + pos[:, 0]) % V
            for l in range(L):
                outs.append(cache.decode_layer(l, tq[l][idx], tk[l][idx], tv[l][idx]).clone())
            return torch.stack(outs)

        dec = GraphedDecoder(forward, lambda cache=cache: cache)
        outs = []
        for t in range(steps):
            if graphed:
                outs.append(dec.step(feed[t], n + t).clone())
            else:
                ids = feed[t].view(B, 1)
                outs.append(forward(ids, torch.full((B, 1), n + t, device="cuda")))
        cache.check_errors()
        st = cache.store
        results.append((torch.stack(outs), st.counts.clone(), st.slot_token.clone(), st.cumulative.clone(), st.arena.clone(),
                        cache.realloc_counter, cache.num_cached, dec.graphs_captured))
    a, b = results
    assert b[7] >= 3 and a[5] == b[5] and a[6] == b[6]
    assert torch.equal(a[0], b[0]), float((a[0] - b[0]).abs().max())
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3]) and torch.equal(a[4], b[4])
