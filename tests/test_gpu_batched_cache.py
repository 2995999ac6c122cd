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
