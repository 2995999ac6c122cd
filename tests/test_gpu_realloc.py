"""Device allocator (skv_alloc_bits) and requantise/repack against the oracle and the fixtures
generated from the reference's _solve_allocation / _requantize_tokens."""
import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc
from tests.gpu_util import assert_close, fill_store, make_store, oracle_attention

pytestmark = pytest.mark.gpu


def _scatter_scores(store, seq, imp):
    """imp indexed by token id -> the store's storage-order score array of one sequence."""
    tok = store.slot_token[seq].long()
    live = tok >= 0
    store.cumulative[seq].zero_()
    store.cumulative[seq][live] = torch.from_numpy(np.asarray(imp, np.float64)).cuda()[tok[live]]


def _alloc_store(n_list, hkv, d, init_bits_seed=0):
    """A store whose sequences hold n_list[b] tokens spread over the buckets (no K/V needed)."""
    B = len(n_list)
    store = make_store(1, B, hkv, d, hkv, max(n_list))
    rng = np.random.default_rng(init_bits_seed)
    for b, n in enumerate(n_list):
        bits = rng.choice((2, 3, 4, 8), size=n)
        bucket = store._bits_lut[torch.from_numpy(bits.astype(np.int64)).cuda()]
        onehot = torch.nn.functional.one_hot(bucket.long(), 4).to(torch.int32)
        pos = ((torch.cumsum(onehot, 0) - onehot) * onehot).sum(-1).to(torch.int32)
        store.counts[b] = onehot.sum(0).to(torch.int32)
        storage = store._base_t[bucket.long()] + pos
        store.slot_token[b, storage.long()] = torch.arange(n, dtype=torch.int32, device="cuda")
        store.next_token[b] = n
    return store


def _device_bits(store, seq, n, new_bits):
    tok = store.slot_token[seq].long()
    live = tok >= 0
    out = torch.zeros(n, dtype=torch.uint8, device="cuda")
    out[tok[live]] = new_bits[seq][live]
    return out.cpu().numpy()


def _oracle_cfg(h, d, beta, bits, **kw):
    return orc.AllocatorConfig(h, d, float(beta), bits, **kw)


def test_allocator_matches_reference_fixtures(golden):
    g = golden("allocation")
    for ci in g["alloc_cases"]:
        spec = g[f"alloc_{ci}_spec"]
        n, h, d, nb = [int(x) for x in spec[:4]]
        bits = [int(x) for x in spec[4:4 + nb]]
        beta, alpha, frac, boost, minhp = g[f"alloc_{ci}_beta"]
        store = _alloc_store([n], h, d, init_bits_seed=int(ci))
        cfg = store.make_alloc_config(float(beta), bits, utility_alpha=float(alpha), high_precision_fraction=float(frac),
                                      high_precision_boost=float(boost), min_high_precision_tokens=int(minhp))
        for imp_key, bits_key in [("imp", "bits1"), ("imp2", "bits2"), ("imp2", "bits3")]:
            _scatter_scores(store, 0, g[f"alloc_{ci}_{imp_key}"])
            new_bits, new_counts, _ = store.allocate_bits(cfg)
            got = _device_bits(store, 0, n, new_bits)
            want = g[f"alloc_{ci}_{bits_key}"]
            assert np.array_equal(got, want), (int(ci), bits_key, int((got != want).sum()))
            hist = [int((want == w).sum()) for w in (2, 3, 4, 8)]
            assert new_counts[0].tolist() == hist
        store.check_errors()


def _random_importance(rng, n, kind):
    ranks = rng.permutation(n) + 1
    imp = (1.0 / ranks ** 1.1).astype(np.float32)
    if kind == 1:
        imp = np.round(imp, 2)                 # many ties and exact zeros
    elif kind == 2:
        imp = (imp * rng.integers(0, 2, n)).astype(np.float32)   # half the tokens never attended
    elif kind == 3:
        imp = np.full(n, 0.25, np.float32)     # all equal
    return imp


@pytest.mark.parametrize("seed", range(6))
def test_allocator_matches_oracle_random(seed):
    rng = np.random.default_rng(100 + seed)
    B = 5
    h, d = [(4, 64), (8, 128)][seed % 2]
    bits = [(2, 3, 4, 8), (2, 4, 8), (2, 3, 4, 8), (3, 4, 8), (2, 3, 4, 8), (4, 8)][seed]
    beta = [0.35, 0.5, 0.25, 0.45, 0.2, 0.4][seed]
    n_list = [int(x) for x in rng.integers(5, 3000, B)]
    n_list[0] = int(rng.integers(1, 12))       # tiny: the serial walk
    n_list[1] = 3000
    store = _alloc_store(n_list, h, d, init_bits_seed=seed)
    kw = dict(high_precision_fraction=[0.02, 0.1, 0.02, 0.0, 0.3, 0.02][seed])
    cfg = store.make_alloc_config(beta, bits, **kw)
    ocfg = _oracle_cfg(h, d, beta, bits, **kw)
    states = [dict() for _ in range(B)]
    for call in range(3):
        imps = [_random_importance(rng, n, (seed + b + call) % 4) for b, n in enumerate(n_list)]
        for b in range(B):
            _scatter_scores(store, b, imps[b])
        new_bits, new_counts, changed = store.allocate_bits(cfg)
        for b, n in enumerate(n_list):
            scores = {t: (float("inf") if t < 4 else float(imps[b][t])) for t in range(n)}
            a = orc.solve_allocation(ocfg, range(n), scores, states[b])
            want = np.array([a[t] for t in range(n)], np.uint8)
            got = _device_bits(store, b, n, new_bits)
            assert np.array_equal(got, want), (seed, call, b, n, int((got != want).sum()))
            # the hysteresis record follows the reference's too
            tok = store.slot_token[b].long()
            live = (tok >= 0).cpu().numpy()
            streak = store.rank_streak[b].cpu().numpy()[live]
            pct = store.rank_pct[b].cpu().numpy()[live]
            ids = tok.cpu().numpy()[live]
            assert np.array_equal(streak, np.array([states[b][int(t)]["streak"] for t in ids]))
            assert np.array_equal(pct, np.array([states[b][int(t)]["pct"] for t in ids]))
    store.check_errors()


def test_allocator_gated_baseline_uses_streaks():
    # a budget so tight that the all-minimum allocation is already past the 0.85 gate: only tokens whose
    # rank moved for `intervals` calls in a row may climb (cache.py:468-472)
    rng = np.random.default_rng(7)
    n, h, d = 400, 4, 64
    store = _alloc_store([n], h, d)
    beta = 0.175
    cfg = store.make_alloc_config(beta, (2, 3, 4, 8))
    ocfg = _oracle_cfg(h, d, beta, (2, 3, 4, 8))
    state = {}
    for call in range(4):
        imp = _random_importance(rng, n, call % 2)
        _scatter_scores(store, 0, imp)
        new_bits, _, _ = store.allocate_bits(cfg)
        a = orc.solve_allocation(ocfg, range(n), {t: (float("inf") if t < 4 else float(imp[t])) for t in range(n)}, state)
        want = np.array([a[t] for t in range(n)], np.uint8)
        assert np.array_equal(_device_bits(store, 0, n, new_bits), want), call


def test_requantize_repack_matches_reference_fixture(golden):
    g = golden("requant")
    L, h, d, n = [int(x) for x in g["requant_shape"]]
    store = make_store(L, 1, h, d, h, n)
    kv = [orc.synth_kv(n, h, d, seed=50 + l) for l in range(L)]
    fill_store(store, [(k[None], v[None]) for k, v in kv], np.full((1, n), 4))   # stored at the default 4 bits
    cfg = store.make_alloc_config(0.35)
    for imp_key, bits_key, tag in (("requant_imp", "requant_bits", "requant"), ("requant_imp2", "requant_bits2", "requant2")):
        _scatter_scores(store, 0, g[imp_key])
        new_bits, _, _ = store.allocate_bits(cfg)
        assert np.array_equal(_device_bits(store, 0, n, new_bits), g[bits_key])
        store.repack(new_bits)
        store.check_errors()
        assert np.array_equal(store.token_bits(0).cpu().numpy(), g[bits_key])
        for l in range(L):
            ids, bits, kc, vc, ks, vs = store.export_sequence(l, 0)
            assert np.array_equal(ids.cpu().numpy(), np.arange(n))
            kdeq = orc.dequantize_rows(kc.cpu().numpy(), ks.cpu().numpy())
            vdeq = orc.dequantize_rows(vc.cpu().numpy(), vs.cpu().numpy())
            assert np.array_equal(kdeq, g[f"{tag}_k_deq_{l}"]), (tag, l)
            assert np.array_equal(vdeq, g[f"{tag}_v_deq_{l}"]), (tag, l)
            if tag == "requant":
                assert np.array_equal(ks.cpu().numpy(), g[f"requant_k_scale_{l}"])
                assert np.array_equal(vs.cpu().numpy(), g[f"requant_v_scale_{l}"])


def test_repack_keeps_per_token_state_and_attention():
    rng = np.random.default_rng(5)
    B, hq, hkv, d, n, L = 3, 8, 2, 128, 900, 2
    store = make_store(L, B, hkv, d, hq, n)
    kvs = []
    for l in range(L):
        k, v = orc.synth_kv(B * n, hkv, d, seed=900 + l)
        kvs.append((k.reshape(B, n, hkv, d), v.reshape(B, n, hkv, d)))
    bits0 = rng.choice((2, 3, 4, 8), size=(B, n))
    fill_store(store, kvs, bits0)
    imps = [_random_importance(rng, n, b % 3) for b in range(B)]
    for b in range(B):
        _scatter_scores(store, b, imps[b])
    # per-layer EMA / first-touch flags: something recognisable per token
    tok = store.slot_token.long().clamp(min=0)
    store.layer_ema[:] = (tok.float() * 0.5)[None] + torch.arange(L, device="cuda").float()[:, None, None]
    store.touched[:] = ((tok % 3) == 0).to(torch.uint8)[None]
    cfg = store.make_alloc_config(0.35)
    ocfg = _oracle_cfg(hkv, d, 0.35, (2, 3, 4, 8))
    new_bits, new_counts, changed = store.allocate_bits(cfg)
    store.repack(new_bits)
    store.check_errors()
    assert torch.equal(store.counts, new_counts)
    for b in range(B):
        a = orc.solve_allocation(ocfg, range(n), {t: (float("inf") if t < 4 else float(imps[b][t])) for t in range(n)}, {})
        want = np.array([a[t] for t in range(n)], np.uint8)
        assert np.array_equal(store.token_bits(b).cpu().numpy(), want)
        assert int(changed[b]) == int((want != bits0[b]).sum())
        tokb = store.slot_token[b].long()
        live = tokb >= 0
        assert int(live.sum()) == n and len(set(tokb[live].tolist())) == n
        ids = tokb[live]
        assert torch.equal(store.cumulative[b][live], torch.from_numpy(imps[b].astype(np.float64)).cuda()[ids])
        for l in range(L):
            assert torch.equal(store.layer_ema[l, b][live], ids.float() * 0.5 + l)
            assert torch.equal(store.touched[l, b][live], ((ids % 3) == 0).to(torch.uint8))
        # freed indices are reset
        assert bool((store.cumulative[b][~live] == 0).all()) and bool((store.rank_streak[b][~live] == -1).all())
    # rows: requantised from the stored codes where the width changed, untouched otherwise
    q = rng.standard_normal((B, hq, d)).astype(np.float32)
    for l in range(L):
        out = store.attention(l, torch.from_numpy(q).cuda()).cpu().numpy()
        store.check_errors()
        for b in range(B):
            a_bits = store.token_bits(b).cpu().numpy()
            k, v = kvs[l][0][b], kvs[l][1][b]
            kq = np.empty(k.shape, np.int8); vq = np.empty(k.shape, np.int8)
            ks = np.empty(k.shape[:2], np.float32); vs = np.empty(k.shape[:2], np.float32)
            for w0 in (2, 3, 4, 8):
                for w1 in (2, 3, 4, 8):
                    sel = (bits0[b] == w0) & (a_bits == w1)
                    if not sel.any():
                        continue
                    for src, cq, cs in ((k, kq, ks), (v, vq, vs)):
                        c0, s0 = orc.quantize_rows(src[sel], w0)
                        if w1 != w0:
                            c0, s0 = orc.requantize_rows(c0, s0, w1)
                        cq[sel], cs[sel] = c0, s0
            ids, bits, kc, vc, ksc, vsc = store.export_sequence(l, b)
            assert np.array_equal(kc.cpu().numpy(), kq) and np.array_equal(vc.cpu().numpy(), vq)
            assert np.array_equal(ksc.cpu().numpy(), ks) and np.array_equal(vsc.cpu().numpy(), vs)
            ref, _ = oracle_attention(q[b], kq, vq, ks, vs, hq // hkv)
            assert_close(out[b], ref, what=f"attention after repack l{l} b{b}")


def test_reallocate_graphed_equals_eager():
    """reallocate_graphed (first call eager + capture, later calls one graph launch) leaves the store in
    exactly the state reallocate() does, also when the importance changes between the calls."""
    rng = np.random.default_rng(11)
    B, hq, hkv, d, n, L = 2, 8, 2, 128, 700, 2
    stores = [make_store(L, B, hkv, d, hq, n) for _ in range(2)]
    kvs = []
    for l in range(L):
        k, v = orc.synth_kv(B * n, hkv, d, seed=300 + l)
        kvs.append((k.reshape(B, n, hkv, d), v.reshape(B, n, hkv, d)))
    bits0 = rng.choice((2, 3, 4, 8), size=(B, n))
    for s in stores:
        fill_store(s, kvs, bits0)
    cfgs = [s.make_alloc_config(0.35) for s in stores]
    for it in range(3):
        imps = [_random_importance(rng, n, (b + it) % 3) for b in range(B)]
        for s in stores:
            for b in range(B):
                _scatter_scores(s, b, imps[b])
        stores[0].reallocate(cfgs[0])
        stores[1].reallocate_graphed(cfgs[1])     # first pass: eager + capture; later passes: replay
        for s in stores:
            s.check_errors()
        a, g = stores
        assert torch.equal(a.counts, g.counts) and torch.equal(a.slot_token, g.slot_token), it
        assert torch.equal(a.arena, g.arena), it
        assert torch.equal(a.cumulative, g.cumulative) and torch.equal(a.rank_streak, g.rank_streak), it
    q = torch.from_numpy(rng.standard_normal((B, hq, d)).astype(np.float32)).cuda()
    assert torch.equal(stores[0].attention(0, q), stores[1].attention(0, q))
