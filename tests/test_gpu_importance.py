"""Fused importance update vs the oracle's restatement of update_attention."""
import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc
from tests.gpu_util import assert_close, fill_store, make_store, oracle_attention, oracle_quantized

pytestmark = pytest.mark.gpu


def test_importance_over_steps_and_layers():
    hq, hkv, d, n0, Lyr, B, steps = 16, 4, 64, 150, 2, 2, 3
    g = hq // hkv
    rng = np.random.default_rng(5)
    store = make_store(Lyr, B, hkv, d, hq, n0 + steps + 1)
    bits = rng.choice([2, 3, 4, 8], size=(B, n0))
    kv = []
    for layer in range(Lyr):
        ks, vs = zip(*[orc.synth_kv(n0, hkv, d, seed=40 + 10 * layer + b) for b in range(B)])
        kv.append((np.stack(ks), np.stack(vs)))
    fill_store(store, kv, bits)
    # oracle state: one per sequence (the reference keeps one cache per sequence)
    ostate = [orc.ImportanceState(Lyr) for _ in range(B)]
    cache = [[list(oracle_quantized(kv[l][0][b], kv[l][1][b], bits[b])) for l in range(Lyr)] for b in range(B)]
    for step in range(steps):
        plan = store.plan_step()
        for layer in range(Lyr):
            q = rng.standard_normal((B, hq, d)).astype(np.float32)
            ck = rng.standard_normal((B, hkv, d)).astype(np.float32)
            cv = rng.standard_normal((B, hkv, d)).astype(np.float32)
            store.attention(layer, torch.from_numpy(q).cuda(), torch.from_numpy(ck).cuda(), torch.from_numpy(cv).cuda(),
                            update_importance=True, cur_storage=plan[3])
            store.append(layer, torch.from_numpy(ck).cuda(), torch.from_numpy(cv).cuda(), plan[0], plan[1], plan[2])
            for b in range(B):
                kq, vq, ks, vs = cache[b][layer]
                _, p = oracle_attention(q[b], kq, vq, ks, vs, g, ck[b], cv[b])
                ostate[b].update(layer, p[None, :, None, :], list(range(p.shape[-1])))
                nk, nv, nks, nvs = oracle_quantized(ck[b][None], cv[b][None], np.array([4]))
                cache[b][layer] = [np.concatenate([kq, nk]), np.concatenate([vq, nv]), np.concatenate([ks, nks]),
                                   np.concatenate([vs, nvs])]
        store.commit_step(plan)
    store.check_errors()
    st = store.slot_token.cpu().numpy()
    cum = store.cumulative.cpu().numpy()
    ema = store.layer_ema.cpu().numpy()
    n = n0 + steps
    for b in range(B):
        valid = st[b] >= 0
        assert valid.sum() == n
        order = np.argsort(st[b][valid])
        got = cum[b][valid][order]
        want = np.array([ostate[b].token_importance[t] for t in range(n)])
        assert_close(got, want, 1e-6, 2e-3, f"cumulative importance seq {b}")
        for layer in range(Lyr):
            got_l = ema[layer, b][valid][order]
            want_l = np.array([ostate[b].layer_importance[(layer, t)] for t in range(n)])
            assert_close(got_l, want_l, 1e-6, 2e-3, f"layer EMA seq {b} layer {layer}")
        hs = store.head_state.cpu().numpy()[b, store.head_parity]
        assert_close(hs, ostate[b].head_importance, 1e-7, 1e-5, "head importance EMA")
    # appended tokens landed in the 4-bit bucket and read back bit-exact
    for b in range(B):
        ids, wb, kc, vc, ks, vs = store.export_sequence(1, b)
        assert np.array_equal(wb.cpu().numpy()[n0:], np.full(steps, 4))
        assert np.array_equal(kc.cpu().numpy(), cache[b][1][0])
        assert np.array_equal(vs.cpu().numpy(), cache[b][1][3])
