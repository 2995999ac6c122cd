"""The CPU oracle against golden vectors recorded from the reference's own
CPU modules (tests/golden/make_golden.py) and against the constants the
reference's tests assert."""
import hashlib

import numpy as np
import pytest

from oracle import smartkv_oracle as orc


def sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8)


@pytest.mark.parametrize("tag", ["a", "b"])
@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_quantize_matches_reference_bit_exact(golden, tag, bits):
    g = golden("quant")
    kq, vq, ks, vs = orc.quantize_per_head(g[f"quant_{tag}_k"], g[f"quant_{tag}_v"], bits)
    assert np.array_equal(kq, g[f"quant_{tag}_kq{bits}"])
    assert np.array_equal(vq, g[f"quant_{tag}_vq{bits}"])
    assert np.array_equal(ks.view(np.uint32), g[f"quant_{tag}_ks{bits}"].view(np.uint32))
    assert np.array_equal(vs.view(np.uint32), g[f"quant_{tag}_vs{bits}"].view(np.uint32))


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_quantize_bulk_digest(golden, bits):
    g = golden("quant")
    k, v = orc.synth_kv(512, 8, 128, seed=3)
    kq, vq, ks, vs = orc.quantize_per_head(k, v, bits)
    assert np.array_equal(sha(kq), g[f"quant_bulk_sha_kq{bits}"])
    assert np.array_equal(sha(vq), g[f"quant_bulk_sha_vq{bits}"])
    assert np.array_equal(sha(ks), g[f"quant_bulk_sha_ks{bits}"])
    assert np.array_equal(sha(vs), g[f"quant_bulk_sha_vs{bits}"])


def test_quantize_reference_test_pins():
    # tests/test_quant_cpu.py:86-100 zero input -> zero codes, scale 1.0
    q, s = orc.quantize_rows(np.zeros((2, 4, 8), np.float32), 8)
    assert not q.any() and np.all(s == 1.0)
    # tests/test_quant_cpu.py:72-84 one-bit degenerate range, :243-258 ranges per width
    x = np.random.default_rng(0).standard_normal((16, 4, 32)).astype(np.float32)
    q1, _ = orc.quantize_rows(x, 1)
    assert q1.min() == 0 and q1.max() == 0
    for bits, lo, hi in [(2, -2, 1), (3, -4, 3), (4, -8, 7), (8, -128, 127)]:
        q, _ = orc.quantize_rows(x, bits)
        assert q.min() >= lo and q.max() <= hi and q.max() == hi


def test_min_budget_and_ratio_constants(golden):
    # tests/test_budget_validation.py:13-55, 125-144
    assert abs(orc.compute_minimum_budget(8, 128, "fp32", False) - 0.53125) < 1e-12
    assert abs(orc.compute_minimum_budget(8, 128, "fp16", False) - 0.515625) < 1e-12
    assert abs(orc.compute_minimum_budget(8, 128, "fp32", True) - 0.15625) < 1e-12
    assert abs(orc.compute_minimum_budget(8, 128, "fp16", True) - 0.140625) < 1e-12
    assert np.allclose(golden("allocation")["min_budget"], [0.53125, 0.515625, 0.15625, 0.140625])
    r = orc.memory_ratio_true({i: 4 for i in range(100)}, 8, 128, "fp16", True)
    assert abs(r - 0.2578125) < 1e-12
    r = orc.memory_ratio_true({i: 2 for i in range(100)}, 8, 128, "fp32", False)
    assert abs(r - 0.515625) < 1e-12


def test_pack_known_bytes():
    # 2-bit: codes+2 -> LSB first, four per byte
    assert orc.pack_codes(np.array([-2, -1, 0, 1], np.int8), 2).tolist() == [0b11100100]
    # 4-bit: even index = low nibble
    assert orc.pack_codes(np.array([-8, 7, 0, -1], np.int8), 4).tolist() == [0xF0, 0x78]
    # 3-bit: eight codes -> 24-bit little-endian word
    codes = np.array([-4, -3, -2, -1, 0, 1, 2, 3], np.int8)
    word = sum((int(c) + 4) << (3 * i) for i, c in enumerate(codes))
    assert orc.pack_codes(codes, 3).tolist() == [word & 255, (word >> 8) & 255, (word >> 16) & 255]
    # 8-bit identity on the two's complement byte
    assert orc.pack_codes(np.array([-128, -1, 0, 127], np.int8), 8).tolist() == [128, 255, 0, 127]
    # partial trailing group is zero filled (tests/test_bit_packing.py:184-205)
    assert orc.pack_codes(np.array([-1, 0, 1], np.int8), 2).tolist() == [0b00111001]
    assert orc.packed_size(100, 3) == 39 and orc.packed_size(3, 2) == 1 and orc.packed_size(5, 4) == 3


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("n", [1, 3, 8, 17, 100, 128, 1000])
def test_pack_roundtrip_all_values(bits, n):
    # tests/test_bit_packing.py:17-49, 207-227: every value of the range survives, odd sizes included
    lo, hi = orc.code_range(bits)
    rng = np.random.default_rng(n * 10 + bits)
    codes = rng.integers(lo, hi + 1, size=n).astype(np.int8)
    codes[: min(n, hi - lo + 1)] = np.arange(lo, hi + 1, dtype=np.int8)[: min(n, hi - lo + 1)]
    packed = orc.pack_codes(codes, bits)
    assert packed.dtype == np.uint8 and packed.size == orc.packed_size(n, bits)
    assert np.array_equal(orc.unpack_codes(packed, bits, n), codes)


def test_row_packing_equals_flat_packing():
    # smartkv/core/cache.py:1069-1070: flat [H*D] pack reshaped to [H, pd]
    rng = np.random.default_rng(5)
    for bits in (2, 3, 4, 8):
        lo, hi = orc.code_range(bits)
        for d in (64, 128):
            codes = rng.integers(lo, hi + 1, size=(3, 4, d)).astype(np.int8)
            rows = orc.pack_rows(codes, bits)
            assert rows.shape == (3, 4, orc.packed_size(d, bits))
            for t in range(3):
                assert np.array_equal(rows[t].reshape(-1), orc.pack_codes(codes[t].reshape(-1), bits))
            assert np.array_equal(orc.unpack_rows(rows, bits, d), codes)


@pytest.mark.parametrize("tag", ["c0s", "l8s"])
def test_attention_oracles(golden, tag):
    g = golden("attention")
    hq, hkv, d, n, b = g[f"attn_{tag}_shape"]
    grp = hq // hkv
    q = g[f"attn_{tag}_q"]
    kq = orc.expand_gqa(g[f"attn_{tag}_kq"], grp)
    vq = orc.expand_gqa(g[f"attn_{tag}_vq"], grp)
    ks = orc.expand_gqa(g[f"attn_{tag}_ks"], grp)
    vs = orc.expand_gqa(g[f"attn_{tag}_vs"], grp)
    ck = orc.expand_gqa(g[f"attn_{tag}_ck"], grp)
    cv = orc.expand_gqa(g[f"attn_{tag}_cv"], grp)
    o, p = orc.streaming_attention(q, kq, ks, vq, vs, tile_size=64, current_k=ck, current_v=cv)
    assert np.allclose(o, g[f"attn_{tag}_stream_out"], rtol=1e-5, atol=1e-6)
    assert np.allclose(p, g[f"attn_{tag}_stream_probs"], rtol=1e-5, atol=1e-8)
    o, p = orc.streaming_attention(q, kq, ks, vq, vs)
    assert np.allclose(o, g[f"attn_{tag}_nocur_out"], rtol=1e-5, atol=1e-6)
    assert np.allclose(p, g[f"attn_{tag}_nocur_probs"], rtol=1e-5, atol=1e-8)
    kk = np.broadcast_to(np.transpose(kq, (1, 0, 2))[None], (b, hq, n, d))
    vv = np.broadcast_to(np.transpose(vq, (1, 0, 2))[None], (b, hq, n, d))
    o2, p2 = orc.dequant_attend(q, kk, np.broadcast_to(ks.T[None], (b, hq, n)), vv, np.broadcast_to(vs.T[None], (b, hq, n)))
    assert np.allclose(o2, g[f"attn_{tag}_dequant_out"], rtol=1e-5, atol=1e-6)
    assert np.allclose(o2, g[f"attn_{tag}_nocur_out"], rtol=1e-4, atol=1e-5)
    # the stored codes themselves are what the quantizer oracle produces at the per-token widths
    k, v = orc.synth_kv(int(n), int(hkv), int(d), seed=21)
    bits = g[f"attn_{tag}_bits"]
    for w in (2, 3, 4, 8):
        sel = bits == w
        kq_w, ks_w = orc.quantize_rows(k[sel], w)
        assert np.array_equal(kq_w, g[f"attn_{tag}_kq"][sel])
        assert np.array_equal(ks_w, g[f"attn_{tag}_ks"][sel])


def test_importance_update(golden):
    g = golden("importance")
    L, hq, n, steps = g["imp_shape"]
    st = orc.ImportanceState(int(L))
    i = 0
    for step in range(steps):
        for layer in range(L):
            p = g[f"imp_probs_{i}"]
            st.update(layer, p, list(range(p.shape[-1])))
            i += 1
    ids = g["imp_token_ids"]
    cum = np.array([st.token_importance[int(t)] for t in ids])
    ema = np.array([[st.layer_importance.get((l, int(t)), np.nan) for t in ids] for l in range(L)])
    assert np.allclose(cum, g["imp_cumulative"], rtol=2e-6, atol=1e-9)
    assert np.allclose(ema, g["imp_layer_ema"], rtol=2e-6, atol=1e-9, equal_nan=True)
    assert np.allclose(st.head_importance, g["imp_head_importance"], rtol=1e-6)
    assert st.global_step == int(g["imp_global_step"][0])


def _cfg_from(g, ci):
    spec = g[f"alloc_{ci}_spec"]
    n, h, d, nb = [int(x) for x in spec[:4]]
    bits = [int(x) for x in spec[4:4 + nb]]
    beta, alpha, frac, boost, minhp = g[f"alloc_{ci}_beta"]
    cfg = orc.AllocatorConfig(h, d, float(beta), bits, utility_alpha=float(alpha), high_precision_fraction=float(frac),
                              high_precision_boost=float(boost), min_high_precision_tokens=int(minhp))
    return n, cfg


def test_allocator_matches_reference_bit_exact(golden):
    g = golden("allocation")
    for ci in g["alloc_cases"]:
        n, cfg = _cfg_from(g, ci)
        state = {}
        for imp_key, bits_key in [("imp", "bits1"), ("imp2", "bits2"), ("imp2", "bits3")]:
            imp = g[f"alloc_{ci}_{imp_key}"]
            scores = {t: (float("inf") if t < 4 else float(imp[t])) for t in range(n)}
            a = orc.solve_allocation(cfg, range(n), scores, state)
            got = np.array([a[t] for t in range(n)], np.uint8)
            assert np.array_equal(got, g[f"alloc_{ci}_{bits_key}"]), (int(ci), bits_key)
        a1 = {t: int(b) for t, b in enumerate(g[f"alloc_{ci}_bits1"])}
        assert abs(orc.memory_ratio_true(a1, cfg.num_heads, cfg.head_dim, "fp32", True) - g[f"alloc_{ci}_ratio1"][0]) < 1e-12
        assert g[f"alloc_{ci}_ratio1"][0] <= cfg.memory_budget + 1e-6


def test_requantize_from_dequantized_codes(golden):
    g = golden("requant")
    L, h, d, n = [int(x) for x in g["requant_shape"]]
    cfg = orc.AllocatorConfig(h, d, 0.35)
    imp = g["requant_imp"]
    bits = orc.solve_allocation(cfg, range(n), {t: (float("inf") if t < 4 else float(imp[t])) for t in range(n)}, {})
    bits = np.array([bits[t] for t in range(n)], np.uint8)
    assert np.array_equal(bits, g["requant_bits"])
    imp2 = g["requant_imp2"]
    bits2 = orc.solve_allocation(cfg, range(n), {t: (float("inf") if t < 4 else float(imp2[t])) for t in range(n)}, {})
    bits2 = np.array([bits2[t] for t in range(n)], np.uint8)
    assert np.array_equal(bits2, g["requant_bits2"])
    for l in range(L):
        k, v = orc.synth_kv(n, h, d, seed=50 + l)
        for x, name in ((k, "k"), (v, "v")):
            q4, s4 = orc.quantize_rows(x, 4)          # stored at the default 4 bits first
            deq1 = np.empty_like(x)
            codes1 = np.empty(x.shape, np.int8)
            scale1 = np.empty(x.shape[:2], np.float32)
            for w in (2, 3, 4, 8):
                sel = bits == w
                if w == 4:
                    codes1[sel], scale1[sel] = q4[sel], s4[sel]
                else:
                    codes1[sel], scale1[sel] = orc.requantize_rows(q4[sel], s4[sel], w)
            deq1 = orc.dequantize_rows(codes1, scale1)
            assert np.array_equal(deq1, g[f"requant_{name}_deq_{l}"])
            assert np.array_equal(scale1, g[f"requant_{name}_scale_{l}"])
            codes2, scale2 = codes1.copy(), scale1.copy()
            for w in (2, 3, 4, 8):
                sel = (bits2 == w) & (bits != bits2)
                codes2[sel], scale2[sel] = orc.requantize_rows(codes1[sel], scale1[sel], w)
            assert np.array_equal(orc.dequantize_rows(codes2, scale2), g[f"requant2_{name}_deq_{l}"])


def test_config0_reference_pipeline(golden):
    g = golden("config0")
    hq, hkv, d, n = 32, 4, 64, 2048
    grp = hq // hkv
    k, v = orc.synth_kv(n, hkv, d, seed=0)
    imp = orc.synth_importance(n, seed=0, zipf_s=1.1)
    cfg = orc.AllocatorConfig(hkv, d, 0.35)
    a = orc.solve_allocation(cfg, range(n), {t: (float("inf") if t < 4 else float(imp[t])) for t in range(n)}, {})
    bits = np.array([a[t] for t in range(n)], np.uint8)
    assert np.array_equal(bits, g["c0_bits"])
    kq = np.empty(k.shape, np.int8); vq = np.empty(v.shape, np.int8)
    ks = np.empty(k.shape[:2], np.float32); vs = np.empty(k.shape[:2], np.float32)
    for w in (2, 3, 4, 8):
        sel = bits == w
        kq[sel], ks[sel] = orc.quantize_rows(k[sel], w)
        vq[sel], vs[sel] = orc.quantize_rows(v[sel], w)
    assert np.array_equal(sha(kq), g["c0_sha_kcodes"])
    assert np.array_equal(sha(vq), g["c0_sha_vcodes"])
    assert np.array_equal(sha(ks), g["c0_sha_kscale"])
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, hq, 1, d)).astype(np.float32)
    ck = rng.standard_normal((1, hkv, d)).astype(np.float32)
    cv = rng.standard_normal((1, hkv, d)).astype(np.float32)
    o, p = orc.streaming_attention(q, orc.expand_gqa(kq, grp), orc.expand_gqa(ks, grp), orc.expand_gqa(vq, grp),
                                   orc.expand_gqa(vs, grp), tile_size=2048, current_k=orc.expand_gqa(ck, grp),
                                   current_v=orc.expand_gqa(cv, grp))
    assert np.allclose(o, g["c0_out"], rtol=1e-5, atol=1e-6)
    assert np.allclose(p.sum(axis=(0, 1, 2)), g["c0_keymass"], rtol=1e-4, atol=1e-7)
    assert np.allclose(p[0, 0, 0], g["c0_probs_head0"], rtol=1e-5, atol=1e-9)
