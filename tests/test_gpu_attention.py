"""Fused packed decode attention vs the CPU oracle (dequantise-then-attend / streaming,
fp32).  Tolerance from the north star: 2e-3 max-abs + 1e-3 relative."""
import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc
from smartkv_b200 import _lib
from tests.gpu_util import assert_close, fill_store, make_store, oracle_attention, oracle_quantized

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-3
LOG2E = 1.4426950408889634


def run_case(hq, hkv, d, lens, seed, q_dtype=np.float32, with_current=True, bits_choices=(2, 3, 4, 8),
             zipf_bits=False):
    """lens: tokens per sequence (ragged, zeros allowed)."""
    B = len(lens)
    n = max(max(lens), 1)
    g = hq // hkv
    rng = np.random.default_rng(seed)
    store = make_store(1, B, hkv, d, hq, n)
    # ragged fill: one plan_bulk call per distinct prefix keeps ids dense per sequence
    ks, vs, bs = [], [], []
    for b in range(B):
        k, v = orc.synth_kv(max(lens[b], 1), hkv, d, seed=seed * 100 + b)
        bits = rng.choice(bits_choices, size=max(lens[b], 1))
        bits[: min(4, bits.size)] = max(bits_choices)
        ks.append(k[: lens[b]]); vs.append(v[: lens[b]]); bs.append(bits[: lens[b]])
    # place tokens sequence by sequence (different lengths): emulate with per-sequence rows
    for b in range(B):
        if lens[b] == 0:
            continue
        bt = torch.zeros((B, lens[b]), dtype=torch.int64, device="cuda")
        # only sequence b receives tokens in this call: build the plan by hand
        bucket = store._bits_lut[torch.from_numpy(bs[b].astype(np.int64)).cuda()]
        onehot = torch.nn.functional.one_hot(bucket.long(), 4).to(torch.int32)
        pos = ((torch.cumsum(onehot, 0) - onehot) * onehot).sum(-1).to(torch.int32)
        store.counts[b] = onehot.sum(0).to(torch.int32)
        storage = store._base_t[bucket.long()] + pos
        store.slot_token[b, storage.long()] = torch.arange(lens[b], dtype=torch.int32, device="cuda")
        store.next_token[b] = lens[b]
        seq = torch.full((lens[b],), b, dtype=torch.int32, device="cuda")
        store.append(0, torch.from_numpy(ks[b]).cuda(), torch.from_numpy(vs[b]).cuda(), seq, bucket.contiguous(),
                     pos.contiguous())
    q = rng.standard_normal((B, hq, d)).astype(q_dtype)
    ck = rng.standard_normal((B, hkv, d)).astype(np.float32) if with_current else None
    cv = rng.standard_normal((B, hkv, d)).astype(np.float32) if with_current else None
    plan = store.plan_step()
    out = store.attention(0, torch.from_numpy(q).cuda(), None if ck is None else torch.from_numpy(ck).cuda(),
                          None if cv is None else torch.from_numpy(cv).cuda(), update_importance=True,
                          cur_storage=plan[3])
    store.check_errors()
    out = out.cpu().numpy()
    logits = store.logits.cpu().numpy()
    lmax, lsum = store.lse_max.cpu().numpy(), store.lse_sum.cpu().numpy()
    cur_prob = store.cur_prob.cpu().numpy()
    slot_token = store.slot_token.cpu().numpy()
    for b in range(B):
        if lens[b] == 0 and not with_current:
            assert np.all(out[b] == 0)
            continue
        kq, vq, kso, vso = oracle_quantized(ks[b], vs[b], bs[b]) if lens[b] else (
            np.zeros((0, hkv, d), np.int8), np.zeros((0, hkv, d), np.int8), np.zeros((0, hkv), np.float32),
            np.zeros((0, hkv), np.float32))
        ref_o, ref_p = oracle_attention(q[b].astype(np.float32), kq, vq, kso, vso, g,
                                        None if ck is None else ck[b], None if cv is None else cv[b])
        assert_close(out[b], ref_o, ATOL, RTOL, f"out seq {b}")
        # probabilities rebuilt from the emitted logits, in token order
        valid = slot_token[b] >= 0
        order = np.argsort(slot_token[b][valid])
        p = np.exp2(logits[b][:, valid][:, order] - lmax[b][:, None]) / lsum[b][:, None]
        assert_close(p, ref_p[:, : lens[b]], 2e-4, 2e-3, f"probs seq {b}")
        if with_current:
            assert_close(cur_prob[b], ref_p[:, lens[b]], 2e-4, 2e-3, f"current-token prob seq {b}")
            assert_close(p.sum(-1) + cur_prob[b], np.ones(hq), 1e-4, 0, "probabilities sum to one")
    return store


@pytest.mark.parametrize("q_dtype", [np.float32, np.float16])
def test_config0_shape(q_dtype):
    # TinyLlama attention shape, context 2048, one decode step
    run_case(32, 4, 64, [2048], seed=0, q_dtype=q_dtype)


@pytest.mark.parametrize("q_dtype", [np.float32, np.float16])
def test_llama8b_shape_ragged_batch(q_dtype):
    run_case(32, 8, 128, [700, 1, 0, 333, 2049, 16], seed=1, q_dtype=q_dtype)


@pytest.mark.parametrize("hq,hkv,d", [(64, 8, 128), (8, 8, 64), (16, 8, 128), (4, 4, 128), (32, 4, 64)])
def test_group_sizes(hq, hkv, d):
    run_case(hq, hkv, d, [257, 100], seed=2)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("d", [64, 128])
def test_uniform_width(bits, d):
    run_case(16, 4, d, [415], seed=3 + bits, bits_choices=(bits,))


def test_no_current_token_and_empty():
    run_case(32, 8, 128, [0, 77], seed=9, with_current=False)


def test_long_context_many_ctas():
    # more blocks than CTAs, several CTAs per (sequence, head) segment
    run_case(32, 8, 128, [40000], seed=11, bits_choices=(2, 3, 4, 8))


def test_golden_reference_outputs(golden):
    """Stored codes recorded from the reference cache + its streaming CPU attention output."""
    g = golden("attention")
    for tag in ("c0s", "l8s"):
        hq, hkv, d, n, b = [int(x) for x in g[f"attn_{tag}_shape"]]
        bits = g[f"attn_{tag}_bits"]
        k, v = orc.synth_kv(n, hkv, d, seed=21)
        store = make_store(1, b, hkv, d, hq, n)
        fill_store(store, [(np.broadcast_to(k, (b,) + k.shape).copy(), np.broadcast_to(v, (b,) + v.shape).copy())],
                   np.broadcast_to(bits, (b, n)).copy())
        for bi in range(b):
            ids, wb, kc, vc, ks, vs = store.export_sequence(0, bi)
            assert np.array_equal(kc.cpu().numpy(), g[f"attn_{tag}_kq"])
            assert np.array_equal(vc.cpu().numpy(), g[f"attn_{tag}_vq"])
            assert np.array_equal(ks.cpu().numpy(), g[f"attn_{tag}_ks"])
        q = torch.from_numpy(g[f"attn_{tag}_q"][:, :, 0]).cuda()
        out = store.attention(0, q, torch.from_numpy(g[f"attn_{tag}_ck"]).cuda(), torch.from_numpy(g[f"attn_{tag}_cv"]).cuda())
        store.check_errors()
        assert_close(out.cpu().numpy(), g[f"attn_{tag}_stream_out"][:, :, 0], ATOL, RTOL, tag)
        out = store.attention(0, q)
        assert_close(out.cpu().numpy(), g[f"attn_{tag}_dequant_out"][:, :, 0], ATOL, RTOL, tag + " no current")


def test_config0_golden_pipeline(golden):
    g = golden("config0")
    hq, hkv, d, n = 32, 4, 64, 2048
    k, v = orc.synth_kv(n, hkv, d, seed=0)
    bits = g["c0_bits"].astype(np.int64)
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, hq, 1, d)).astype(np.float32)
    ck = rng.standard_normal((1, hkv, d)).astype(np.float32)
    cv = rng.standard_normal((1, hkv, d)).astype(np.float32)
    store = make_store(1, 1, hkv, d, hq, n)
    fill_store(store, [(k[None], v[None])], bits[None])
    plan = store.plan_step()
    out = store.attention(0, torch.from_numpy(q[:, :, 0]).cuda(), torch.from_numpy(ck).cuda(), torch.from_numpy(cv).cuda(),
                          update_importance=True, cur_storage=plan[3])
    store.check_errors()
    assert_close(out.cpu().numpy(), g["c0_out"][:, :, 0], ATOL, RTOL, "config 0 output")
    # per-key probability mass summed over heads (unweighted) against the reference's
    logits = store.logits.cpu().numpy()[0]
    lmax, lsum = store.lse_max.cpu().numpy()[0], store.lse_sum.cpu().numpy()[0]
    st = store.slot_token.cpu().numpy()[0]
    valid = st >= 0
    order = np.argsort(st[valid])
    p = np.exp2(logits[:, valid][:, order] - lmax[:, None]) / lsum[:, None]
    mass = np.concatenate([p.sum(0), [store.cur_prob.cpu().numpy()[0].sum()]])
    assert_close(mass, g["c0_keymass"], 1e-4, 2e-3, "config 0 key mass")


def test_wait_limit_expiry_sets_the_error_flag_and_leaves_the_context_usable():
    """Every device-side wait of the attention kernel is bounded.  With the limit cut to one poll the consumer
    warps give up before the first bytes can have arrived: the launch must still return, report the timeout
    through the error flag, and the same store must give the right answer once the limit is restored."""
    lib = _lib.lib()
    store = run_case(32, 8, 128, [3000, 500], seed=77)
    rng = np.random.default_rng(0)
    q = torch.from_numpy(rng.standard_normal((2, 32, 128)).astype(np.float32)).cuda()
    good = store.attention(0, q).clone()
    store.check_errors()
    assert lib.skv_set_wait_limit(1) == 0
    try:
        store.attention(0, q)
        torch.cuda.synchronize()
        with pytest.raises(_lib.SmartKVLibraryError, match="wait"):
            store.check_errors()
    finally:
        assert lib.skv_set_wait_limit(1 << 24) == 0
    store.err.zero_()
    again = store.attention(0, q).clone()
    store.check_errors()
    assert torch.equal(again, good)


@pytest.mark.parametrize("q_dtype", [np.float16, np.float32])
def test_large_value_magnitudes_do_not_overflow_fp16(q_dtype):
    """V rows of magnitude 1e3..1e4 at 2 and 3 bits have V scales in the thousands, and the P operand of the
    P.V product is probability x V scale in fp16.  The kernel raises its running maximum for such tiles, so the
    output stays finite and within the tolerance scaled by the magnitude of V."""
    hq, hkv, d, n = 32, 8, 128, 515
    rng = np.random.default_rng(21)
    k, v = orc.synth_kv(n, hkv, d, seed=21)
    v = (v * rng.uniform(1e3, 1e4, size=(n, hkv, 1))).astype(np.float32)
    v[::7] *= 1e-4                                   # ordinary rows next to the outliers
    bits = rng.choice([2, 3], size=n)
    store = make_store(1, 1, hkv, d, hq, n)
    fill_store(store, [(k[None], v[None])], bits[None])
    q = (4.0 * rng.standard_normal((1, hq, d))).astype(q_dtype)      # peaked softmax: probabilities near one
    out = store.attention(0, torch.from_numpy(q).cuda()).cpu().numpy()[0]
    store.check_errors()
    assert np.all(np.isfinite(out))
    kq, vq, ks, vs = oracle_quantized(k, v, bits)
    ref, _ = oracle_attention(q[0].astype(np.float32), kq, vq, ks, vs, hq // hkv)
    assert_close(out, ref, 2e-3 * 1e4, 2e-3, "large V magnitudes")


def test_large_v_scale_created_by_a_reallocation_is_guarded_too():
    """V rows of magnitude ~300 stored at 8 bits have scales of ~2.4; moved to 2 bits by a reallocation their
    scale becomes ~300.  The requantise kernel must record that in the arena, or the attention kernel would
    multiply probabilities near one by it in fp16 unchecked."""
    hq, hkv, d, n = 32, 8, 128, 300
    rng = np.random.default_rng(8)
    k, v = orc.synth_kv(n, hkv, d, seed=8)
    v = (v * 100.0).astype(np.float32)
    store = make_store(1, 1, hkv, d, hq, n)
    fill_store(store, [(k[None], v[None])], np.full((1, n), 8))
    new_bits = torch.zeros((1, store.slots), dtype=torch.uint8, device="cuda")
    base8 = store.bucket_base[3]
    new_bits[0, base8: base8 + n] = 2
    store.repack(new_bits, max_moves=n)
    store.check_errors()
    assert store.counts[0].tolist() == [n, 0, 0, 0]
    q = (4.0 * rng.standard_normal((1, hq, d))).astype(np.float16)
    out = store.attention(0, torch.from_numpy(q).cuda()).cpu().numpy()[0]
    store.check_errors()
    assert np.all(np.isfinite(out))
    ids, bits, kc, vc, ks, vs = store.export_sequence(0, 0)
    assert float(vs.max()) > 64.0
    ref, _ = oracle_attention(q[0].astype(np.float32), kc.cpu().numpy(), vc.cpu().numpy(), ks.cpu().numpy(),
                              vs.cpu().numpy(), hq // hkv)
    assert_close(out, ref, 2e-3 * 300, 2e-3, "V scales grown by a reallocation")
