"""The host-side mirror of the reference's Python interface (smartkv.kernels, smartkv.core,
smartkv.models) checked against the oracle.  The cases follow the reference's own tests
(tests/test_bit_packing.py, tests/test_quant_cuda.py, tests/test_cache.py)."""
import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu


def test_pack_unpack_tensor_bytes_and_errors():
    from smartkv_b200.kernels import bit_packing as bp
    rng = np.random.default_rng(0)
    for bits in (2, 3, 4, 8):
        lo, hi = orc.code_range(bits)
        for n in (1, 7, 8, 100, 4096 + 5):
            codes = rng.integers(lo, hi + 1, n).astype(np.int8)
            packed = bp.pack_tensor(torch.from_numpy(codes).cuda(), bits)
            if bits < 8:
                assert packed.dtype == torch.uint8 and packed.numel() == bp.compute_packed_size(n, bits)
                assert np.array_equal(packed.cpu().numpy(), orc.pack_codes(codes, bits))
            back = bp.unpack_tensor(packed, bits, (n,))
            assert back.dtype == torch.int8 and np.array_equal(back.cpu().numpy(), codes)
    x = torch.randint(-4, 3, (8, 16, 128), dtype=torch.int8, device="cuda")
    assert torch.equal(bp.unpack_tensor(bp.pack_tensor(x, 3), 3, (8, 16, 128)), x)
    with pytest.raises(ValueError):
        bp.pack_tensor(x.float(), 3)
    with pytest.raises(ValueError):
        bp.pack_tensor(x, 5)
    with pytest.raises(ValueError):
        bp.compute_packed_size(10, 7)
    assert bp.get_compression_ratio(2) == 4.0 and bp.get_memory_savings_vs_fp16(4) == 0.25


def test_quantize_per_head_cuda_matches_oracle():
    from smartkv_b200.core._quant_cuda import quantize_per_head_cuda, pack_values, unpack_values
    k, v = orc.synth_kv(50, 4, 64, seed=1)
    k[3] = 0.0                                  # zero rows keep scale 1
    for bits in (2, 3, 4, 8):
        kq, vq, ks, vs = quantize_per_head_cuda(torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), bits)
        okq, ovq, oks, ovs = orc.quantize_per_head(k, v, bits)
        assert np.array_equal(kq.cpu().numpy(), okq) and np.array_equal(vq.cpu().numpy(), ovq)
        assert np.array_equal(ks.cpu().numpy(), oks) and np.array_equal(vs.cpu().numpy(), ovs)
        assert torch.equal(unpack_values(pack_values(kq, bits), bits, kq.shape), kq)
    with pytest.raises(ValueError):
        quantize_per_head_cuda(torch.from_numpy(k), torch.from_numpy(v), 4)


def _quantized(n, h, d, bits_choices, seed):
    k, v = orc.synth_kv(n, h, d, seed=seed)
    rng = np.random.default_rng(seed)
    bits = rng.choice(bits_choices, size=n)
    kq = np.empty(k.shape, np.int8); vq = np.empty(k.shape, np.int8)
    ks = np.empty(k.shape[:2], np.float32); vs = np.empty(k.shape[:2], np.float32)
    for w in set(bits_choices):
        sel = bits == w
        if sel.any():
            kq[sel], ks[sel] = orc.quantize_rows(k[sel], w)
            vq[sel], vs[sel] = orc.quantize_rows(v[sel], w)
    return k, v, bits, kq, vq, ks, vs


@pytest.mark.parametrize("q_len", [1, 3])
def test_quantized_attention_matches_dequantise_then_attend(q_len):
    from smartkv_b200.kernels import quantized_attention
    B, H, d, n = 2, 8, 128, 300
    rng = np.random.default_rng(2)
    kqs, vqs, kss, vss = [], [], [], []
    for b in range(B):
        _, _, _, kq, vq, ks, vs = _quantized(n, H, d, (8,), seed=10 + b)
        kqs.append(kq.transpose(1, 0, 2)); vqs.append(vq.transpose(1, 0, 2)); kss.append(ks.T); vss.append(vs.T)
    kq, vq, ks, vs = (np.stack(x) for x in (kqs, vqs, kss, vss))
    q = rng.standard_normal((B, H, q_len, d)).astype(np.float32)
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    out = quantized_attention(t(q), t(kq), t(ks), t(vq), t(vs))
    ref, _ = orc.dequant_attend(q, kq, ks, vq, vs)
    assert out.shape == (B, H, q_len, d)
    assert_close(out.cpu().numpy(), ref, what="quantized_attention")
    # the [B, k, H, d] layout is accepted too (kernels/__init__.py:28-41)
    out2 = quantized_attention(t(q), t(kq.transpose(0, 2, 1, 3)), t(ks), t(vq.transpose(0, 2, 1, 3)), t(vs))
    assert torch.equal(out, out2)
    # additive mask [B, 1, q, k], as the reference's kernels take it (smartkv/csrc/quantized_attention.cu:213-216)
    mask = rng.standard_normal((B, 1, q_len, n)).astype(np.float32) * 3.0
    mask[:, :, :, ::7] = -1e4                      # some keys masked out altogether
    out3 = quantized_attention(t(q), t(kq), t(ks), t(vq), t(vs), attention_mask=t(mask))
    ref3, _ = orc.dequant_attend(q, kq, ks, vq, vs, mask=mask)
    assert_close(out3.cpu().numpy(), ref3, what="quantized_attention with an additive mask")
    with pytest.raises(NotImplementedError):       # one mask row per (sequence, query position): heads share it
        quantized_attention(t(q), t(kq), t(ks), t(vq), t(vs),
                            attention_mask=t(rng.standard_normal((B, H, q_len, n)).astype(np.float32)))


def test_cache_store_retrieve_like_the_reference():
    from smartkv_b200 import SmartKVCache
    L, H, d = 2, 4, 64
    cache = SmartKVCache(num_layers=L, num_heads=H, head_dim=d, memory_budget=0.5, max_tokens=512)
    assert cache.available_bits == [8, 4, 3, 2]                 # sorted descending, like the reference
    assert cache.use_packing and cache.min_budget == pytest.approx(0.1875)     # (2 bits * 512 + 4*4*32) / (512 * 16)
    k, v = orc.synth_kv(20, H, d, seed=3)
    kt, vt = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    cache.quantize_and_store(0, 0, kt[0], vt[0])
    assert cache.get_precision(0) == 4 and cache.precision_map == {0: 4}     # unseen tokens are stored at 4 bits
    assert (0, 0) in cache.k_cache and (1, 0) not in cache.k_cache
    rk, rv = cache.retrieve(0, 0)
    q4, s4 = orc.quantize_rows(k[:1], 4)
    assert np.array_equal(rk.cpu().numpy(), orc.dequantize_rows(q4, s4)[0])
    with pytest.raises(KeyError):
        cache.retrieve(1, 0)
    with pytest.raises(KeyError):
        cache.retrieve(0, 99)
    cache.precision_map[5] = 8
    cache.precision_map[6] = 2
    cache.quantize_and_store_batch(0, list(range(1, 20)), kt[1:], vt[1:])
    cache.quantize_and_store_batch(1, list(range(0, 20)), kt, vt)
    assert len(cache) == 20 and cache.total_tokens_stored == 40
    keys, values = cache.retrieve_all(0)
    assert keys.shape == (20, H, d)
    bits = np.full(20, 4); bits[5] = 8; bits[6] = 2
    for t in range(20):
        cq, cs = orc.quantize_rows(k[t:t + 1], int(bits[t]))
        assert np.array_equal(keys[t].cpu().numpy(), orc.dequantize_rows(cq, cs)[0]), t
    ks2, _ = cache.retrieve_all(0, [7, 3, 99])
    assert ks2.shape[0] == 2 and torch.equal(ks2[0], keys[7]) and torch.equal(ks2[1], keys[3])
    rq = cache.retrieve_all_quantized(1)
    assert rq["token_ids"].tolist() == list(range(20)) and rq["k_qx"].dtype == torch.int8
    assert rq["k_scale"].shape == (20, H)
    stats = cache.get_memory_stats()
    assert stats["num_tokens"] == 20 and stats["num_cache_entries"] == 40 and stats["storage_mode"] == "packed"
    assert stats["precision_distribution"] == {"8-bit": 1, "4-bit": 18, "3-bit": 0, "2-bit": 1}
    assert "SmartKVCache(layers=2" in repr(cache)
    cache.clear()
    assert len(cache) == 0 and cache.retrieve_all(0)[0].shape[0] == 0


def test_cache_importance_allocation_and_requantisation():
    from smartkv_b200 import SmartKVCache
    from smartkv_b200.kernels import quantized_attention_bucketed
    L, H, d, n = 2, 4, 64, 256
    cache = SmartKVCache(num_layers=L, num_heads=H, head_dim=d, memory_budget=0.35, realloc_freq=16, max_tokens=512)
    kv = [orc.synth_kv(n, H, d, seed=50 + l) for l in range(L)]
    for l in range(L):
        cache.quantize_and_store_batch(l, list(range(n)), torch.from_numpy(kv[l][0]).cuda(), torch.from_numpy(kv[l][1]).cuda())
    # importance through the cache-level contract: probabilities [1, heads, 1, keys] with the ids of the keys
    rng = np.random.default_rng(4)
    probs = rng.dirichlet(np.full(n, 0.05), size=(1, H, 1)).astype(np.float32)
    ref = orc.ImportanceState(L)
    cache.token_counter = 1        # keep the automatic trigger out of this step (cache.py:276)
    cache.update_attention(0, torch.from_numpy(probs).cuda(), list(range(n)))
    ref.update(0, probs, range(n))
    got = np.array([cache.get_importance(t) for t in range(n)])
    want = np.array([ref.token_importance[t] for t in range(n)])
    assert np.allclose(got, want, rtol=1e-5, atol=1e-9)
    assert cache.global_step == 1 and cache.last_seen[n - 1] == 1
    # allocation: bit-exact with the reference's allocator on the same scores
    alloc = cache.allocate_precision(0, list(range(n)))
    ocfg = orc.AllocatorConfig(H, d, 0.35)
    scores = orc.allocation_scores(range(n), {t: float(got[t]) for t in range(n)}, {t: 1 for t in range(n)}, 1)
    want_alloc = orc.solve_allocation(ocfg, range(n), scores, {})
    assert alloc == want_alloc and cache.precision_map == want_alloc
    assert cache.get_memory_stats()["memory_ratio_true"] <= 0.35 + 1e-6
    # stored tokens were requantised from their 4-bit codes in every layer
    bits = np.array([want_alloc[t] for t in range(n)])
    for l in range(L):
        keys, values = cache.retrieve_all(l)
        for x, got_x in ((kv[l][0], keys), (kv[l][1], values)):
            q4, s4 = orc.quantize_rows(x, 4)
            deq = orc.dequantize_rows(q4, s4)
            for w in (2, 3, 8):
                sel = bits == w
                if sel.any():
                    c, s = orc.requantize_rows(q4[sel], s4[sel], w)
                    deq[sel] = orc.dequantize_rows(c, s)
            assert np.array_equal(got_x.cpu().numpy(), deq), l
    # bucket views feed the bucketed attention entry point
    views = cache.get_bucket_views(0)
    assert set(views) <= {2, 3, 4, 8} and sum(v["token_ids"].numel() for v in views.values()) == n
    q = rng.standard_normal((1, H, 1, d)).astype(np.float32)
    out = quantized_attention_bucketed(torch.from_numpy(q).cuda(), views)
    rq = cache.retrieve_all_quantized(0)
    ref_out, _ = orc.dequant_attend(q, rq["k_qx"].cpu().numpy().transpose(1, 0, 2)[None], rq["k_scale"].cpu().numpy().T[None],
                                    rq["v_qx"].cpu().numpy().transpose(1, 0, 2)[None], rq["v_scale"].cpu().numpy().T[None])
    assert_close(out.cpu().numpy(), ref_out, what="bucketed attention")


def test_cache_fused_decode_step_matches_oracle():
    from smartkv_b200 import SmartKVCache
    L, Hq, H, d, n = 1, 8, 2, 128, 200
    cache = SmartKVCache(num_layers=L, num_heads=H, head_dim=d, memory_budget=0.5, max_tokens=512, num_query_heads=Hq)
    k, v, bits, kq, vq, ks, vs = _quantized(n, H, d, (2, 3, 4, 8), seed=8)
    for t in range(n):
        cache.precision_map[t] = int(bits[t])
    cache.token_counter = 1
    cache.quantize_and_store_batch(0, list(range(n)), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
    rng = np.random.default_rng(1)
    q = rng.standard_normal((Hq, d)).astype(np.float32)
    ck = rng.standard_normal((H, d)).astype(np.float32)
    cv = rng.standard_normal((H, d)).astype(np.float32)
    e = lambda x: orc.expand_gqa(x, Hq // H)
    ref, p = orc.streaming_attention(q[None, :, None, :], e(kq), e(ks), e(vq), e(vs), tile_size=64,
                                     current_k=e(ck[None]), current_v=e(cv[None]))
    out = cache.fused_decode_attention(0, torch.from_numpy(q).cuda(), torch.from_numpy(ck).cuda(),
                                       torch.from_numpy(cv).cuda(), token_id=n)
    assert_close(out.cpu().numpy(), ref[0, :, 0], what="fused decode")
    # per-key mass: every cached key and the current token were keys of this call
    imp = orc.ImportanceState(L)
    imp.update(0, p, range(n + 1))
    got = np.array([cache.get_importance(t) for t in range(n + 1)])
    want = np.array([imp.token_importance[t] for t in range(n + 1)])
    assert np.allclose(got, want, rtol=2e-3, atol=1e-5)
    cache.quantize_and_store(0, n, torch.from_numpy(ck).cuda(), torch.from_numpy(cv).cuda())
    assert cache.store.counts.sum().item() == n + 1


def test_llama_wrapper_generates_and_tracks_the_dense_model():
    transformers = pytest.importorskip("transformers")
    from smartkv_b200 import LlamaSmartKV, SmartKVConfig
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=320, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                   bos_token_id=1, eos_token_id=2, pad_token_id=0)
    model = transformers.LlamaForCausalLM(cfg).cuda().float().eval()
    ids = torch.randint(3, 320, (1, 24), device="cuda")
    with torch.no_grad():
        dense = model(ids).logits
        dense_gen = model.generate(ids, max_new_tokens=6, do_sample=False)
    wrapped = LlamaSmartKV(model, SmartKVConfig(enabled=True, memory_budget=0.6, available_bits=[8], device="cuda"))
    assert wrapped.smartkv_cache is not None and wrapped.config is model.config      # attribute delegation
    with torch.no_grad():
        logits = wrapped(ids).logits
    assert torch.allclose(logits, dense, atol=1e-4, rtol=1e-4)      # prefill attends over the unquantised prompt
    wrapped.reset_cache()
    with torch.no_grad():
        gen = wrapped.generate(ids, max_new_tokens=6, do_sample=False)
    assert gen.shape == dense_gen.shape
    cache = wrapped.smartkv_cache
    assert len(cache) == 24 + 5 and cache.store.counts.sum().item() == 24 + 5   # the last token is never fed back
    stats = wrapped.get_smartkv_stats()
    # the prompt got its widths from the allocation of the first update; tokens appended later enter at the
    # default 4 bits whatever available_bits says (cache.py:1214), as in the reference
    assert stats["num_tokens"] == 29 and stats["precision_distribution"]["8-bit"] == 24
    # 8-bit keys/values: the decode logits stay close to the dense model's
    wrapped.reset_cache()
    with torch.no_grad():
        wrapped(ids[:, :-1])
        step = wrapped(ids[:, -1:]).logits[0, -1]
    assert torch.allclose(step, dense[0, -1], atol=5e-2, rtol=5e-2)
    wrapped.disable_smartkv()
    with torch.no_grad():
        assert torch.equal(wrapped(ids).logits, dense)
    # mixed widths under a budget: generation runs, reallocation happens, the budget holds
    wrapped.enable_smartkv(memory_budget=0.4)
    wrapped.smartkv_config.available_bits = [2, 3, 4, 8]
    wrapped.enable_smartkv()
    wrapped.reset_cache()
    with torch.no_grad():
        wrapped.generate(ids, max_new_tokens=40, do_sample=False)
    stats = wrapped.get_smartkv_stats()
    assert stats["realloc_count"] >= 1 and stats["memory_ratio_true"] <= 0.4 + 1e-6
    assert wrapped.smartkv_cache.store.counts.sum().item() == 24 + 39


def test_tinyllama_shape_fused_decode_matches_dequantised_path():
    """The end-to-end generation workload scaled down in depth only: TinyLlama-1.1B attention shape (hidden 2048, 32 query /
    4 KV heads, head_dim 64, vocab 32000), random N(0, 0.02) fp16 weights, 512 random prompt ids, budget 0.5.
    The fused decode path (packed kernels, current token in full precision) and the dequantise-then-attend
    path over the same cache must give the same next-token logits."""
    transformers = pytest.importorskip("transformers")
    from smartkv_b200 import LlamaSmartKV, SmartKVConfig
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=4,
                                   num_attention_heads=32, num_key_value_heads=4, max_position_embeddings=2048,
                                   initializer_range=0.02, bos_token_id=1, eos_token_id=2)
    model = transformers.LlamaForCausalLM(cfg).cuda().half().eval()
    ids = torch.randint(3, 32000, (1, 512), device="cuda")
    wrapped = LlamaSmartKV(model, SmartKVConfig(enabled=True, memory_budget=0.5, device="cuda"))
    steps = []
    for fused in (True, False):
        wrapped.reset_cache()
        wrapped.set_use_fused_gpu(fused)
        with torch.no_grad():
            wrapped(ids[:, :-1])
            logits = wrapped(ids[:, -1:]).logits[0, -1].float()
        steps.append(logits)
        stats = wrapped.get_smartkv_stats()
        assert stats["num_tokens"] == 512 and stats["memory_ratio_true"] <= 0.5 + 1e-6
        dist_ = stats["precision_distribution"]
        assert sum(dist_.values()) == 512 and sum(1 for c in dist_.values() if c > 0) >= 2     # mixed widths
    assert torch.allclose(steps[0], steps[1], atol=2e-2, rtol=2e-2), float((steps[0] - steps[1]).abs().max())
    assert int(steps[0].argmax()) == int(steps[1].argmax())
    wrapped.set_use_fused_gpu(True)
    wrapped.reset_cache()
    with torch.no_grad():
        out = wrapped.generate(ids, max_new_tokens=24, do_sample=False)
    assert out.shape == (1, 512 + 24)
    assert wrapped.smartkv_cache.store.counts.sum().item() == 512 + 23


def test_cache_grows_past_its_initial_capacity():
    from smartkv_b200 import SmartKVCache
    L, H, d = 2, 2, 64
    cache = SmartKVCache(num_layers=L, num_heads=H, head_dim=d, memory_budget=0.5, max_tokens=100)
    cap0 = cache.store.caps[2]
    n = 3 * cap0 + 17                      # forces two doublings of the 4-bit bucket
    kv = [orc.synth_kv(n, H, d, seed=60 + l) for l in range(L)]
    cache.token_counter = 1
    step = 50
    for lo in range(0, n, step):
        hi = min(n, lo + step)
        for l in range(L):
            cache.quantize_and_store_batch(l, list(range(lo, hi)), torch.from_numpy(kv[l][0][lo:hi]).cuda(),
                                           torch.from_numpy(kv[l][1][lo:hi]).cuda())
    assert cache.store.caps[2] > cap0 and len(cache) == n and cache.store.counts.sum().item() == n
    for l in range(L):
        keys, values = cache.retrieve_all(l)
        q4, s4 = orc.quantize_rows(kv[l][0], 4)
        assert np.array_equal(keys.cpu().numpy(), orc.dequantize_rows(q4, s4)), l
        q4, s4 = orc.quantize_rows(kv[l][1], 4)
        assert np.array_equal(values.cpu().numpy(), orc.dequantize_rows(q4, s4)), l
    # attention over the grown store
    rng = np.random.default_rng(2)
    q = rng.standard_normal((H, d)).astype(np.float32)
    ck = rng.standard_normal((H, d)).astype(np.float32)
    cv = rng.standard_normal((H, d)).astype(np.float32)
    out = cache.fused_decode_attention(0, torch.from_numpy(q).cuda(), torch.from_numpy(ck).cuda(),
                                       torch.from_numpy(cv).cuda(), token_id=n, update_importance=False)
    kq, ks = orc.quantize_rows(kv[0][0], 4)
    vq, vs = orc.quantize_rows(kv[0][1], 4)
    ref, _ = orc.streaming_attention(q[None, :, None, :], kq, ks, vq, vs, tile_size=512, current_k=ck[None], current_v=cv[None])
    assert_close(out.cpu().numpy(), ref[0, :, 0], what="attention after growth")
