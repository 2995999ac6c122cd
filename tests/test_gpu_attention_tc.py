"""The tensor-memory (tcgen05) decode-attention kernel -- head_dim 128, fp16 queries -- against the CPU
oracle (fp32 dequantise-then-attend / streaming), and against the mma.sync fragment kernel on the same
store.  Tolerance from the north star: 2e-3 max-abs + 1e-3 relative."""
import numpy as np
import pytest
import torch

from smartkv_b200 import _lib
from tests.gpu_util import assert_close
from tests.test_gpu_attention import run_case

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _tensor_memory_path():
    _lib.lib().skv_set_attention_path(2)
    yield
    _lib.lib().skv_set_attention_path(0)


def test_tensor_memory_kernel_is_selected():
    from tests.gpu_util import make_store
    store = make_store(1, 1, 8, 128, 32, 256)
    import ctypes
    assert _lib.lib().skv_attn_partials_per_run(ctypes.byref(store.desc), _lib.DTYPE_F16) == 4
    assert _lib.lib().skv_attn_partials_per_run(ctypes.byref(store.desc), _lib.DTYPE_F32) == 7   # fp32 queries: fragment kernel
    _lib.lib().skv_set_attention_path(0)
    assert _lib.lib().skv_attn_partials_per_run(ctypes.byref(store.desc), _lib.DTYPE_F16) == 11


@pytest.mark.parametrize("bits", [8, 4, 2, 3])
def test_uniform_width(bits):
    run_case(32, 8, 128, [415], seed=3 + bits, bits_choices=(bits,), q_dtype=np.float16)


@pytest.mark.parametrize("n", [1, 15, 16, 17, 127, 128, 129, 300])
def test_block_edges(n):
    # fewer keys than one 128-key block, exactly one, one more; every width present
    run_case(32, 8, 128, [n], seed=40 + n, q_dtype=np.float16)


@pytest.mark.parametrize("hq,hkv", [(8, 8), (16, 8), (32, 8), (24, 4), (64, 8), (40, 8)])
def test_group_sizes(hq, hkv):
    run_case(hq, hkv, 128, [257, 100], seed=2, q_dtype=np.float16)


def test_ragged_batch_with_empty_sequences():
    run_case(32, 8, 128, [700, 1, 0, 333, 2049, 16], seed=1, q_dtype=np.float16)


def test_no_current_token_and_empty():
    run_case(32, 8, 128, [0, 77], seed=9, with_current=False, q_dtype=np.float16)


def test_long_context_many_ctas():
    run_case(32, 8, 128, [40000], seed=11, q_dtype=np.float16)


def test_many_sequences_many_runs_per_cta():
    # more (sequence, head) segments than CTAs: every CTA walks several runs, the query ring wraps
    run_case(16, 8, 128, [200 + 37 * i for i in range(48)], seed=12, q_dtype=np.float16)


def test_large_value_magnitudes():
    """V rows with magnitudes of 1e3..1e4 at 2 and 3 bits: the V scale of such rows is far beyond what an
    fp16 probability-times-scale product can hold.  The fixed-point P of this kernel is normalised per block,
    so nothing overflows; the tolerance is the north star's, scaled by the smallest factor applied to V."""
    from oracle import smartkv_oracle as orc
    from tests.gpu_util import fill_store, make_store, oracle_attention, oracle_quantized
    hq, hkv, d, n = 32, 8, 128, 515
    rng = np.random.default_rng(21)
    k, v = orc.synth_kv(n, hkv, d, seed=21)
    v = (v * rng.uniform(1e3, 1e4, size=(n, hkv, 1))).astype(np.float32)
    bits = rng.choice([2, 3], size=n)
    store = make_store(1, 1, hkv, d, hq, n)
    fill_store(store, [(k[None], v[None])], bits[None])
    q = rng.standard_normal((1, hq, d)).astype(np.float16)
    out = store.attention(0, torch.from_numpy(q).cuda()).cpu().numpy()[0]
    store.check_errors()
    assert np.all(np.isfinite(out))
    kq, vq, ks, vs = oracle_quantized(k, v, bits)
    ref, _ = oracle_attention(q[0].astype(np.float32), kq, vq, ks, vs, hq // hkv)
    assert_close(out, ref, 2e-3 * 1e3, 1e-3, "large V magnitudes")


@pytest.mark.parametrize("path", [2, 1])
@pytest.mark.parametrize("q_dtype", [np.float16, np.float32])
def test_additive_mask_and_current_token_mask(path, q_dtype):
    """Mask indexed by token id (the reference indexes it by the key's global slot,
    smartkv/csrc/quantized_attention.cu:570-575) plus the mask value of the current token; both kernels."""
    from oracle import smartkv_oracle as orc
    from tests.gpu_util import fill_store, make_store, oracle_quantized
    _lib.lib().skv_set_attention_path(path)
    hq, hkv, d, n, B = 32, 8, 128, 700, 2
    g = hq // hkv
    rng = np.random.default_rng(33)
    ks_, vs_, bs_ = [], [], []
    for b in range(B):
        k, v = orc.synth_kv(n, hkv, d, seed=50 + b)
        ks_.append(k); vs_.append(v); bs_.append(rng.choice([2, 3, 4, 8], size=n))
    store = make_store(1, B, hkv, d, hq, n)
    fill_store(store, [(np.stack(ks_), np.stack(vs_))], np.stack(bs_))
    q = rng.standard_normal((B, hq, d)).astype(q_dtype)
    ck = rng.standard_normal((B, hkv, d)).astype(np.float32)
    cv = rng.standard_normal((B, hkv, d)).astype(np.float32)
    mask = rng.standard_normal((B, n)).astype(np.float32)
    mask[:, 5::11] = -1e4
    cur_mask = np.array([0.7, -1.3], np.float32)
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    out = store.attention(0, t(q), t(ck), t(cv), mask=t(mask), cur_mask=t(cur_mask)).cpu().numpy()
    store.check_errors()
    e = lambda x: orc.expand_gqa(x, g)
    for b in range(B):
        kq, vq, ksc, vsc = oracle_quantized(ks_[b], vs_[b], bs_[b])
        ref, _ = orc.streaming_attention(q[b].astype(np.float32)[None, :, None, :], e(kq), e(ksc), e(vq), e(vsc),
                                         mask=mask[b][None, None, None, :], tile_size=2048, current_k=e(ck[b][None]),
                                         current_v=e(cv[b][None]), current_mask=np.full((1, 1, 1, 1), cur_mask[b], np.float32))
        assert_close(out[b], ref[0, :, 0], 2e-3, 1e-3, f"masked attention, sequence {b}")


def test_matches_fragment_kernel():
    """Same store, same query: the two kernels agree far inside the parity tolerance."""
    lib = _lib.lib()
    store = run_case(32, 8, 128, [3000, 1234], seed=5, q_dtype=np.float16)
    rng = np.random.default_rng(0)
    q = torch.from_numpy(rng.standard_normal((2, 32, 128)).astype(np.float16)).cuda()
    outs = []
    for path in (2, 1):
        lib.skv_set_attention_path(path)
        store._plan_valid = False
        outs.append(store.attention(0, q).clone().cpu().numpy())
        store.check_errors()
    assert_close(outs[0], outs[1], 5e-4, 5e-4, "tensor-memory vs fragment kernel")
