"""The prompt pass (skv_prefill_attention): causal attention over the unquantised prompt and the per-key
attention mass of the importance update, against the oracle's dense fp32 attention with a causal mask
(orc.dequant_attend on codes = values, scale 1) and ImportanceState.update on the resulting probabilities.
Inputs are fp16; the oracle sees the same fp16-rounded numbers.  Tolerance: 2e-3 absolute + 1e-3 relative
on the output (stored as fp16, so one more half-ulp relative), 2e-3 relative on the mass."""
import numpy as np
import pytest
import torch

from oracle import smartkv_oracle as orc
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu


def oracle_prefill(q, k, v, group, state):
    """q [n, Hq, D], k / v [n, Hkv, D] fp32 -> (out [n, Hq, D], key mass [n]) for one sequence."""
    n = q.shape[0]
    kk = orc.expand_gqa(k.transpose(1, 0, 2)[None], group)          # [1, Hq, n, D]
    vv = orc.expand_gqa(v.transpose(1, 0, 2)[None], group)
    mask = np.where(np.arange(n)[None, :] > np.arange(n)[:, None], -np.inf, 0.0).astype(np.float32)
    ones = np.ones(kk.shape[:3], np.float32)
    out, probs = orc.dequant_attend(q.transpose(1, 0, 2)[None], kk, ones, vv, ones, mask=mask[None, None])
    mass = state.update(0, probs, list(range(n)))
    return out[0].transpose(1, 0, 2), mass


@pytest.mark.parametrize("hq,hkv,d,n,B", [(32, 4, 64, 200, 2), (32, 8, 128, 131, 1), (8, 8, 64, 64, 1), (16, 2, 128, 1, 1),
                                          (32, 4, 64, 515, 1)])
def test_prefill_attention_and_key_mass(hq, hkv, d, n, B):
    from smartkv_b200.prefill import causal_prefill_attention
    rng = np.random.default_rng(hq + n)
    q = rng.standard_normal((B, n, hq, d)).astype(np.float16)
    k = rng.standard_normal((B, n, hkv, d)).astype(np.float16)
    v = rng.standard_normal((B, n, hkv, d)).astype(np.float16)
    w = rng.uniform(0.5, 1.5, size=(B, hq)).astype(np.float32)
    qt, kt, vt = (torch.from_numpy(x).cuda() for x in (q, k, v))
    out, mass = causal_prefill_attention(qt, kt, vt, torch.from_numpy(w).cuda())
    torch.cuda.synchronize()
    out, mass = out.float().cpu().numpy(), mass.cpu().numpy()
    for b in range(B):
        st = orc.ImportanceState(1)
        # make the oracle's head weights the ones handed to the kernel: the weights are a function of the
        # head EMA, which the oracle updates from the probabilities; fix its output instead
        st.head_weights = lambda probs, wb=w[b]: wb
        ref, ref_mass = oracle_prefill(q[b].astype(np.float32), k[b].astype(np.float32), v[b].astype(np.float32),
                                       hq // hkv, st)
        assert_close(out[b], ref, 2e-3, 2e-3, f"prompt attention, sequence {b}")
        assert np.allclose(mass[b], ref_mass, rtol=2e-3, atol=1e-4), np.abs(mass[b] - ref_mass).max()
        assert abs(mass[b].sum() - n * w[b].sum()) <= 1e-3 * n * w[b].sum()       # every query row sums to one


def test_prefill_accepts_the_transposed_views_of_an_attention_module():
    """q / k / v as a Llama attention holds them: [B, H, n, D] views of [B, n, H*D] projections."""
    from smartkv_b200.prefill import causal_prefill_attention
    B, n, hq, hkv, d = 2, 96, 32, 4, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    qp = torch.randn((B, n, hq * d), generator=g, device="cuda").half()
    kp = torch.randn((B, n, hkv * d), generator=g, device="cuda").half()
    vp = torch.randn((B, n, hkv * d), generator=g, device="cuda").half()
    q, k, v = qp.view(B, n, hq, d), kp.view(B, n, hkv, d), vp.view(B, n, hkv, d)
    out, mass = causal_prefill_attention(q, k, v)
    qh, kh, vh = (x.transpose(1, 2).float() for x in (q, k, v))
    kh, vh = kh.repeat_interleave(hq // hkv, 1), vh.repeat_interleave(hq // hkv, 1)
    s = qh @ kh.transpose(2, 3) / d ** 0.5
    idx = torch.arange(n, device="cuda")
    s = s.masked_fill(idx[None, :] > idx[:, None], float("-inf"))
    p = torch.softmax(s, -1)
    ref = (p @ vh).transpose(1, 2)
    assert torch.allclose(out.float(), ref, atol=2e-3, rtol=2e-3)
    assert torch.allclose(mass, p.sum(dim=(1, 2)), rtol=2e-3, atol=1e-4)


def test_prefill_rejects_what_it_cannot_run():
    from smartkv_b200 import SmartKVLibraryError
    from smartkv_b200.prefill import causal_prefill_attention
    q = torch.randn((1, 8, 4, 64), device="cuda")
    with pytest.raises(TypeError):
        causal_prefill_attention(q, q, q)                                   # fp32
    h = torch.randn((1, 8, 4, 96), device="cuda").half()
    with pytest.raises(SmartKVLibraryError):
        causal_prefill_attention(h, h, h)                                   # head_dim 96
