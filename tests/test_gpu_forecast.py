"""``enable_forecast`` (the reference's online importance predictor, smartkv/core/forecast.py and
smartkv/core/cache.py:313-336, :746-804) on the mirror cache, against a run of the reference's own cache on
the same seeded attention rows (fixture tests/golden/forecast.npz).  The predictor is host code in both; what
can differ is the last bit of an importance sum computed on the GPU, so the comparison allows a few
borderline widths and asks for the same training history."""
import os

import numpy as np
import pytest
import torch

from tests.e2e_model import forecast_inputs

pytestmark = pytest.mark.gpu
Z = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "forecast.npz")


def test_forecast_blend_tracks_the_reference():
    from smartkv_b200 import SmartKVCache
    z = np.load(Z)
    L, H, D, n, steps = (int(x) for x in z["f_shape"])
    prompt, rows = forecast_inputs(L, H, n, steps)
    rng = np.random.default_rng(42)
    torch.manual_seed(123)
    c = SmartKVCache(num_layers=L, num_heads=H, head_dim=D, memory_budget=0.45, device="cuda", enable_forecast=True,
                     forecast_update_interval=16, forecast_blend=0.5, forecast_lr=0.05, max_tokens=n + steps + 8)
    assert c.enable_forecast and c.forecast_predictor is not None
    updates = [0]
    orig = c.forecast_predictor.update
    c.forecast_predictor.update = lambda f, t: (updates.__setitem__(0, updates[0] + 1), orig(f, t))[1]
    ids = list(range(n))
    for l in range(L):
        c.update_attention(l, torch.from_numpy(prompt[l]).cuda(), ids)
        c.quantize_and_store_batch(l, ids, torch.from_numpy(rng.standard_normal((n, H, D)).astype(np.float32)).cuda(),
                                   torch.from_numpy(rng.standard_normal((n, H, D)).astype(np.float32)).cuda())
    for t in range(steps):
        keys = list(range(n + t + 1))
        for l in range(L):
            c.update_attention(l, torch.from_numpy(rows[t][l]).cuda(), keys)
            c.quantize_and_store(l, n + t, torch.from_numpy(rng.standard_normal((H, D)).astype(np.float32)).cuda(),
                                 torch.from_numpy(rng.standard_normal((H, D)).astype(np.float32)).cuda())
    c.store.check_errors()
    assert c.realloc_counter == int(z["f_reallocs"]) and updates[0] == int(z["f_updates"])
    imp = np.array([c.get_importance(t) for t in range(n + steps)])
    assert np.allclose(imp, z["f_importance"], rtol=1e-5, atol=1e-6)
    w0 = c.forecast_predictor.params[0].detach().numpy()
    assert np.allclose(w0, z["f_w0"], atol=2e-3), np.abs(w0 - z["f_w0"]).max()
    assert abs(c.forecast_last_loss - float(z["f_last_loss"])) <= 1e-3
    bits = np.array([c.get_precision(t) for t in range(n + steps)])
    assert (bits == z["f_bits"]).mean() >= 0.97, (bits == z["f_bits"]).mean()
    assert c.get_memory_stats()["memory_ratio_true"] <= 0.45 + 1e-6
