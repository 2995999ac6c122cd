"""The importance predictor (smartkv_b200/core/forecast.py) against the reference's own
``ForecastPredictor`` (fixture tests/golden/forecast.npz): same seed -> the same initial weights, the same
predictions, and the same five Adam updates, bit for bit.  Host code, no GPU needed."""
import os

import numpy as np
import torch

Z = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "forecast.npz")


def test_predictor_matches_the_reference_bit_for_bit():
    from smartkv_b200.core.forecast import ForecastPredictor
    z = np.load(Z)
    torch.manual_seed(321)
    p = ForecastPredictor(6, lr=0.05)
    x, t = torch.from_numpy(z["fp_x"]), torch.from_numpy(z["fp_t"])
    assert np.array_equal(p.params[0].detach().numpy(), z["fp_w0_init"])
    assert np.array_equal(p.predict(x).numpy(), z["fp_pred_init"])
    losses = np.array([p.update(x, t) for _ in range(5)])
    assert np.array_equal(losses, z["fp_losses"]) and p.last_loss == float(z["fp_losses"][-1])
    assert np.array_equal(p.params[2].detach().numpy(), z["fp_w1_after"])
    assert np.array_equal(p.predict(x).numpy(), z["fp_pred_after"])


def test_predictor_without_hidden_layer_is_one_linear_map():
    from smartkv_b200.core.forecast import ForecastPredictor
    torch.manual_seed(0)
    p = ForecastPredictor(6, hidden_dim=0)
    assert len(p.params) == 2 and p.params[0].shape == (1, 6)
    x = torch.randn(5, 6)
    assert torch.allclose(p.predict(x), (x @ p.params[0].detach().t() + p.params[1].detach()).squeeze(-1))
