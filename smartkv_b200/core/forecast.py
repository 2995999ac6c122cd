"""Mirror of ``smartkv.core.forecast`` (smartkv/core/forecast.py:26-62): the small online regressor whose
prediction of a token's next importance is blended into the allocation scores
(smartkv/core/cache.py:313-336).  Host-side policy, as in the reference: a 6 -> 16 -> 1 perceptron trained with
Adam on (feature, log1p(importance)) pairs, a few dozen rows per update.

Written over four plain tensors instead of ``nn.Module`` objects.  They are drawn exactly as ``nn.Linear`` draws
its parameters (first layer's weight, its bias, second layer's weight, its bias; each uniform in
+-1/sqrt(fan_in)), so a seeded construction starts from the weights a seeded construction of the reference's
predictor starts from, and ``torch.nn.functional.linear`` is the same addmm the module would run."""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn.functional as F


def _linear_params(fan_out: int, fan_in: int, device) -> List[torch.Tensor]:
    # nn.Linear.reset_parameters: kaiming_uniform_(weight, a=sqrt(5)), then the bias in +-1/sqrt(fan_in)
    gain = math.sqrt(2.0 / (1.0 + math.sqrt(5.0) ** 2))
    w_bound = math.sqrt(3.0) * (gain / math.sqrt(fan_in))
    weight = torch.empty((fan_out, fan_in), dtype=torch.float32).uniform_(-w_bound, w_bound)
    b_bound = 1.0 / math.sqrt(fan_in) if fan_in > 0 else 0.0
    bias = torch.empty(fan_out, dtype=torch.float32).uniform_(-b_bound, b_bound)
    return [weight.to(device).requires_grad_(True), bias.to(device).requires_grad_(True)]


class ForecastPredictor:
    def __init__(self, feature_dim: int, hidden_dim: int = 16, lr: float = 5e-2, device: str = "cpu") -> None:
        self.device = torch.device(device)
        dims = [feature_dim, hidden_dim, 1] if hidden_dim and hidden_dim > 0 else [feature_dim, 1]
        self.params: List[torch.Tensor] = []          # weight, bias per layer, in the order nn.Linear would draw them
        for fan_in, fan_out in zip(dims[:-1], dims[1:]):
            self.params += _linear_params(fan_out, fan_in, self.device)
        self.optimizer = torch.optim.Adam(self.params, lr=lr)
        self._loss: Optional[float] = None

    def _net(self, x: torch.Tensor) -> torch.Tensor:
        layers = len(self.params) // 2
        for i in range(layers):
            x = F.linear(x, self.params[2 * i], self.params[2 * i + 1])
            if i + 1 < layers:
                x = torch.relu(x)
        return x.squeeze(-1)

    def predict(self, features: torch.Tensor) -> torch.Tensor:
        """features [n, feature_dim] -> predictions [n] on the CPU."""
        with torch.no_grad():
            return self._net(features.to(self.device)).cpu()

    def update(self, features: torch.Tensor, targets: torch.Tensor) -> float:
        """One Adam step on the mean squared error of the batch; returns the loss."""
        loss = F.mse_loss(self._net(features.to(self.device)), targets.to(self.device))
        self.optimizer.zero_grad()
        loss.backward()
        self.optimizer.step()
        self._loss = float(loss.item())
        return self._loss

    @property
    def last_loss(self) -> Optional[float]:
        return self._loss
