"""Mirror of ``smartkv.core.forecast`` (smartkv/core/forecast.py:26-62): the small online regressor whose
prediction of a token's next importance is blended into the allocation scores
(smartkv/core/cache.py:313-336).  Host-side policy, as in the reference: a 6 -> 16 -> 1 perceptron trained with
Adam on (feature, log1p(importance)) pairs, a few dozen rows per update."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn


class ForecastPredictor:
    def __init__(self, feature_dim: int, hidden_dim: int = 16, lr: float = 5e-2, device: str = "cpu") -> None:
        self.device = torch.device(device)
        # layer order fixes the order of the random draws of the initialisation, so that a seeded construction
        # gives the weights a seeded construction of the reference's predictor gives
        layers = [nn.Linear(feature_dim, hidden_dim), nn.ReLU(), nn.Linear(hidden_dim, 1)] if hidden_dim and hidden_dim > 0 \
            else [nn.Linear(feature_dim, 1)]
        self.model = nn.Sequential(*layers).to(self.device)
        self.optimizer = torch.optim.Adam(self.model.parameters(), lr=lr)
        self._loss: Optional[float] = None

    def predict(self, features: torch.Tensor) -> torch.Tensor:
        """features [n, feature_dim] -> predictions [n] on the CPU."""
        self.model.eval()
        with torch.no_grad():
            return self.model(features.to(self.device)).squeeze(-1).detach().cpu()

    def update(self, features: torch.Tensor, targets: torch.Tensor) -> float:
        """One Adam step on the mean squared error of the batch; returns the loss."""
        self.model.train()
        preds = self.model(features.to(self.device)).squeeze(-1)
        loss = nn.functional.mse_loss(preds, targets.to(self.device))
        self.optimizer.zero_grad()
        loss.backward()
        self.optimizer.step()
        self._loss = float(loss.item())
        return self._loss

    @property
    def last_loss(self) -> Optional[float]:
        return self._loss
