"""Experimental objective functions and regularisers as modules
(python/lbann/contrib/modules/objective_functions.py)."""
from __future__ import annotations

from ...frontend import core as L
from ...modules import Module


def _two(inputs):
    if len(inputs) != 2:
        raise ValueError("expected two inputs: predictions and labels")
    return inputs


class CrossEntropyWithUncertainty(Module):
    """-log of the probability mass on the allowed classes (labels are 0/1 masks that may
    mark several classes)."""

    def forward(self, inputs):
        pred, label = _two(inputs)
        return L.Negative(L.Log(L.Reduction(L.Multiply(pred, label), mode="sum")))


class GeometricDistributionNegativeLogLikelihood(Module):
    """-sum(k log(1 - p) + log p) for counts k and success probabilities p."""

    def forward(self, inputs):
        pred, label = _two(inputs)
        one_minus = L.AddConstant(L.Negative(pred), constant=1.0)
        full = L.WeightedSum([L.Multiply(label, L.Log(one_minus)), L.Log(pred)], scaling_factors=[-1.0, -1.0])
        return L.Reduction(full, mode="sum")


class PoissonDistributionNegativeLogLikelihood(Module):
    """sum(rate - k log rate + log k!), with log k! = lgamma(k + 1) evaluated by Stirling's
    series (there is no log-gamma layer): k is clamped below at 1, where the series is exact
    to 1e-3 and log 0! = log 1! = 0 anyway."""

    def forward(self, inputs):
        pred, label = _two(inputs)
        k = L.Clamp(label, min=1.0, max=3.0e38)
        logk = L.Log(k)
        # lgamma(k + 1) = k log k - k + 0.5 log(2 pi k) + 1 / (12 k)
        lg = L.WeightedSum([L.Multiply(k, logk), k, logk, L.Reciprocal(k)],
                           scaling_factors=[1.0, -1.0, 0.5, 1.0 / 12.0])
        lg = L.AddConstant(lg, constant=0.9189385332046727)           # 0.5 log(2 pi)
        full = L.WeightedSum([pred, L.Multiply(label, L.Log(pred)), lg], scaling_factors=[1.0, -1.0, 1.0])
        return L.Reduction(full, mode="sum")


class GroupLasso(Module):
    """Sum over the columns of a ``height x width`` weights matrix of their Euclidean norms."""

    def __init__(self, weights, height, width):
        super().__init__()
        self.weights, self.height, self.width = weights, height, width

    def forward(self, _=None):
        w = L.WeightsLayer(weights=self.weights, dims=[self.width, self.height])
        sl = L.Slice(w, axis=0, slice_points=list(range(self.width + 1)))
        cols = [L.Sqrt(L.L2Norm2(L.Identity(sl))) for _ in range(self.width)]
        return L.Sum(cols) if len(cols) > 1 else cols[0]


class L1WeightRegularization(Module):
    def __init__(self, weights, dims):
        super().__init__()
        self.weights, self.dims = weights, list(dims)

    def forward(self, _=None):
        return L.L1Norm(L.WeightsLayer(weights=self.weights, dims=self.dims))
