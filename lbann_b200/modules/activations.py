"""Activation helpers composed from primitive layers (python/lbann/modules/activations.py)."""
import math

from ..frontend import core as L


def Gelu(x):
    """x * Phi(x) with the exact error function."""
    return L.Gelu(x)


def Gelu_approx(x):
    """tanh approximation 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))."""
    x3 = L.Multiply(L.Square(x), x)
    inner = L.Scale(L.Add(x, L.Scale(x3, constant=0.044715)), constant=math.sqrt(2.0 / math.pi))
    return L.Multiply(L.Scale(x, constant=0.5), L.AddConstant(L.Tanh(inner), constant=1.0))


def Silu(x):
    """x * sigmoid(x)."""
    return L.Multiply(x, L.Sigmoid(x))
