"""Entrywise operators: CUDA kernels (``csrc/elementwise.cu``) with PyTorch CPU twins.

``unary(name, x, p0, p1)`` / ``binary(name, a, b)`` are differentiable; on CUDA tensors the
forward and backward both run the library's vectorised kernels, on CPU tensors plain
PyTorch expressions with the same formulas.  Operator list and semantics follow the
reference's operator layers (src/operators/**, src/proto/operators.proto:35-196).
"""
from __future__ import annotations

import math

import torch

from . import native
from .native import c_float, c_int, c_ll, c_void_p

UNARY = ["identity", "logical_not", "abs", "negative", "sign", "round", "ceil", "floor",
         "reciprocal", "square", "sqrt", "rsqrt", "safe_reciprocal", "exp", "expm1", "log",
         "log1p", "cos", "sin", "tan", "acos", "asin", "atan", "cosh", "sinh", "tanh", "acosh",
         "asinh", "atanh", "erf", "erfinv", "gelu", "log_sigmoid", "selu", "sigmoid", "softplus",
         "softsign", "relu", "leaky_relu", "elu", "add_constant", "scale", "subtract_constant",
         "constant_subtract", "max_constant", "min_constant", "equal_constant",
         "not_equal_constant", "less_constant", "less_equal_constant", "greater_constant",
         "greater_equal_constant", "clamp", "gelu_tanh"]
BINARY = ["add", "subtract", "multiply", "divide", "mod", "pow", "safe_divide",
          "squared_difference", "max", "min", "equal", "not_equal", "less", "less_equal",
          "greater", "greater_equal", "logical_and", "logical_or", "logical_xor",
          "binary_cross_entropy", "sigmoid_binary_cross_entropy", "boolean_accuracy",
          "boolean_false_negative", "boolean_false_positive", "add_relu"]
UNARY_CODE = {n: i for i, n in enumerate(UNARY)}
BINARY_CODE = {n: i for i, n in enumerate(BINARY)}

_SELU_A, _SELU_S = 1.6732632423543772, 1.0507009873554805


def _safe(y):
    return torch.where(torch.isfinite(y), y, torch.zeros_like(y))


_CPU_UNARY = {
    "identity": lambda x, a, b: x,
    "logical_not": lambda x, a, b: (x == 0).to(x.dtype),
    "abs": lambda x, a, b: x.abs(),
    "negative": lambda x, a, b: -x,
    "sign": lambda x, a, b: torch.sign(x),
    "round": lambda x, a, b: torch.where(x >= 0, torch.floor(x + 0.5), torch.ceil(x - 0.5)).detach() + 0 * x,
    "ceil": lambda x, a, b: torch.ceil(x).detach() + 0 * x,
    "floor": lambda x, a, b: torch.floor(x).detach() + 0 * x,
    "reciprocal": lambda x, a, b: 1 / x,
    "square": lambda x, a, b: x * x,
    "sqrt": lambda x, a, b: torch.sqrt(x),
    "rsqrt": lambda x, a, b: torch.rsqrt(x),
    "safe_reciprocal": lambda x, a, b: _safe(1 / x),
    "exp": lambda x, a, b: torch.exp(x),
    "expm1": lambda x, a, b: torch.expm1(x),
    "log": lambda x, a, b: torch.log(x),
    "log1p": lambda x, a, b: torch.log1p(x),
    "cos": lambda x, a, b: torch.cos(x),
    "sin": lambda x, a, b: torch.sin(x),
    "tan": lambda x, a, b: torch.tan(x),
    "acos": lambda x, a, b: torch.acos(x),
    "asin": lambda x, a, b: torch.asin(x),
    "atan": lambda x, a, b: torch.atan(x),
    "cosh": lambda x, a, b: torch.cosh(x),
    "sinh": lambda x, a, b: torch.sinh(x),
    "tanh": lambda x, a, b: torch.tanh(x),
    "acosh": lambda x, a, b: torch.acosh(x),
    "asinh": lambda x, a, b: torch.asinh(x),
    "atanh": lambda x, a, b: torch.atanh(x),
    "erf": lambda x, a, b: torch.erf(x),
    "erfinv": lambda x, a, b: torch.erfinv(x),
    "gelu": lambda x, a, b: torch.nn.functional.gelu(x),
    "gelu_tanh": lambda x, a, b: torch.nn.functional.gelu(x, approximate="tanh"),
    "log_sigmoid": lambda x, a, b: torch.nn.functional.logsigmoid(x),
    "selu": lambda x, a, b: torch.nn.functional.selu(x),
    "sigmoid": lambda x, a, b: torch.sigmoid(x),
    "softplus": lambda x, a, b: torch.nn.functional.softplus(x),
    "softsign": lambda x, a, b: torch.nn.functional.softsign(x),
    "relu": lambda x, a, b: torch.relu(x),
    "leaky_relu": lambda x, a, b: torch.nn.functional.leaky_relu(x, a),
    "elu": lambda x, a, b: torch.nn.functional.elu(x, a),
    "add_constant": lambda x, a, b: x + a,
    "scale": lambda x, a, b: x * a,
    "subtract_constant": lambda x, a, b: x - a,
    "constant_subtract": lambda x, a, b: a - x,
    "max_constant": lambda x, a, b: torch.clamp(x, min=a),
    "min_constant": lambda x, a, b: torch.clamp(x, max=a),
    "equal_constant": lambda x, a, b: (x == a).to(x.dtype),
    "not_equal_constant": lambda x, a, b: (x != a).to(x.dtype),
    "less_constant": lambda x, a, b: (x < a).to(x.dtype),
    "less_equal_constant": lambda x, a, b: (x <= a).to(x.dtype),
    "greater_constant": lambda x, a, b: (x > a).to(x.dtype),
    "greater_equal_constant": lambda x, a, b: (x >= a).to(x.dtype),
    "clamp": lambda x, a, b: torch.clamp(x, a, b),
}


def _bce(p, t):
    out = torch.zeros_like(p)
    out = out + torch.where(t > 0, -t * torch.log(p), torch.zeros_like(p))
    out = out + torch.where(t < 1, -(1 - t) * torch.log(1 - p), torch.zeros_like(p))
    return out


def _sig_bce(x, t):
    z = torch.clamp(t, 0, 1)
    return torch.where(x > 0, (1 - z) * x + torch.log1p(torch.exp(-x.abs())),
                       -x * z + torch.log1p(torch.exp(-x.abs())))


_CPU_BINARY = {
    "add": lambda a, b: a + b,
    "subtract": lambda a, b: a - b,
    "multiply": lambda a, b: a * b,
    "divide": lambda a, b: a / b,
    "mod": lambda a, b: torch.fmod(a, b),
    "pow": lambda a, b: torch.pow(a, b),
    "safe_divide": lambda a, b: _safe(a / b),
    "squared_difference": lambda a, b: (a - b) ** 2,
    "max": lambda a, b: torch.maximum(a, b),
    "min": lambda a, b: torch.minimum(a, b),
    "equal": lambda a, b: (a == b).to(a.dtype),
    "not_equal": lambda a, b: (a != b).to(a.dtype),
    "less": lambda a, b: (a < b).to(a.dtype),
    "less_equal": lambda a, b: (a <= b).to(a.dtype),
    "greater": lambda a, b: (a > b).to(a.dtype),
    "greater_equal": lambda a, b: (a >= b).to(a.dtype),
    "logical_and": lambda a, b: ((a != 0) & (b != 0)).to(a.dtype),
    "logical_or": lambda a, b: ((a != 0) | (b != 0)).to(a.dtype),
    "logical_xor": lambda a, b: ((a != 0) ^ (b != 0)).to(a.dtype),
    "binary_cross_entropy": _bce,
    "sigmoid_binary_cross_entropy": _sig_bce,
    "boolean_accuracy": lambda a, b: ((a >= 0.5) == (b >= 0.5)).to(a.dtype),
    "boolean_false_negative": lambda a, b: ((a < 0.5) & (b >= 0.5)).to(a.dtype),
    "boolean_false_positive": lambda a, b: ((a >= 0.5) & (b < 0.5)).to(a.dtype),
}

_configured = False


def _lib():
    global _configured
    lib = native.cuda_lib()
    if not _configured:
        lib.lb_unary.restype = c_int
        lib.lb_unary.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_float,
                                 c_float, c_int, c_void_p]
        lib.lb_binary.restype = c_int
        lib.lb_binary.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int,
                                  c_int, c_int, c_void_p]
        _configured = True
    return lib


def _dense(t: torch.Tensor) -> bool:
    return t.is_contiguous() or t.is_contiguous(memory_format=torch.channels_last) or \
        (t.dim() == 5 and t.is_contiguous(memory_format=torch.channels_last_3d))


def unary_raw(code: int, x, dy, p0: float, p1: float, mode: int):
    """Launch the unary kernel on a dense tensor (any memory format); returns a tensor with
    the same strides as ``x``."""
    out = torch.empty_like(x)
    rc = _lib().lb_unary(x.data_ptr(), native.ptr(dy), out.data_ptr(), x.numel(), code, mode,
                         float(p0), float(p1), native.dtype_code(x.dtype), native.stream_ptr())
    native.check(rc, "lb_unary")
    native.count_launch()
    return out


class _Unary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, code, p0, p1):
        ctx.save_for_backward(x)
        ctx.args = (code, p0, p1)
        return unary_raw(code, x, None, p0, p1, 0)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        code, p0, p1 = ctx.args
        if dy.stride() != x.stride():
            dy = torch.empty_like(x).copy_(dy)
        return unary_raw(code, x, dy, p0, p1, 1), None, None, None


class _Binary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, code):
        ctx.save_for_backward(a, b)
        ctx.code = code
        out = torch.empty_like(a)
        rc = _lib().lb_binary(a.data_ptr(), b.data_ptr(), 0, out.data_ptr(), 0, a.numel(), code,
                              0, native.dtype_code(a.dtype), native.stream_ptr())
        native.check(rc, "lb_binary")
        native.count_launch()
        return out

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        if ctx.code == BINARY_CODE["add"]:
            return dy, dy, None          # no kernel, no copies
        if dy.stride() != a.stride():
            dy = torch.empty_like(a).copy_(dy)
        da, db = torch.empty_like(a), torch.empty_like(a)
        rc = _lib().lb_binary(a.data_ptr(), b.data_ptr(), dy.data_ptr(), da.data_ptr(),
                              db.data_ptr(), a.numel(), ctx.code, 1,
                              native.dtype_code(a.dtype), native.stream_ptr())
        native.check(rc, "lb_binary")
        native.count_launch()
        return da, db, None


class _AddRelu(torch.autograd.Function):
    """relu(a + b) in one kernel; backward is one masking pass on the saved output and both
    inputs receive the same gradient tensor."""

    @staticmethod
    def forward(ctx, a, b):
        out = torch.empty_like(a)
        rc = _lib().lb_binary(a.data_ptr(), b.data_ptr(), 0, out.data_ptr(), 0, a.numel(),
                              BINARY_CODE["add_relu"], 0, native.dtype_code(a.dtype), native.stream_ptr())
        native.check(rc, "lb_binary")
        native.count_launch()
        ctx.save_for_backward(out)
        return out

    @staticmethod
    def backward(ctx, dy):
        (out,) = ctx.saved_tensors
        if dy.stride() != out.stride():
            dy = torch.empty_like(out).copy_(dy)
        g = unary_raw(UNARY_CODE["relu"], out, dy, 0.0, 0.0, 1)
        return g, g


def add_relu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """relu(a + b); one native kernel each way for dense same-layout CUDA tensors."""
    if (a.is_cuda and a.dtype in _NATIVE_DTYPES and a.dtype == b.dtype and a.shape == b.shape
            and a.stride() == b.stride() and _dense(a) and a.numel() > 0):
        return _AddRelu.apply(a, b)
    return torch.relu(a + b)


_NATIVE_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def unary(name: str, x: torch.Tensor, p0: float = 0.0, p1: float = 0.0) -> torch.Tensor:
    if x.is_cuda and x.dtype in _NATIVE_DTYPES and _dense(x) and x.numel() > 0:
        return _Unary.apply(x, UNARY_CODE[name], float(p0), float(p1))
    return _CPU_UNARY[name](x, p0, p1)


def binary(name: str, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if (a.is_cuda and a.dtype in _NATIVE_DTYPES and a.shape == b.shape and a.dtype == b.dtype
            and a.stride() == b.stride() and _dense(a) and a.numel() > 0):
        return _Binary.apply(a, b, BINARY_CODE[name])
    return _CPU_BINARY[name](a, b)
