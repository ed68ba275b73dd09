"""GEMM front door: tcgen05 kernel on CUDA tensors, plain PyTorch on CPU tensors.

``gemm(a, b, trans_a, trans_b)`` computes ``op(a) @ op(b)`` for 2-D or batched 3-D
row-major tensors, with the epilogue ``act(alpha * acc + beta * out + bias)``.
No transposes are materialised: a transposed operand is handed to the kernel as an
"MN-major" operand.  Mirrors what the reference asks of cuBLAS through ``El::Gemm``
(src/layers/learning/fully_connected.cpp:511-636) including the destination / gradient
scale factors used to accumulate straight into optimizer buffers
(include/lbann/optimizers/optimizer_impl.hpp:263-285).
"""
from __future__ import annotations

import ctypes

import torch

from . import native
from .native import c_float, c_int, c_ll, c_void_p

_ACT_FN = {
    native.ACT_NONE: lambda x, p: x,
    native.ACT_RELU: lambda x, p: torch.relu(x),
    native.ACT_LEAKY: lambda x, p: torch.nn.functional.leaky_relu(x, p),
    native.ACT_GELU: lambda x, p: torch.nn.functional.gelu(x),
    native.ACT_TANH: lambda x, p: torch.tanh(x),
    native.ACT_SIGMOID: lambda x, p: torch.sigmoid(x),
}

_configured = False


def _lib():
    global _configured
    lib = native.cuda_lib()
    if not _configured:
        lib.lb_gemm_tc.restype = c_int
        lib.lb_gemm_tc.argtypes = [
            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
            c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_int, c_int, c_int, c_int,
            c_float, c_float, c_int, c_int, c_float, c_int, c_void_p]
        _configured = True
    return lib


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """Return ``t`` or a copy whose rows start on 16-byte boundaries with a legal pitch."""
    if t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and t.stride(-2) % 8 == 0 and (
            t.dim() == 2 or (t.stride(0) % 8 == 0 and t.stride(0) >= 0)):
        return t
    cols = t.shape[-1]
    pitch = (cols + 7) // 8 * 8
    buf = torch.zeros(*t.shape[:-1], pitch, dtype=t.dtype, device=t.device)
    buf[..., :cols].copy_(t)
    return buf[..., :cols]


def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
         alpha: float = 1.0, beta: float = 0.0, bias: torch.Tensor | None = None,
         bias_per_row: bool = False, act: int = native.ACT_NONE, act_param: float = 0.0,
         bn_hint: int = 0) -> torch.Tensor:
    batched = a.dim() == 3
    if batched != (b.dim() == 3):
        raise ValueError("gemm: both operands must be 2-D or both 3-D")
    M = a.shape[-1] if trans_a else a.shape[-2]
    K = a.shape[-2] if trans_a else a.shape[-1]
    Kb = b.shape[-1] if trans_b else b.shape[-2]
    N = b.shape[-2] if trans_b else b.shape[-1]
    if K != Kb:
        raise ValueError(f"gemm: inner dimensions differ ({K} vs {Kb})")
    nb = a.shape[0] if batched else 1
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else a.dtype

    if not a.is_cuda:
        A = a.float().transpose(-1, -2) if trans_a else a.float()
        B = b.float().transpose(-1, -2) if trans_b else b.float()
        acc = alpha * (A @ B)
        if bias is not None:
            acc = acc + (bias.float().unsqueeze(-1) if bias_per_row else bias.float())
        if beta != 0.0 and out is not None:
            acc = acc + beta * out.float()
        acc = _ACT_FN[act](acc, act_param)
        if out is None:
            return acc.to(out_dtype)
        out.copy_(acc)
        return out

    if a.dtype not in (torch.float16, torch.bfloat16):
        a = a.to(torch.bfloat16)
    if b.dtype != a.dtype:
        b = b.to(a.dtype)
    a = _tma_ready(a)
    b = _tma_ready(b)
    if out is None:
        shape = (nb, M, N) if batched else (M, N)
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
        if beta != 0.0:
            out.zero_()
    elif out.stride(-1) != 1:
        raise ValueError("gemm: output must have unit stride in its last dimension")
    if bias is not None and bias.dtype != torch.float32:
        bias = bias.float()
    scratch = native.offer_splitk(M * nb, N, a.device) if K >= 512 else None
    rc = _lib().lb_gemm_tc(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), native.ptr(bias), M, N, K, nb,
        a.stride(-2), b.stride(-2), out.stride(-2),
        a.stride(0) if batched else 0, b.stride(0) if batched else 0,
        out.stride(0) if batched else 0,
        1 if trans_a else 0, 0 if trans_b else 1,
        native.dtype_code(a.dtype), native.dtype_code(out.dtype),
        float(alpha), float(beta), 2 if bias_per_row else 1, int(act), float(act_param),
        int(bn_hint), native.stream_ptr())
    native.check(rc, "lb_gemm_tc")
    native.count_launch()
    del scratch         # enqueued: the allocator may hand the workspace to later work of this stream
    return out
