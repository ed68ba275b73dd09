"""Fused scaled-dot-product attention (``csrc/attention_tc.cu``) with its PyTorch twin.

``attention(q, k, v, num_heads, scale, causal)`` takes token-major tensors ``[B, S, E]``
(any batch / token strides, e.g. the three column blocks of a packed ``[B, S, 3E]``
projection) and returns ``[B, S, E]``: per head ``softmax(scale * Q K^T [+ causal mask]) V``.
``attention_packed(qkv, ...)`` is the self-attention form whose backward writes the three
gradients straight into one ``[B, S, 3E]`` tensor.

The reference builds this from eight layers and keeps the ``[heads, S, S]`` scores in memory
(python/lbann/modules/transformer/attention.py:215-299); ``exec/model.py`` recognises that
sub-graph and routes it here.  On a GPU with 16-bit inputs, head dimension 128 and sequence
lengths that are multiples of 128 the tcgen05 kernels run; anything else takes the PyTorch
formulation below (fp32 softmax), which is also the test oracle.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import native
from .native import c_float, c_int, c_ll, c_void_p

_configured = False


def _lib():
    global _configured
    lib = native.cuda_lib()
    if not _configured:
        P = ctypes.POINTER(c_ll)
        lib.lb_attention_fwd.restype = c_int
        lib.lb_attention_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                         c_int, c_int, P, P, P, P, c_float, c_int, c_int, c_void_p]
        lib.lb_attention_bwd.restype = c_int
        lib.lb_attention_bwd.argtypes = [c_void_p] * 10 + [c_int, c_int, c_int, c_int] + [P] * 8 + \
            [c_float, c_int, c_int, c_void_p]
        _configured = True
    return lib


def reference_attention(q, k, v, num_heads: int, scale: float, causal: bool) -> torch.Tensor:
    """The same function in plain PyTorch (scores and softmax in fp32)."""
    B, Sq, E = q.shape
    Sk = k.shape[1]
    D = E // num_heads
    qh = q.reshape(B, Sq, num_heads, D).permute(0, 2, 1, 3).float()
    kh = k.reshape(B, Sk, num_heads, D).permute(0, 2, 1, 3).float()
    vh = v.reshape(B, Sk, num_heads, D).permute(0, 2, 1, 3).float()
    s = (qh @ kh.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).triu(1)
        s = s.masked_fill(mask, float("-inf"))
    o = torch.softmax(s, dim=-1) @ vh
    return o.permute(0, 2, 1, 3).reshape(B, Sq, E).to(q.dtype)


def native_ok(q, k, v, num_heads: int, causal: bool) -> bool:
    if not (q.is_cuda and q.dtype in (torch.float16, torch.bfloat16) and k.dtype == q.dtype
            and v.dtype == q.dtype):
        return False
    B, Sq, E = q.shape
    Sk = k.shape[1]
    if E != num_heads * 128 or Sq % 128 or Sk % 128 or (causal and Sq != Sk):
        return False
    for t in (q, k, v):
        if t.stride(2) != 1 or t.stride(1) % 8 or t.stride(0) % 8 or t.data_ptr() % 16:
            return False
    return True


def _strides(t):
    """(batch, token, head) element strides of a [B, S, H * 128] tensor."""
    return (c_ll * 3)(t.stride(0), t.stride(1), 128)


def _fwd(q, k, v, H, scale, causal):
    B, Sq, E = q.shape
    o = torch.empty((B, Sq, E), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    rc = _lib().lb_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                 B, H, Sq, k.shape[1], _strides(q), _strides(k), _strides(v),
                                 _strides(o), float(scale), int(bool(causal)),
                                 native.dtype_code(q.dtype), native.stream_ptr())
    native.check(rc, "lb_attention_fwd")
    native.count_launch()
    return o, lse


def _bwd(q, k, v, o, do, lse, dq, dk, dv, H, scale, causal):
    B, Sq, E = q.shape
    if do.stride(2) != 1 or do.stride(1) % 8 or do.stride(0) % 8 or do.data_ptr() % 16:
        do = do.contiguous()
    delta = torch.empty_like(lse)
    rc = _lib().lb_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(),
                                 lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                 dv.data_ptr(), B, H, Sq, k.shape[1], _strides(q), _strides(k),
                                 _strides(v), _strides(o), _strides(do), _strides(dq), _strides(dk),
                                 _strides(dv), float(scale), int(bool(causal)),
                                 native.dtype_code(q.dtype), native.stream_ptr())
    native.check(rc, "lb_attention_bwd")
    native.count_launch(3)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, H, scale, causal):
        o, lse = _fwd(q, k, v, H, scale, causal)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (H, scale, causal)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        H, scale, causal = ctx.meta
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
        _bwd(q, k, v, o, do, lse, dq, dk, dv, H, scale, causal)
        return dq, dk, dv, None, None, None


class _AttentionPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, H, scale, causal):
        E = qkv.shape[2] // 3
        q, k, v = qkv[:, :, :E], qkv[:, :, E:2 * E], qkv[:, :, 2 * E:]
        o, lse = _fwd(q, k, v, H, scale, causal)
        ctx.save_for_backward(qkv, o, lse)
        ctx.meta = (H, scale, causal)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        H, scale, causal = ctx.meta
        E = qkv.shape[2] // 3
        q, k, v = qkv[:, :, :E], qkv[:, :, E:2 * E], qkv[:, :, 2 * E:]
        dqkv = torch.empty(qkv.shape, dtype=qkv.dtype, device=qkv.device)
        _bwd(q, k, v, o, do, lse, dqkv[:, :, :E], dqkv[:, :, E:2 * E], dqkv[:, :, 2 * E:], H, scale, causal)
        return dqkv, None, None, None


def attention(q, k, v, num_heads: int, scale: float | None = None, causal: bool = False) -> torch.Tensor:
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1] // num_heads)
    if native_ok(q, k, v, num_heads, causal):
        return _Attention.apply(q, k, v, num_heads, float(scale), bool(causal))
    return reference_attention(q, k, v, num_heads, float(scale), bool(causal))


def attention_packed(qkv, num_heads: int, scale: float | None = None, causal: bool = False) -> torch.Tensor:
    """Self-attention on a packed ``[B, S, 3E]`` projection (queries, keys, values side by
    side along the last dimension)."""
    E = qkv.shape[2] // 3
    if scale is None:
        scale = 1.0 / math.sqrt(E // num_heads)
    q, k, v = qkv[:, :, :E], qkv[:, :, E:2 * E], qkv[:, :, 2 * E:]
    if qkv.dim() == 3 and native_ok(q, k, v, num_heads, causal):
        return _AttentionPacked.apply(qkv, num_heads, float(scale), bool(causal))
    return reference_attention(q, k, v, num_heads, float(scale), bool(causal))
