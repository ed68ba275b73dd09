"""Convolution front door (channels-last): tcgen05 implicit GEMM on CUDA, PyTorch on CPU.

Tensors handed to the kernels are NDHWC views ``[N, D, H, W, C]`` (2-D convolutions use
``D = 1``) and filters are tap-major ``[taps, Kout, C]``.  ``pack_filter`` converts the
reference's ``Kout x C x [D x] H x W`` kernel layout
(src/layers/learning/base_convolution.cpp:352-391) to that form.
"""
from __future__ import annotations

import ctypes

import torch

from . import native
from .native import c_float, c_int, c_void_p

_configured = False


def _lib():
    global _configured
    lib = native.cuda_lib()
    if not _configured:
        lib.lb_conv_fwd_tc.restype = c_int
        lib.lb_conv_fwd_tc.argtypes = [
            c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_int),
            ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong),
            c_int, c_int, c_float, c_float, c_int, c_float, c_void_p]
        lib.lb_conv_fwd_halo_tc.restype = c_int
        lib.lb_conv_fwd_halo_tc.argtypes = [
            c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_int),
            ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong),
            c_int, c_int, c_float, c_float, c_int, c_float, c_void_p, c_void_p]
        lib.lb_conv_wgrad_tc.restype = c_int
        lib.lb_conv_wgrad_tc.argtypes = [
            c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_int),
            ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong),
            ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, c_int, c_float, c_void_p]
        _configured = True
    return lib


class HaloSyncArgs(ctypes.Structure):
    """Mirror of ``lb::HaloSyncArgs`` (csrc/halo_sync.cuh)."""
    _fields_ = [("up_dst", c_void_p), ("down_dst", c_void_p), ("up_flag", c_void_p),
                ("down_flag", c_void_p), ("top_flag", c_void_p), ("bot_flag", c_void_p),
                ("local", c_void_p), ("h", ctypes.c_longlong)]


def norm3(v, fill):
    """Broadcast a scalar / 1-/2-/3-tuple to (d, h, w), filling missing dims with ``fill``."""
    if isinstance(v, int):
        return (v, v, v)
    v = tuple(int(i) for i in v)
    return (fill,) * (3 - len(v)) + v


def pack_filter(w: torch.Tensor, dtype: torch.dtype, *, for_dgrad: bool = False) -> torch.Tensor:
    """``Kout x C x k...`` -> ``[taps, Kout, C]``; for the data gradient the taps are
    reversed and the channel roles swapped: ``[taps, C, Kout]``."""
    K, C = w.shape[0], w.shape[1]
    taps = w[0, 0].numel()
    wt = w.reshape(K, C, taps)
    if for_dgrad:
        return wt.flip(2).permute(2, 1, 0).contiguous().to(dtype)
    return wt.permute(2, 0, 1).contiguous().to(dtype)


def out_size(i, k, p, s, d):
    return (i + 2 * p - d * (k - 1) - 1) // s + 1


def conv_fwd(x: torch.Tensor, w_taps: torch.Tensor, ksize, *, pad=0, stride=1, dilation=1,
             bias: torch.Tensor | None = None, act: int = native.ACT_NONE,
             act_param: float = 0.0, out: torch.Tensor | None = None,
             out_dtype: torch.dtype | None = None, alpha: float = 1.0, beta: float = 0.0,
             out_dims=None, halo=None) -> torch.Tensor:
    """x: [N, D, H, W, C] view (C contiguous).  w_taps: [taps, Kout, C].  Returns NDHWC.
    ``halo``: a ``HaloSyncArgs`` structure (csrc/halo_sync.cuh) when ``x`` is a rank's
    depth-extended tensor in symmetric memory: the kernel then exchanges the halo planes with
    the depth neighbours itself (CUDA only, depth padding 0)."""
    N, D, H, W, C = x.shape
    kd, kh, kw = norm3(ksize, 1)
    pd, ph, pw = norm3(pad, 0)
    sd, sh, sw = norm3(stride, 1)
    dd, dh, dw = norm3(dilation, 1)
    Kout = w_taps.shape[1]
    if out_dims is None:
        Do, Ho, Wo = out_size(D, kd, pd, sd, dd), out_size(H, kh, ph, sh, dh), out_size(W, kw, pw, sw, dw)
    else:
        Do, Ho, Wo = out_dims
    out_dtype = out_dtype or (out.dtype if out is not None else x.dtype)

    if not x.is_cuda:
        wt = w_taps.float().reshape(kd, kh, kw, Kout, C).permute(3, 4, 0, 1, 2)
        xin = x.float().permute(0, 4, 1, 2, 3)
        # out_dims may ask for fewer/more outputs than the canonical formula (data gradient
        # with asymmetric implicit padding): pad on the far side as needed.
        extra = [max(0, (o - 1) * s + d_ * (k - 1) + 1 - (i + 2 * p))
                 for o, s, d_, k, i, p in ((Do, sd, dd, kd, D, pd), (Ho, sh, dh, kh, H, ph),
                                           (Wo, sw, dw, kw, W, pw))]
        lo = [max(p, 0) for p in (pd, ph, pw)]
        xin = torch.nn.functional.pad(xin, (lo[2], lo[2] + extra[2], lo[1], lo[1] + extra[1],
                                            lo[0], lo[0] + extra[0]))
        crop = [max(-p, 0) for p in (pd, ph, pw)]
        xin = xin[:, :, crop[0]:, crop[1]:, crop[2]:]
        y = torch.nn.functional.conv3d(xin, wt, None, (sd, sh, sw), 0, (dd, dh, dw))
        y = y[:, :, :Do, :Ho, :Wo].permute(0, 2, 3, 4, 1) * alpha
        if bias is not None:
            y = y + bias.float()
        if beta != 0.0 and out is not None:
            y = y + beta * out.float()
        from .gemm import _ACT_FN
        y = _ACT_FN[act](y, act_param)
        if out is None:
            return y.to(out_dtype).contiguous()
        out.copy_(y)
        return out

    if x.stride(4) != 1:
        raise ValueError("conv_fwd: channel dimension must be contiguous")
    if w_taps.dtype != x.dtype or not w_taps.is_contiguous():
        w_taps = w_taps.to(x.dtype).contiguous()
    if out is None:
        out = torch.empty((N, Do, Ho, Wo, Kout), dtype=out_dtype, device=x.device)
        if beta != 0.0:
            out.zero_()
    geom = (c_int * 21)(N, D, H, W, C, Do, Ho, Wo, Kout, kd, kh, kw, pd, ph, pw, sd, sh, sw,
                        dd, dh, dw)
    xs = (ctypes.c_longlong * 4)(x.stride(0), x.stride(1), x.stride(2), x.stride(3))
    ys = (ctypes.c_longlong * 4)(out.stride(0), out.stride(1), out.stride(2), out.stride(3))
    if bias is not None and bias.dtype != torch.float32:
        bias = bias.float()
    scratch = native.offer_splitk(N * Do * Ho * Wo, Kout, x.device) if C * kd * kh * kw >= 512 else None
    rc = _lib().lb_conv_fwd_halo_tc(x.data_ptr(), w_taps.data_ptr(), out.data_ptr(), native.ptr(bias),
                                    geom, xs, ys, native.dtype_code(x.dtype),
                                    native.dtype_code(out.dtype), float(alpha), float(beta), int(act),
                                    float(act_param),
                                    ctypes.cast(ctypes.pointer(halo), c_void_p) if halo is not None else None,
                                    native.stream_ptr())
    native.check(rc, "lb_conv_fwd_halo_tc")
    native.count_launch()
    del scratch
    return out


def conv_wgrad(x: torch.Tensor, dy: torch.Tensor, ksize, *, pad=0, stride=1, dilation=1,
               out: torch.Tensor | None = None, alpha: float = 1.0) -> torch.Tensor:
    """Filter gradient, ADDED (times ``alpha``) into ``out``, an fp32 tensor in the
    reference's ``Kout x C x [kd x] kh x kw`` layout (zero-initialised when omitted).

    x: [N, D, H, W, C] view, dy: [N, Do, Ho, Wo, Kout] view, channels contiguous.
    """
    N, D, H, W, C = x.shape
    _, Do, Ho, Wo, Kout = dy.shape
    kd, kh, kw = norm3(ksize, 1)
    pd, ph, pw = norm3(pad, 0)
    sd, sh, sw = norm3(stride, 1)
    dd, dh, dw = norm3(dilation, 1)
    taps = kd * kh * kw
    if out is None:
        out = torch.zeros((Kout, C, kd, kh, kw), dtype=torch.float32, device=x.device)
    if not x.is_cuda:
        xin = x.float().permute(0, 4, 1, 2, 3)
        g = dy.float().permute(0, 4, 1, 2, 3)
        wshape = (Kout, C, kd, kh, kw)
        gw = torch.nn.grad.conv3d_weight(xin, wshape, g, (sd, sh, sw), (pd, ph, pw), (dd, dh, dw))
        out.view(wshape).add_(gw, alpha=alpha)
        return out
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise ValueError("conv_wgrad: out must be a contiguous fp32 tensor")
    if dy.dtype != x.dtype:
        dy = dy.to(x.dtype)
    geom = (c_int * 21)(N, D, H, W, C, Do, Ho, Wo, Kout, kd, kh, kw, pd, ph, pw, sd, sh, sw,
                        dd, dh, dw)
    xs = (ctypes.c_longlong * 4)(x.stride(0), x.stride(1), x.stride(2), x.stride(3))
    ys = (ctypes.c_longlong * 4)(dy.stride(0), dy.stride(1), dy.stride(2), dy.stride(3))
    rc = _lib().lb_conv_wgrad_tc(x.data_ptr(), dy.data_ptr(), out.data_ptr(), geom, xs, ys,
                                 1, C * taps, taps, native.dtype_code(x.dtype), float(alpha),
                                 native.stream_ptr())
    native.check(rc, "lb_conv_wgrad_tc")
    native.count_launch()
    return out
