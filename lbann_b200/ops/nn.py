"""Differentiable building blocks over the native kernels.

Each function takes PyTorch tensors; CUDA 16-bit tensors run the sm_100a kernels of this
library (forward and backward), anything else runs the equivalent PyTorch expression so
the whole framework also works on CPU in fp32.  Weight gradients of the native paths are
ACCUMULATED straight into the fp32 gradient buffer of the weight (``WeightHandle.grad``),
mirroring the reference's destination-scale / gradient-scale contract
(include/lbann/optimizers/optimizer_impl.hpp:208-290).
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from . import native
from .conv import conv_fwd, conv_wgrad, norm3, out_size, pack_filter
from .elementwise import UNARY_CODE, unary_raw
from .gemm import gemm
from .native import c_float, c_int, c_ll, c_void_p

_HALF = (torch.float16, torch.bfloat16)
_ACT_UNARY = {native.ACT_RELU: "relu", native.ACT_LEAKY: "leaky_relu"}
_configured = False


def _lib():
    global _configured
    lib = native.cuda_lib()
    if not _configured:
        P = ctypes.POINTER
        lib.lb_pool_fwd.restype = c_int
        lib.lb_pool_fwd.argtypes = [c_void_p, c_void_p, P(c_int), P(c_ll), c_int, c_void_p]
        lib.lb_pool_fwd_strided.restype = c_int
        lib.lb_pool_fwd_strided.argtypes = [c_void_p, c_void_p, P(c_int), P(c_ll), c_ll, c_int, c_void_p]
        lib.lb_pool_fwd_idx.restype = c_int
        lib.lb_pool_fwd_idx.argtypes = [c_void_p, c_void_p, c_void_p, P(c_int), P(c_ll), c_ll, c_int, c_void_p]
        lib.lb_pool_fwd_tiled.restype = c_int
        lib.lb_pool_fwd_tiled.argtypes = [c_void_p, c_void_p, c_void_p, P(c_int), P(c_ll), c_ll, c_int, c_void_p]
        lib.lb_pool_bwd_tiled_idx.restype = c_int
        lib.lb_pool_bwd_tiled_idx.argtypes = [c_void_p, c_void_p, c_void_p, P(c_int), c_int, c_float,
                                              c_ll, c_int, c_void_p]
        lib.lb_pool_bwd_tiled_strided.restype = c_int
        lib.lb_pool_bwd_tiled_strided.argtypes = [c_void_p, c_void_p, c_void_p, P(c_int), c_int, c_float,
                                                  c_ll, c_int, c_void_p]
        VPP = P(c_void_p)
        lib.lb_bn_fused_ws_floats.restype = c_int
        lib.lb_bn_fused_ws_floats.argtypes = [c_int]
        lib.lb_bn_fused_fwd.restype = c_int
        lib.lb_bn_fused_fwd.argtypes = [c_void_p] * 8 + [c_ll, c_int, c_float, c_float, c_float, c_float,
                                                       c_int, c_float, c_int, VPP, VPP, c_int, c_int, c_ll,
                                                       c_void_p, c_void_p]
        lib.lb_bn_fused_bwd.restype = c_int
        lib.lb_bn_fused_bwd.argtypes = [c_void_p] * 9 + [c_ll, c_int, c_float, c_float, c_float, c_int,
                                                       c_float, c_int, VPP, VPP, c_int, c_int, c_ll,
                                                       c_void_p, c_void_p]
        lib.lb_pool_bwd.restype = c_int
        lib.lb_pool_bwd.argtypes = [c_void_p, c_void_p, c_void_p, P(c_int), P(c_ll), c_int, c_void_p]
        lib.lb_layer_norm_fwd.restype = c_int
        lib.lb_layer_norm_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_ll, c_int, c_float, c_int, c_void_p]
        lib.lb_layer_norm_bwd.restype = c_int
        lib.lb_layer_norm_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p]
        lib.lb_bn_partial_sums.restype = c_int
        lib.lb_bn_partial_sums.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p]
        lib.lb_pack_filter.restype = c_int
        lib.lb_pack_filter.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                       c_int, c_void_p]
        lib.lb_outer_accum.restype = c_int
        lib.lb_outer_accum.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_ll, c_float,
                                       c_float, c_int, c_void_p]
        lib.lb_bn_finalize_apply.restype = c_int
        lib.lb_bn_finalize_apply.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int,
                                             c_float, c_float, c_float, c_float, c_int, c_float,
                                             c_int, c_void_p]
        lib.lb_bn_apply_fixed.restype = c_int
        lib.lb_bn_apply_fixed.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_ll, c_int, c_float, c_int, c_float, c_int, c_void_p]
        lib.lb_bn_bwd_sums.restype = c_int
        lib.lb_bn_bwd_sums.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_ll, c_int, c_int, c_float, c_int, c_float, c_int, c_int, c_void_p]
        lib.lb_bn_bwd_apply.restype = c_int
        lib.lb_bn_bwd_apply.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_ll, c_int, c_int, c_float, c_float, c_float,
                                        c_int, c_float, c_int, c_void_p]
        lib.lb_softmax_fwd.restype = c_int
        lib.lb_softmax_fwd.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_int, c_float, c_int, c_int,
                                       c_void_p]
        lib.lb_softmax_bwd.restype = c_int
        lib.lb_softmax_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_float,
                                       c_int, c_int, c_void_p]
        lib.lb_softmax_ce_fwd.restype = c_int
        lib.lb_softmax_ce_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int,
                                          c_void_p]
        lib.lb_softmax_ce_bwd.restype = c_int
        lib.lb_softmax_ce_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                                          c_ll, c_int, c_int, c_void_p]
        lib.lb_sample_loss_fwd.restype = c_int
        lib.lb_sample_loss_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int,
                                           c_void_p]
        lib.lb_sample_loss_bwd.restype = c_int
        lib.lb_sample_loss_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll,
                                           c_ll, c_int, c_int, c_void_p]
        lib.lb_topk_accuracy.restype = c_int
        lib.lb_topk_accuracy.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int,
                                         c_void_p]
        lib.lb_pool_bwd_tiled.restype = c_int
        lib.lb_pool_bwd_tiled.argtypes = [c_void_p, c_void_p, c_void_p, P(c_int), c_int, c_float,
                                          c_int, c_void_p]
        lib.lb_conv_c8_fwd.restype = c_int
        lib.lb_conv_c8_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, P(c_int), P(c_ll),
                                       P(c_ll), c_int, c_int, c_int, c_float, c_void_p]
        lib.lb_planar_to_pixels.restype = c_int
        lib.lb_planar_to_pixels.argtypes = [c_void_p, c_void_p, c_int, c_int, c_ll, c_ll, c_int, c_void_p]
        lib.lb_conv_c8_fwd_pool.restype = c_int
        lib.lb_conv_c8_fwd_pool.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, P(c_int),
                                            P(c_ll), P(c_ll), c_int, c_int, c_int, c_float, c_void_p]
        lib.lb_conv_c8_wgrad.restype = c_int
        lib.lb_conv_c8_wgrad.argtypes = [c_void_p, c_void_p, c_void_p, P(c_int), P(c_ll), P(c_ll),
                                         c_ll, c_ll, c_ll, c_int, c_int, c_float, c_void_p]
        _configured = True
    return lib


def _native_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in _HALF


class WeightHandle:
    """What a native op needs from a weight: the fp32 master tensor (autograd leaf), its
    fp32 gradient buffer, and cached 16-bit / repacked copies valid for one optimizer step."""

    def __init__(self, master: torch.Tensor, grad: Optional[torch.Tensor] = None,
                 compute16: Optional[torch.Tensor] = None):
        self.master = master
        self.grad = grad
        self.compute16 = compute16      # kept in sync by the fused optimizer when present
        self.version = 0
        self._cache = {}

    def bump(self):
        self.version += 1
        self._cache.clear()

    def cast(self, dtype: torch.dtype) -> torch.Tensor:
        if dtype == torch.float32:
            return self.master.detach()
        if self.compute16 is not None and self.compute16.dtype == dtype:
            return self.compute16
        key = ("cast", dtype)
        if key not in self._cache:
            self._cache[key] = self.master.detach().to(dtype)
        return self._cache[key]

    def packed(self, kind: str, dtype: torch.dtype, fn: Callable[[], torch.Tensor]) -> torch.Tensor:
        key = (kind, dtype)
        if key not in self._cache:
            self._cache[key] = fn()
        return self._cache[key]

    def add_grad(self, g: torch.Tensor):
        if self.grad is None:
            return
        self.grad.add_(g.reshape(self.grad.shape).to(self.grad.dtype))

    def mark_ready(self):
        """One user's backward has written its contribution to ``grad``.  When all users of
        this step have, ``on_grad_ready`` (set by a data-parallel context) starts reducing the
        gradient while the rest of backward still runs."""
        cb = getattr(self, "on_grad_ready", None)
        if cb is None:
            return
        self.pending_uses = getattr(self, "pending_uses", 1) - 1
        if self.pending_uses == 0:
            cb()


def column_sums(x2d: torch.Tensor) -> torch.Tensor:
    """fp32 sum over rows of a [rows, C] 16-bit CUDA tensor (native when C % 8 == 0)."""
    rows, C = x2d.shape
    if _native_ok(x2d) and C % 8 == 0 and x2d.is_contiguous() and rows > 0:
        reps = _bn_replicas(rows)
        sums = torch.zeros(reps, 2 * C, dtype=torch.float32, device=x2d.device)
        rc = _lib().lb_bn_partial_sums(x2d.data_ptr(), sums.data_ptr(), rows, C, 1,
                                       native.dtype_code(x2d.dtype), reps, native.stream_ptr())
        native.check(rc, "lb_bn_partial_sums")
        native.count_launch()
        return (sums.sum(0) if reps > 1 else sums[0])[:C]
    return x2d.float().sum(0)


def _bn_replicas(rows: int) -> int:
    """Copies of the partial-sum buffer that the reduction kernels spread their atomics over
    (the caller adds them up): the L2 serialises atomics on one cache line."""
    return 16 if rows >= 8192 else 1


def _act_grad_from_output(y: torch.Tensor, dy: torch.Tensor, act: int, p: float) -> torch.Tensor:
    """dy * act'(.) for activations whose derivative is a function of the output sign."""
    if act == native.ACT_NONE:
        return dy
    if dy.stride() != y.stride():
        dy = torch.empty_like(y).copy_(dy)
    return unary_raw(UNARY_CODE[_ACT_UNARY[act]], y, dy, p, 0.0, 1)


# --------------------------------------------------------------------------- linear
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_leaf, b_leaf, wh: WeightHandle, bh: Optional[WeightHandle], act, act_p):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        w16 = wh.cast(x.dtype)
        bias = bh.master.detach() if bh is not None else None
        y = gemm(x2, w16, trans_b=True, bias=bias, act=act, act_param=act_p)
        ctx.save_for_backward(x2, y if act != native.ACT_NONE else None)
        ctx.meta = (wh, bh, act, act_p, x.shape)
        return y.reshape(*x.shape[:-1], w16.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, y = ctx.saved_tensors
        wh, bh, act, act_p, xshape = ctx.meta
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dy2 = _act_grad_from_output(y, dy2, act, act_p) if y is not None else dy2
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, wh.cast(dy2.dtype)).reshape(xshape)
        if wh.grad is not None:
            _weight_grad(dy2, x2, wh.grad.view(wh.master.shape))
            wh.mark_ready()     # data-parallel runs start reducing this gradient right away
        if bh is not None and bh.grad is not None:
            bh.grad.add_(column_sums(dy2))
            bh.mark_ready()
        return dx, None, None, None, None, None, None


def _pack_both(wh: WeightHandle, dtype: torch.dtype, Kout, Cin, Kp, Cp, ksize) -> None:
    """Fill the handle's cache with the forward and the data-gradient filter layouts in one
    launch (they are valid until the optimizer changes the weights)."""
    if ("fwd", dtype) in wh._cache or not wh.master.is_cuda or wh.master.dtype != torch.float32:
        return
    m = wh.master.detach()
    if not m.is_contiguous():
        return
    taps = 1
    for k in ksize:
        taps *= int(k)
    fwd = torch.empty((taps, Kp, Cp), dtype=dtype, device=m.device)
    dgrad = torch.empty((taps, Cp, Kp), dtype=dtype, device=m.device)
    rc = _lib().lb_pack_filter(m.data_ptr(), fwd.data_ptr(), dgrad.data_ptr(), Kout, Cin, taps, Kp, Cp,
                               native.dtype_code(dtype), native.stream_ptr())
    native.check(rc, "lb_pack_filter")
    native.count_launch()
    wh._cache[("fwd", dtype)] = fwd
    wh._cache[("dgrad", dtype)] = dgrad


def _weight_grad(dy2: torch.Tensor, x2: torch.Tensor, grad: torch.Tensor) -> None:
    """grad[out, in] += dy2^T x2.  Mini-batches of at most 16 rows make this a rank-K update
    bound by the fp32 read-modify-write of ``grad``; a plain kernel does it at memory speed,
    everything else goes to the tensor-core GEMM."""
    K = dy2.shape[0]
    if (K in (1, 2, 4, 8, 16) and grad.dtype == torch.float32 and grad.is_contiguous()
            and x2.shape[1] % 4 == 0 and dy2.dtype == x2.dtype and _native_ok(x2)):
        rc = _lib().lb_outer_accum(dy2.data_ptr(), x2.data_ptr(), grad.data_ptr(), K, dy2.shape[1],
                                   x2.shape[1], 1.0, 1.0, native.dtype_code(x2.dtype),
                                   native.stream_ptr())
        if rc != -2:
            native.check(rc, "lb_outer_accum")
            native.count_launch()
            return
    gemm(dy2, x2, trans_a=True, out=grad, beta=1.0)


def linear(x, wh: WeightHandle, bh: Optional[WeightHandle] = None, act: int = native.ACT_NONE,
           act_param: float = 0.0):
    """y = act(x @ W^T + b) over the last dimension; W is [out, in]."""
    if _native_ok(x) and act in (native.ACT_NONE, native.ACT_RELU, native.ACT_LEAKY):
        return _Linear.apply(x, wh.master, bh.master if bh is not None else None, wh, bh, act,
                             float(act_param))
    w = wh.master if wh.master.dtype == x.dtype else wh.master.to(x.dtype)
    b = None if bh is None else (bh.master if bh.master.dtype == x.dtype else bh.master.to(x.dtype))
    y = F.linear(x, w, b)
    from .gemm import _ACT_FN
    return _ACT_FN[act](y, act_param)


# --------------------------------------------------------------------------- convolution
def _sample_dense(t: torch.Tensor) -> bool:
    """NDHWC tensor whose samples are dense (only the sample stride may leave a gap)."""
    N, D, H, W, C = t.shape
    return (t.stride(4) == 1 and t.stride(3) == C and t.stride(2) == W * C
            and t.stride(1) == H * W * C and t.stride(0) >= D * H * W * C)


def _cl_view(x: torch.Tensor) -> torch.Tensor:
    """[N, C, (D,) H, W] logical tensor -> channels-last NDHWC view (copying if needed)."""
    if x.dim() == 4:
        x = x.contiguous(memory_format=torch.channels_last)
        return x.permute(0, 2, 3, 1).unsqueeze(1)
    if x.dim() == 3:
        x = x.unsqueeze(2)  # N, C, 1, W
        x = x.contiguous(memory_format=torch.channels_last)
        return x.permute(0, 2, 3, 1).unsqueeze(1)
    v = x.permute(0, 2, 3, 4, 1)
    if _sample_dense(v):      # dense samples, possibly with a gap between them (halo planes)
        return v
    x = x.contiguous(memory_format=torch.channels_last_3d)
    return x.permute(0, 2, 3, 4, 1)


def _from_cl(y: torch.Tensor, ndim: int) -> torch.Tensor:
    """NDHWC tensor -> logical [N, C, ...] view with channels-last strides."""
    if ndim == 5:
        return y.permute(0, 4, 1, 2, 3)
    if ndim == 4:
        return y.squeeze(1).permute(0, 3, 1, 2)
    return y.squeeze(1).squeeze(1).permute(0, 2, 1)


def _pad_channels(x_cl: torch.Tensor, mult: int = 8) -> torch.Tensor:
    C = x_cl.shape[-1]
    if C % mult == 0:
        return x_cl
    return F.pad(x_cl, (0, mult - C % mult))


def _upsample_zero(dy_cl: torch.Tensor, stride, out_dims) -> torch.Tensor:
    """Insert zeros between the elements of dy (data gradient of a strided convolution)."""
    N, Do, Ho, Wo, K = dy_cl.shape
    sd, sh, sw = stride
    up = torch.zeros((N, (Do - 1) * sd + 1, (Ho - 1) * sh + 1, (Wo - 1) * sw + 1, K),
                     dtype=dy_cl.dtype, device=dy_cl.device)
    up[:, ::sd, ::sh, ::sw, :] = dy_cl
    return up


class _Conv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_leaf, b_leaf, wh, bh, ksize, pad, stride, dil, act, act_p, skip_act_grad):
        ndim = x.dim()
        x_cl = _pad_channels(_cl_view(x))
        Kout, Cin = wh.master.shape[0], wh.master.shape[1]
        Kp = (Kout + 7) // 8 * 8
        Cp = x_cl.shape[-1]

        def pack_fwd():
            w = wh.master.detach().reshape(Kout, Cin, -1)
            if Kp != Kout or Cp != Cin:
                w = F.pad(w, (0, 0, 0, Cp - Cin, 0, Kp - Kout))
            return pack_filter(w.reshape(Kp, Cp, *ksize), x.dtype)

        _pack_both(wh, x.dtype, Kout, Cin, Kp, Cp, ksize)
        wt = wh.packed("fwd", x.dtype, pack_fwd)
        bias = None
        if bh is not None:
            bias = bh.master.detach()
            if Kp != Kout:
                bias = F.pad(bias, (0, Kp - Kout))
        y = conv_fwd(x_cl, wt, ksize, pad=pad, stride=stride, dilation=dil, bias=bias, act=act,
                     act_param=act_p)
        ctx.save_for_backward(x_cl, y if (act != native.ACT_NONE and not skip_act_grad) else None)
        ctx.meta = (wh, bh, ksize, pad, stride, dil, act, act_p, ndim, Kout, Cin, Kp, Cp)
        out = y[..., :Kout] if Kp != Kout else y
        return _from_cl(out, ndim)

    @staticmethod
    def backward(ctx, dy):
        x_cl, y = ctx.saved_tensors
        wh, bh, ksize, pad, stride, dil, act, act_p, ndim, Kout, Cin, Kp, Cp = ctx.meta
        dy_cl = _cl_view(dy)
        if Kp != Kout:
            dy_cl = _pad_channels(dy_cl)
        if not dy_cl.is_contiguous():
            dy_cl = dy_cl.contiguous()
        if y is not None:
            dy_cl = _act_grad_from_output(y, dy_cl, act, act_p)
        N, D, H, W, _ = x_cl.shape
        dx = None
        if ctx.needs_input_grad[0]:
            def pack_bwd():
                w = wh.master.detach().reshape(Kout, Cin, -1)
                if Kp != Kout or Cp != Cin:
                    w = F.pad(w, (0, 0, 0, Cp - Cin, 0, Kp - Kout))
                return pack_filter(w.reshape(Kp, Cp, *ksize), dy.dtype, for_dgrad=True)

            wt = wh.packed("dgrad", dy.dtype, pack_bwd)
            src = dy_cl if stride == (1, 1, 1) else _upsample_zero(dy_cl, stride, (D, H, W))
            bpad = tuple(d * (k - 1) - p for d, k, p in zip(dil, ksize, pad))
            dx_cl = conv_fwd(src, wt, ksize, pad=bpad, stride=1, dilation=dil, out_dims=(D, H, W))
            if Cp != Cin:
                dx_cl = dx_cl[..., :Cin]
            dx = _from_cl(dx_cl, ndim)
        if wh.grad is not None:
            if Kp == Kout and Cp == Cin:
                conv_wgrad(x_cl, dy_cl, ksize, pad=pad, stride=stride, dilation=dil,
                           out=wh.grad.view(Kout, Cin, *ksize))
            else:
                tmp = conv_wgrad(x_cl, dy_cl, ksize, pad=pad, stride=stride, dilation=dil)
                wh.grad.add_(tmp[:Kout, :Cin].reshape(wh.grad.shape))
            wh.mark_ready()
        if bh is not None and bh.grad is not None:
            bh.grad.add_(column_sums(dy_cl.reshape(-1, dy_cl.shape[-1]))[:Kout])
            bh.mark_ready()
        return (dx,) + (None,) * 11


def _first_layer_pixels(x, cr: int):
    """The [N, D, H, W, cr] pixel layout the first-layer kernels read (cr = 4 or 8 channels
    per pixel, zero beyond the tensor's own).  A planar [N, C, D, H, W] tensor is
    interleaved by one vectorised kernel (csrc/layout.cu)."""
    N, C = x.shape[0], x.shape[1]
    sp = tuple(x.shape[2:])
    S = 1
    for v in sp:
        S *= v
    if (x.dim() == 5 and x.dtype in (torch.float16, torch.bfloat16) and S % 8 == 0 and x.stride(1) == S
            and x[0].is_contiguous() and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0):
        y = torch.empty((N,) + sp + (cr,), dtype=x.dtype, device=x.device)
        native.check(_lib().lb_planar_to_pixels(x.data_ptr(), y.data_ptr(), N, C, S, x.stride(0), cr,
                                                native.stream_ptr()), "lb_planar_to_pixels")
        native.count_launch()
        return y
    x_in = _cl_view(x)
    x_cl = F.pad(x_in, (0, cr - C)) if C != cr else x_in
    return x_cl if x_cl.is_contiguous() else x_cl.contiguous()


class _ConvC8(torch.autograd.Function):
    """First-layer convolution: at most 8 input channels, kernel (kd, kh, 3), stride 1, no
    dilation, "same" padding along W.  Forward and filter gradient use the dedicated
    16-bytes-per-pixel tcgen05 kernels (csrc/conv_c8_tc.cu); the data gradient, when one is
    needed at all, goes through the generic path."""

    @staticmethod
    def forward(ctx, x, w_leaf, b_leaf, wh, bh, ksize, pad, act, act_p, skip_act_grad):
        ndim = x.dim()
        Cin = x.shape[1]
        # pixels are 8 bytes (<= 4 channels, W a multiple of 16) or 16 bytes; an input that
        # already has 4 or 8 channels in that layout is used as it is
        cr = 4 if (Cin <= 4 and x.shape[-1] % 16 == 0) else 8
        x_cl = _first_layer_pixels(x, cr)
        x_bwd = x_cl
        Kout = wh.master.shape[0]
        kd, kh, _ = ksize

        def pack():
            # K index = tap * cr + channel, padded to a multiple of 16; rows padded to 32
            w = wh.master.detach().reshape(Kout, Cin, kd * kh * 3).permute(0, 2, 1)   # K, tap, C
            w = F.pad(w, (0, cr - Cin)).reshape(Kout, -1)
            kpad = (w.shape[1] + 15) // 16 * 16
            w = F.pad(w, (0, kpad - w.shape[1], 0, 32 - Kout))
            # [K chunk][32 rows][8 elements]
            return w.reshape(32, kpad // 8, 8).permute(1, 0, 2).contiguous().to(x.dtype)

        wt = wh.packed("c8fwd", x.dtype, pack)
        N, D, H, W, _ = x_cl.shape
        Do = D + 2 * pad[0] - kd + 1
        y = torch.empty((N, Do, H, W, Kout), dtype=x.dtype, device=x.device)
        geom = (c_int * 10)(N, D, H, W, Kout, kd, kh, pad[0], pad[1], Do)
        xs = (c_ll * 4)(x_cl.stride(0), x_cl.stride(1), x_cl.stride(2), x_cl.stride(3))
        ys = (c_ll * 4)(y.stride(0), y.stride(1), y.stride(2), y.stride(3))
        bias = bh.master.detach() if bh is not None else None
        native.check(_lib().lb_conv_c8_fwd(x_cl.data_ptr(), wt.data_ptr(), y.data_ptr(),
                                           native.ptr(bias), geom, xs, ys,
                                           native.dtype_code(x.dtype), native.dtype_code(x.dtype),
                                           int(act), float(act_p), native.stream_ptr()),
                     "lb_conv_c8_fwd")
        native.count_launch()
        ctx.save_for_backward(x_bwd, y if (act != native.ACT_NONE and not skip_act_grad) else None)
        xs = (c_ll * 4)(x_bwd.stride(0), x_bwd.stride(1), x_bwd.stride(2), x_bwd.stride(3))
        ctx.meta = (wh, bh, ksize, pad, act, act_p, ndim, Kout, Cin, geom, xs)
        return _from_cl(y, ndim)

    @staticmethod
    def backward(ctx, dy):
        x_cl, y = ctx.saved_tensors
        wh, bh, ksize, pad, act, act_p, ndim, Kout, Cin, geom, xs = ctx.meta
        dy_cl = _cl_view(dy)
        if not dy_cl.is_contiguous():
            dy_cl = dy_cl.contiguous()
        if y is not None:
            dy_cl = _act_grad_from_output(y, dy_cl, act, act_p)
        dx = None
        if ctx.needs_input_grad[0]:
            def pack_bwd():
                w = F.pad(wh.master.detach().reshape(Kout, Cin, -1), (0, 0, 0, 8 - Cin))
                return pack_filter(w.reshape(Kout, 8, *ksize), dy.dtype, for_dgrad=True)
            wt = wh.packed("dgrad", dy.dtype, pack_bwd)
            bpad = tuple(k - 1 - p for k, p in zip(ksize, pad))
            N, D, H, W, _ = x_cl.shape
            dx_cl = conv_fwd(dy_cl, wt, ksize, pad=bpad, stride=1, out_dims=(D, H, W))
            dx = _from_cl(dx_cl[..., :Cin], ndim)
        if wh.grad is not None:
            taps = ksize[0] * ksize[1] * 3
            ys = (c_ll * 4)(dy_cl.stride(0), dy_cl.stride(1), dy_cl.stride(2), dy_cl.stride(3))
            native.check(_lib().lb_conv_c8_wgrad(x_cl.data_ptr(), dy_cl.data_ptr(),
                                                 wh.grad.data_ptr(), geom, xs, ys, 1, Cin * taps,
                                                 taps, Cin, native.dtype_code(x_cl.dtype), 1.0,
                                                 native.stream_ptr()), "lb_conv_c8_wgrad")
            native.count_launch()
            wh.mark_ready()
        if bh is not None and bh.grad is not None:
            bh.grad.add_(column_sums(dy_cl.reshape(-1, Kout)))
            bh.mark_ready()
        return (dx,) + (None,) * 9


class PoolFusion:
    """A request to run the 2 x 2 x 2 max pooling that follows a first-layer convolution (and
    its folded activation) inside the convolution kernel.  ``out_alloc`` as for ``_Pool``;
    ``done`` tells the caller whether the returned tensor is already pooled."""

    def __init__(self, out_alloc=None):
        self.out_alloc = out_alloc
        self.done = False


class _ConvC8Pool(torch.autograd.Function):
    """First-layer convolution + activation + 2 x 2 x 2 max pooling (stride 2) in one kernel
    (csrc/conv_c8_tc.cu, conv_c8_fwd_pool_kernel): the full-resolution activation is never
    written.  Backward expands the pooled gradient with the recorded arg-max bytes (the
    separate pooling layer's kernel) and feeds the first-layer filter-gradient kernel."""

    @staticmethod
    def forward(ctx, x, w_leaf, b_leaf, wh, bh, pad, act, act_p, out_alloc):
        ndim = x.dim()
        Cin = x.shape[1]
        x_cl = _first_layer_pixels(x, 4)
        Kout = wh.master.shape[0]

        def pack():
            w = wh.master.detach().reshape(Kout, Cin, 27).permute(0, 2, 1)
            w = F.pad(w, (0, 4 - Cin)).reshape(Kout, -1)
            kpad = (w.shape[1] + 15) // 16 * 16
            w = F.pad(w, (0, kpad - w.shape[1], 0, 32 - Kout))
            return w.reshape(32, kpad // 8, 8).permute(1, 0, 2).contiguous().to(x.dtype)

        wt = wh.packed("c8fwd", x.dtype, pack)
        N, D, H, W, _ = x_cl.shape
        Do = D + 2 * pad[0] - 2
        shape = (N, Do // 2, H // 2, W // 2, Kout)
        y = out_alloc(shape, x.dtype) if out_alloc is not None else None
        if y is None or not _sample_dense(y):
            y = torch.empty(shape, dtype=x.dtype, device=x.device)
        idx = torch.empty(shape, dtype=torch.uint8, device=x.device)
        geom = (c_int * 10)(N, D, H, W, Kout, 3, 3, pad[0], pad[1], Do)
        xs = (c_ll * 4)(x_cl.stride(0), x_cl.stride(1), x_cl.stride(2), x_cl.stride(3))
        ys = (c_ll * 4)(y.stride(0), y.stride(1), y.stride(2), y.stride(3))
        bias = bh.master.detach() if bh is not None else None
        native.check(_lib().lb_conv_c8_fwd_pool(x_cl.data_ptr(), wt.data_ptr(), y.data_ptr(),
                                                idx.data_ptr(), native.ptr(bias), geom, xs, ys,
                                                native.dtype_code(x.dtype), native.dtype_code(x.dtype),
                                                int(act), float(act_p), native.stream_ptr()),
                     "lb_conv_c8_fwd_pool")
        native.count_launch()
        ctx.save_for_backward(x_cl, idx)
        ctx.meta = (wh, bh, pad, act, act_p, ndim, Kout, Cin, geom, xs, (N, Do, H, W, Kout))
        return _from_cl(y, ndim)

    @staticmethod
    def backward(ctx, dy):
        x_cl, idx = ctx.saved_tensors
        wh, bh, pad, act, act_p, ndim, Kout, Cin, geom, xs, full = ctx.meta
        dyp = _cl_view(dy)
        if not dyp.is_contiguous():
            dyp = dyp.contiguous()
        N, Do, H, W, _ = full
        # gradient of pooling and activation at full resolution
        dy_cl = torch.empty(full, dtype=dy.dtype, device=dy.device)
        tg = (c_int * 8)(N, Do, H, W, Kout, 2, 2, 2)
        native.check(_lib().lb_pool_bwd_tiled_idx(idx.data_ptr(), dyp.data_ptr(), dy_cl.data_ptr(), tg,
                                                  int(act), float(act_p), dy_cl.stride(0),
                                                  native.dtype_code(dy.dtype), native.stream_ptr()),
                     "lb_pool_bwd_tiled_idx")
        native.count_launch()
        dx = None
        if ctx.needs_input_grad[0]:
            ksize = (3, 3, 3)

            def pack_bwd():
                w = F.pad(wh.master.detach().reshape(Kout, Cin, -1), (0, 0, 0, 8 - Cin))
                return pack_filter(w.reshape(Kout, 8, *ksize), dy.dtype, for_dgrad=True)
            wt = wh.packed("dgrad", dy.dtype, pack_bwd)
            bpad = tuple(k - 1 - p for k, p in zip(ksize, pad))
            D = x_cl.shape[1]
            dx_cl = conv_fwd(dy_cl, wt, ksize, pad=bpad, stride=1, out_dims=(D, H, W))
            dx = _from_cl(dx_cl[..., :Cin], ndim)
        if wh.grad is not None:
            ys = (c_ll * 4)(dy_cl.stride(0), dy_cl.stride(1), dy_cl.stride(2), dy_cl.stride(3))
            native.check(_lib().lb_conv_c8_wgrad(x_cl.data_ptr(), dy_cl.data_ptr(),
                                                 wh.grad.data_ptr(), geom, xs, ys, 1, Cin * 27,
                                                 27, Cin, native.dtype_code(x_cl.dtype), 1.0,
                                                 native.stream_ptr()), "lb_conv_c8_wgrad")
            native.count_launch()
            wh.mark_ready()
        if bh is not None and bh.grad is not None:
            bh.grad.add_(column_sums(dy_cl.reshape(-1, Kout)))
            bh.mark_ready()
        return (dx,) + (None,) * 8


def _c8_pool_ok(x, Cin, Kout, k3, p3) -> bool:
    """Shapes the fused convolution + pooling kernel covers: 4-channel pixels, 3 x 3 x 3
    filter, even output extents."""
    if os.environ.get("LBANN_DISABLE_CONV_POOL_FUSION", "") not in ("", "0"):
        return False
    D, H, W = x.shape[2:]
    Do = D + 2 * p3[0] - 2
    return (Cin <= 4 and tuple(k3) == (3, 3, 3) and p3[1] == 1 and W % 16 == 0 and H % 2 == 0
            and Do % 2 == 0 and Do > 0 and x.dtype in (torch.float16, torch.bfloat16))


def convolution(x, wh: WeightHandle, bh: Optional[WeightHandle], ksize, pad, stride, dilation,
                groups: int = 1, act: int = native.ACT_NONE, act_param: float = 0.0,
                skip_act_grad: bool = False, fuse_pool: Optional["PoolFusion"] = None):
    """N-d convolution on a logical [N, C, spatial...] tensor; kernel Kout x C/groups x k...
    ``skip_act_grad``: the consumer applies the fused activation's gradient itself.
    ``fuse_pool``: the consumer is a 2 x 2 x 2 max pooling with stride 2; where the
    first-layer kernel covers the shape the pooled tensor is returned and
    ``fuse_pool.done`` is set."""
    nsp = x.dim() - 2
    if _native_ok(x) and groups == 1 and act in (native.ACT_NONE, native.ACT_RELU, native.ACT_LEAKY):
        k3, p3, s3, d3 = norm3(ksize, 1), norm3(pad, 0), norm3(stride, 1), norm3(dilation, 1)
        Kout, Cin = wh.master.shape[0], wh.master.shape[1]
        if (Cin <= 8 and k3[2] == 3 and p3[2] == 1 and s3 == (1, 1, 1) and d3 == (1, 1, 1)
                and Kout <= 32 and Kout % 8 == 0 and k3[0] * k3[1] * 32 <= 512
                and x.shape[-1] % 8 == 0
                and p3[0] in (0, (k3[0] - 1) // 2) and k3[0] % 2 == 1 and 2 * p3[1] == k3[1] - 1
                and wh.grad is not None and wh.grad.is_contiguous()):
            if fuse_pool is not None and x.dim() == 5 and _c8_pool_ok(x, Cin, Kout, k3, p3):
                fuse_pool.done = True
                return _ConvC8Pool.apply(x, wh.master, bh.master if bh is not None else None, wh, bh,
                                         p3, act, float(act_param), fuse_pool.out_alloc)
            return _ConvC8.apply(x, wh.master, bh.master if bh is not None else None, wh, bh, k3,
                                 p3, act, float(act_param), bool(skip_act_grad))
        return _Conv.apply(x, wh.master, bh.master if bh is not None else None, wh, bh, k3, p3, s3,
                           d3, act, float(act_param), bool(skip_act_grad))
    w = wh.master if wh.master.dtype == x.dtype else wh.master.to(x.dtype)
    b = None if bh is None else (bh.master if bh.master.dtype == x.dtype else bh.master.to(x.dtype))
    fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nsp]
    y = fn(x, w, b, tuple(stride), tuple(pad), tuple(dilation), groups)
    from .gemm import _ACT_FN
    return _ACT_FN[act](y, act_param)


def deconvolution(x, wh: WeightHandle, bh, ksize, pad, stride, dilation, output_padding,
                  groups: int = 1):
    """Transposed convolution; kernel stored Cin x Cout/groups x k... (PyTorch convention,
    which is also the reference's: src/layers/learning/deconvolution.cpp)."""
    nsp = x.dim() - 2
    w = wh.master if wh.master.dtype == x.dtype else wh.master.to(x.dtype)
    b = None if bh is None else (bh.master if bh.master.dtype == x.dtype else bh.master.to(x.dtype))
    ks, st = tuple(ksize), tuple(stride)
    if (_native_ok(x) and groups == 1 and ks == st and all(p == 0 for p in pad)
            and all(d == 1 for d in dilation) and all(o == 0 for o in output_padding)):
        # Non-overlapping up-convolution (U-Net k2 s2): a per-pixel GEMM followed by a
        # depth-to-space rearrangement.  Both run natively (GEMM + autograd of views).
        return _deconv_as_gemm(x, wh, bh, ks)
    fn = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[nsp]
    return fn(x, w, b, st, tuple(pad), tuple(output_padding), groups, tuple(dilation))


def _deconv_as_gemm(x, wh, bh, ks):
    ndim = x.dim()
    x_cl = _cl_view(x)                         # N, D, H, W, Cin
    N, D, H, W, Cin = x_cl.shape
    Cout = wh.master.shape[1]
    k3 = norm3(ks, 1)
    taps = k3[0] * k3[1] * k3[2]
    w2d = wh.packed("deconv2d", x.dtype, lambda: wh.master.detach().reshape(Cin, Cout * taps)
                    .t().contiguous().to(x.dtype))     # [Cout*taps, Cin]
    y = _DeconvGemm.apply(x_cl.reshape(-1, Cin), wh.master, wh, w2d)   # [pix, Cout*taps]
    y = y.reshape(N, D, H, W, Cout, k3[0], k3[1], k3[2])
    y = y.permute(0, 1, 5, 2, 6, 3, 7, 4).reshape(N, D * k3[0], H * k3[1], W * k3[2], Cout)
    if bh is not None:
        y = y + bh.master.to(y.dtype)
    return _from_cl(y, ndim)


class _DeconvGemm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, w_leaf, wh, w2d):
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w2d)
        ctx.wh = wh
        return gemm(x2, w2d, trans_b=True)

    @staticmethod
    def backward(ctx, dy):
        x2, w2d = ctx.saved_tensors
        wh = ctx.wh
        if not dy.is_contiguous():
            dy = dy.contiguous()
        dx = gemm(dy, w2d) if ctx.needs_input_grad[0] else None
        if wh.grad is not None:
            # grad of W[Cin, Cout*taps] = x^T dy
            gemm(x2, dy, trans_a=True, out=wh.grad.view(x2.shape[1], dy.shape[1]), beta=1.0)
            wh.mark_ready()
        return dx, None, None, None


# --------------------------------------------------------------------------- pooling
_POOL_MODE = {"max": 0, "average": 1, "average_no_pad": 2}


class _Pool(torch.autograd.Function):
    """``out_alloc`` / ``dx_alloc``: optional callables (shape, dtype) -> NDHWC tensor (or
    None) that place the output / the input gradient, e.g. inside a consumer's buffer with
    halo planes; samples must be dense, the sample stride may leave a gap."""

    @staticmethod
    def forward(ctx, x, ksize, pad, stride, mode, bwd_act, bwd_act_p, out_alloc=None, dx_alloc=None):
        ndim = x.dim()
        x_cl = _cl_view(x)
        ctx.bwd_act = (bwd_act, bwd_act_p)
        ctx.win = (ksize, pad, stride, mode)
        ctx.dx_alloc = dx_alloc
        N, D, H, W, C = x_cl.shape
        Do, Ho, Wo = (out_size(D, ksize[0], pad[0], stride[0], 1),
                      out_size(H, ksize[1], pad[1], stride[1], 1),
                      out_size(W, ksize[2], pad[2], stride[2], 1))
        y = out_alloc((N, Do, Ho, Wo, C), x.dtype) if out_alloc is not None else None
        if y is None or not _sample_dense(y):
            y = torch.empty((N, Do, Ho, Wo, C), dtype=x.dtype, device=x.device)
        geom = (c_int * 18)(N, D, H, W, C, Do, Ho, Wo, *ksize, *pad, *stride, mode)
        xs = (c_ll * 4)(x_cl.stride(0), x_cl.stride(1), x_cl.stride(2), x_cl.stride(3))
        # non-overlapping max pooling: record where the maxima sit (a byte per output), so
        # that backward reads dy and those bytes instead of scanning x again
        tiled = (mode == 0 and ksize == stride and pad == (0, 0, 0) and D % ksize[0] == 0
                 and H % ksize[1] == 0 and W % ksize[2] == 0 and ksize[0] * ksize[1] * ksize[2] <= 128)
        idx = None
        if tiled and x.requires_grad and os.environ.get("LBANN_POOL_RESCAN", "") in ("", "0"):
            idx = torch.empty((N, Do, Ho, Wo, C), dtype=torch.uint8, device=x.device)
        rc = -2
        if tiled:       # the window-per-thread kernel (2x2x2 and 2x2 windows); -2: not one of those
            tg = (c_int * 8)(N, D, H, W, C, *ksize)
            rc = _lib().lb_pool_fwd_tiled(x_cl.data_ptr(), y.data_ptr(), native.ptr(idx), tg, xs, y.stride(0),
                                          native.dtype_code(x.dtype), native.stream_ptr())
        if rc == -2:
            rc = _lib().lb_pool_fwd_idx(x_cl.data_ptr(), y.data_ptr(), native.ptr(idx), geom, xs, y.stride(0),
                                        native.dtype_code(x.dtype), native.stream_ptr())
        native.check(rc, "lb_pool_fwd")
        native.count_launch()
        if idx is not None:
            ctx.save_for_backward(idx)
            ctx.x_shape = tuple(x_cl.shape)
        else:
            ctx.save_for_backward(x_cl)
            ctx.x_shape = None
        ctx.x_dtype = x.dtype
        ctx.meta = (geom, ndim)
        return _from_cl(y, ndim)

    @staticmethod
    def backward(ctx, dy):
        geom, ndim = ctx.meta
        dy_cl = _cl_view(dy)
        if not dy_cl.is_contiguous():
            dy_cl = dy_cl.contiguous()
        ksize, pad, stride, mode = ctx.win
        nothing = (None,) * 8
        if ctx.x_shape is not None:
            (idx,) = ctx.saved_tensors
            N, D, H, W, C = ctx.x_shape
            dx = ctx.dx_alloc(ctx.x_shape, ctx.x_dtype) if ctx.dx_alloc is not None else None
            if dx is None or not _sample_dense(dx):
                dx = torch.empty(ctx.x_shape, dtype=ctx.x_dtype, device=dy.device)
            tg = (c_int * 8)(N, D, H, W, C, *ksize)
            rc = _lib().lb_pool_bwd_tiled_idx(idx.data_ptr(), dy_cl.data_ptr(), dx.data_ptr(), tg,
                                              int(ctx.bwd_act[0]), float(ctx.bwd_act[1]), dx.stride(0),
                                              native.dtype_code(ctx.x_dtype), native.stream_ptr())
            native.check(rc, "lb_pool_bwd_tiled_idx")
            native.count_launch()
            return (_from_cl(dx, ndim),) + nothing
        (x_cl,) = ctx.saved_tensors
        N, D, H, W, C = x_cl.shape
        tiled = (mode == 0 and ksize == stride and pad == (0, 0, 0) and x_cl.is_contiguous()
                 and D % ksize[0] == 0 and H % ksize[1] == 0 and W % ksize[2] == 0)
        if tiled:
            dx = ctx.dx_alloc(tuple(x_cl.shape), x_cl.dtype) if ctx.dx_alloc is not None else None
            if dx is None or not _sample_dense(dx):
                dx = torch.empty(x_cl.shape, dtype=x_cl.dtype, device=x_cl.device)
            tg = (c_int * 8)(N, D, H, W, C, *ksize)
            rc = _lib().lb_pool_bwd_tiled_strided(x_cl.data_ptr(), dy_cl.data_ptr(), dx.data_ptr(), tg,
                                                  int(ctx.bwd_act[0]), float(ctx.bwd_act[1]),
                                                  dx.stride(0), native.dtype_code(x_cl.dtype),
                                                  native.stream_ptr())
            native.check(rc, "lb_pool_bwd_tiled_strided")
            native.count_launch()
            return (_from_cl(dx, ndim),) + nothing
        dx = torch.empty(x_cl.shape, dtype=x_cl.dtype, device=x_cl.device)
        xs = (c_ll * 4)(x_cl.stride(0), x_cl.stride(1), x_cl.stride(2), x_cl.stride(3))
        rc = _lib().lb_pool_bwd(x_cl.data_ptr(), dy_cl.data_ptr(), dx.data_ptr(), geom, xs,
                                native.dtype_code(x_cl.dtype), native.stream_ptr())
        native.check(rc, "lb_pool_bwd")
        native.count_launch()
        if ctx.bwd_act[0] != native.ACT_NONE:
            dx = _act_grad_from_output(x_cl, dx, ctx.bwd_act[0], ctx.bwd_act[1])
        return (_from_cl(dx, ndim),) + nothing


def pooling(x, ksize, pad, stride, mode: str, bwd_act: int = native.ACT_NONE,
            bwd_act_param: float = 0.0, out_alloc=None, dx_alloc=None):
    """``bwd_act``: also apply the gradient of that activation (taken from the sign of x) in
    the backward pass - used when the producer fused the activation into its epilogue.
    ``out_alloc`` / ``dx_alloc``: see ``_Pool``."""
    nsp = x.dim() - 2
    if _native_ok(x) and x.shape[1] % 8 == 0:
        return _Pool.apply(x, norm3(ksize, 1), norm3(pad, 0), norm3(stride, 1), _POOL_MODE[mode],
                           int(bwd_act), float(bwd_act_param), out_alloc, dx_alloc)
    if bwd_act != native.ACT_NONE:
        raise RuntimeError("pooling: fused activation gradient needs the native path")
    ks, pd, st = tuple(ksize), tuple(pad), tuple(stride)
    if mode == "max":
        return {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[nsp](x, ks, st, pd)
    fn = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nsp]
    return fn(x, ks, st, pd, count_include_pad=(mode == "average"))


# --------------------------------------------------------------------------- batch norm
class GroupSum:
    """In-place sum of an fp32 tensor over the ranks of a symmetric group, as a callable that
    also names the group: the fused batch-norm kernels then do the reduction themselves."""

    def __init__(self, group, fn):
        self.group, self.fn = group, fn

    def __call__(self, t):
        return self.fn(t)


_bn_workspaces = {}


def _bn_ws(owner, tag, rows, C, device):
    key = (id(owner), tag, rows, C)
    ws = _bn_workspaces.get(key)
    if ws is None:
        ws = torch.zeros(_lib().lb_bn_fused_ws_floats(C), dtype=torch.float32, device=device)
        _bn_workspaces[key] = ws
    return ws


def _bn_fused_peers(reduce_fn):
    """(staging ptrs, pad ptrs, rank, world, slot stride, counters) for the fused kernels, or
    None when the statistics group cannot be served by them."""
    if reduce_fn is None:
        return (None, None, 0, 1, 0, None)
    g = getattr(reduce_fn, "group", None)
    if g is None or not g.native or g.poisoned:
        return None
    return (g.staging._c_ptrs, g.pad._c_ptrs, g.rank, g.world, 4096, g.ctr_ptr)


class _BatchNormFused(torch.autograd.Function):
    """Training-mode batch norm as one cooperative kernel per direction, statistics over the
    ranks of a symmetric group reduced inside the kernel (csrc/bn_fused.cu)."""

    @staticmethod
    def forward(ctx, x, s_leaf, b_leaf, sh, bh, run_mean, run_var, eps, decay, correction,
                reduce_fn, count_scale, act, act_p, peers):
        ndim = x.dim()
        x_cl = _cl_view(x)
        if not x_cl.is_contiguous():
            x_cl = x_cl.contiguous()
        C = x_cl.shape[-1]
        rows = x_cl.numel() // C
        staging, pads, rank, world, stride, ctr = peers
        count = float(rows * count_scale)
        y = torch.empty_like(x_cl)
        stats = torch.empty(2 * C, dtype=torch.float32, device=x.device)
        scale = sh.master.detach() if sh is not None else None
        bias = bh.master.detach() if bh is not None else None
        owner = sh if sh is not None else (bh if bh is not None else run_mean)
        ws = _bn_ws(owner, "fwd", rows, C, x.device)
        rc = _lib().lb_bn_fused_fwd(x_cl.data_ptr(), native.ptr(scale), native.ptr(bias), y.data_ptr(),
                                    stats.data_ptr(), native.ptr(run_mean), native.ptr(run_var),
                                    ws.data_ptr(), rows, C, count, float(correction), float(eps),
                                    float(decay), act, float(act_p), native.dtype_code(x.dtype),
                                    staging, pads, rank, world, stride, ctr, native.stream_ptr())
        native.check(rc, "lb_bn_fused_fwd")
        native.count_launch()
        ctx.save_for_backward(x_cl, stats, y if act else None)
        ctx.meta = (sh, bh, eps, correction, count, act, act_p, ndim, peers, owner)
        return _from_cl(y, ndim)

    @staticmethod
    def backward(ctx, dy):
        x_cl, stats, y = ctx.saved_tensors
        sh, bh, eps, correction, count, act, act_p, ndim, peers, owner = ctx.meta
        dy_cl = _cl_view(dy)
        if not dy_cl.is_contiguous():
            dy_cl = dy_cl.contiguous()
        C = x_cl.shape[-1]
        rows = x_cl.numel() // C
        staging, pads, rank, world, stride, ctr = peers
        scale = sh.master.detach() if sh is not None else None
        dscale = sh.grad.view(-1) if (sh is not None and sh.grad is not None) else None
        dbias = bh.grad.view(-1) if (bh is not None and bh.grad is not None) else None
        dx = torch.empty_like(x_cl)
        ws = _bn_ws(owner, "bwd", rows, C, x_cl.device)
        rc = _lib().lb_bn_fused_bwd(x_cl.data_ptr(), dy_cl.data_ptr(), native.ptr(y), stats.data_ptr(),
                                    native.ptr(scale), dx.data_ptr(), native.ptr(dscale),
                                    native.ptr(dbias), ws.data_ptr(), rows, C, count, float(correction),
                                    float(eps), act, float(act_p), native.dtype_code(x_cl.dtype),
                                    staging, pads, rank, world, stride, ctr, native.stream_ptr())
        native.check(rc, "lb_bn_fused_bwd")
        native.count_launch()
        if dscale is not None:
            sh.mark_ready()
        if dbias is not None:
            bh.mark_ready()
        return (_from_cl(dx, ndim),) + (None,) * 14


class _BatchNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, s_leaf, b_leaf, sh, bh, run_mean, run_var, eps, decay, correction,
                reduce_fn, count_scale, act, act_p):
        ndim = x.dim()
        x_cl = _cl_view(x)
        if not x_cl.is_contiguous():
            x_cl = x_cl.contiguous()
        C = x_cl.shape[-1]
        rows = x_cl.numel() // C
        lib = _lib()
        dt = native.dtype_code(x.dtype)
        reps = _bn_replicas(rows)
        sums = torch.zeros(reps, 2 * C, dtype=torch.float32, device=x.device)
        native.check(lib.lb_bn_partial_sums(x_cl.data_ptr(), sums.data_ptr(), rows, C, 1, dt, reps,
                                            native.stream_ptr()), "lb_bn_partial_sums")
        sums = sums.sum(0) if reps > 1 else sums[0]
        if reduce_fn is not None:
            reduce_fn(sums)
        count = float(rows * count_scale)
        y = torch.empty_like(x_cl)
        stats = torch.empty(2 * C, dtype=torch.float32, device=x.device)
        scale = sh.master.detach() if sh is not None else None
        bias = bh.master.detach() if bh is not None else None
        native.check(lib.lb_bn_finalize_apply(
            x_cl.data_ptr(), sums.data_ptr(), native.ptr(scale), native.ptr(bias), y.data_ptr(),
            stats.data_ptr(), native.ptr(run_mean), native.ptr(run_var), rows, C, 1, count,
            float(correction), float(eps), float(decay), act, float(act_p), dt,
            native.stream_ptr()), "lb_bn_finalize_apply")
        native.count_launch(2)
        ctx.save_for_backward(x_cl, stats, y if act else None)
        ctx.meta = (sh, bh, eps, correction, reduce_fn, count, act, act_p, ndim)
        return _from_cl(y, ndim)

    @staticmethod
    def backward(ctx, dy):
        x_cl, stats, y = ctx.saved_tensors
        sh, bh, eps, correction, reduce_fn, count, act, act_p, ndim = ctx.meta
        dy_cl = _cl_view(dy)
        if not dy_cl.is_contiguous():
            dy_cl = dy_cl.contiguous()
        C = x_cl.shape[-1]
        rows = x_cl.numel() // C
        lib = _lib()
        dt = native.dtype_code(x_cl.dtype)
        reps = _bn_replicas(rows)
        bsums = torch.zeros(reps, 4 * C, dtype=torch.float32, device=x_cl.device)
        scale = sh.master.detach() if sh is not None else None
        native.check(lib.lb_bn_bwd_sums(x_cl.data_ptr(), dy_cl.data_ptr(), native.ptr(y),
                                        stats.data_ptr(), native.ptr(scale), bsums.data_ptr(),
                                        rows, C, 1, float(eps), act, float(act_p), dt, reps,
                                        native.stream_ptr()), "lb_bn_bwd_sums")
        bsums = bsums.sum(0) if reps > 1 else bsums[0]
        # parameter gradients use the local partial sums (the optimizer's allreduce sums ranks)
        if sh is not None and sh.grad is not None:
            sh.grad.add_(bsums[:C])
            sh.mark_ready()
        if bh is not None and bh.grad is not None:
            bh.grad.add_(bsums[C:2 * C])
            bh.mark_ready()
        if reduce_fn is not None:
            reduce_fn(bsums[2 * C:])
        dx = torch.empty_like(x_cl)
        native.check(lib.lb_bn_bwd_apply(x_cl.data_ptr(), dy_cl.data_ptr(), native.ptr(y),
                                         stats.data_ptr(), native.ptr(scale), bsums.data_ptr(),
                                         dx.data_ptr(), rows, C, 1, count, float(correction),
                                         float(eps), act, float(act_p), dt, native.stream_ptr()),
                     "lb_bn_bwd_apply")
        native.count_launch(2)
        return (_from_cl(dx, ndim),) + (None,) * 13


def batch_norm(x, sh, bh, run_mean, run_var, training: bool, eps: float, decay: float,
               bessel: bool = True, reduce_fn=None, count_scale: float = 1.0,
               act: int = native.ACT_NONE, act_param: float = 0.0):
    """Batch normalisation over (N, spatial) per channel with the reference's variance
    definition.  ``reduce_fn(t)`` sums an fp32 tensor in place over the statistics group
    (``count_scale`` = number of ranks in it)."""
    C = x.shape[1]
    correction = 1.0 if bessel else 0.0
    if _native_ok(x) and C % 8 == 0:
        if training:
            peers = _bn_fused_peers(reduce_fn) if (2 * C <= 4096 and not os.environ.get(
                "LBANN_BN_SEPARATE_KERNELS")) else None
            if peers is not None:
                return _BatchNormFused.apply(x, sh.master if sh else None, bh.master if bh else None,
                                             sh, bh, run_mean, run_var, eps, decay, correction,
                                             reduce_fn, count_scale, act, float(act_param), peers)
            return _BatchNorm.apply(x, sh.master if sh else None, bh.master if bh else None, sh, bh,
                                    run_mean, run_var, eps, decay, correction, reduce_fn,
                                    count_scale, act, float(act_param))
        x_cl = _cl_view(x)
        if not x_cl.is_contiguous():
            x_cl = x_cl.contiguous()
        y = torch.empty_like(x_cl)
        rows = x_cl.numel() // C
        native.check(_lib().lb_bn_apply_fixed(
            x_cl.data_ptr(), run_mean.data_ptr(), run_var.data_ptr(),
            native.ptr(sh.master.detach() if sh else None),
            native.ptr(bh.master.detach() if bh else None), y.data_ptr(), rows, C, float(eps), act,
            float(act_param), native.dtype_code(x.dtype), native.stream_ptr()), "lb_bn_apply_fixed")
        native.count_launch()
        return _from_cl(y, x.dim())
    # reference semantics in PyTorch (fp32 statistics)
    dims = [0] + list(range(2, x.dim()))
    shape = [1, C] + [1] * (x.dim() - 2)
    xf = x.float()
    if training:
        n = x.numel() / C
        s = torch.stack([xf.sum(dims), (xf * xf).sum(dims)])
        if reduce_fn is not None:
            # the entry count travels with the sums: the ranks' shares of a mini-batch may differ
            # (the last mini-batch of an epoch, a sample-parallel tail behind a partitioned part)
            s = _ReduceSum.apply(torch.cat([s, s.new_full((1, C), n)]), reduce_fn)
            n = s[2].detach()
            var_scale = n / (n - correction).clamp_min(1.0)
        else:
            var_scale = n / (n - correction)
        mean = s[0] / n
        var = (s[1] / n - mean * mean) * var_scale
        var = torch.clamp(var, min=eps)
        with torch.no_grad():
            if run_mean is not None:
                # .data: the running statistics are views of the parameter arena, whose version
                # counter is shared with every weight saved for the backward pass
                run_mean.data.mul_(decay).add_((1 - decay) * mean.detach())
                run_var.data.mul_(decay).add_((1 - decay) * var.detach())
    else:
        mean, var = run_mean, run_var
    y = (xf - mean.view(shape)) * torch.rsqrt(var.view(shape) + eps)
    if sh is not None:
        y = y * sh.master.view(shape)
    if bh is not None:
        y = y + bh.master.view(shape)
    from .gemm import _ACT_FN
    return _ACT_FN[act](y, act_param).to(x.dtype)


class _ReduceSum(torch.autograd.Function):
    """Differentiable in-place sum over ranks (the gradient of a sum-allreduce is a
    sum-allreduce)."""

    @staticmethod
    def forward(ctx, t, reduce_fn):
        ctx.reduce_fn = reduce_fn
        out = t.clone()
        reduce_fn(out)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        ctx.reduce_fn(g)
        return g, None


# --------------------------------------------------------------------------- layer norm
class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, s_leaf, b_leaf, sh, bh, cols, eps):
        xc = x.contiguous()
        rows = xc.numel() // cols
        y = torch.empty_like(xc)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        scale = sh.master.detach().reshape(-1) if sh is not None else None
        bias = bh.master.detach().reshape(-1) if bh is not None else None
        native.check(_lib().lb_layer_norm_fwd(xc.data_ptr(), native.ptr(scale), native.ptr(bias),
                                              y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows,
                                              cols, float(eps), native.dtype_code(x.dtype),
                                              native.stream_ptr()), "lb_layer_norm_fwd")
        native.count_launch()
        ctx.save_for_backward(xc, mean, rstd)
        ctx.meta = (sh, bh, cols)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, mean, rstd = ctx.saved_tensors
        sh, bh, cols = ctx.meta
        dyc = dy.contiguous()
        rows = xc.numel() // cols
        dx = torch.empty_like(xc)
        scale = sh.master.detach().reshape(-1) if sh is not None else None
        dscale = sh.grad.view(-1) if (sh is not None and sh.grad is not None) else None
        dbias = bh.grad.view(-1) if (bh is not None and bh.grad is not None) else None
        native.check(_lib().lb_layer_norm_bwd(xc.data_ptr(), dyc.data_ptr(), native.ptr(scale),
                                              mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                              native.ptr(dscale), native.ptr(dbias), rows, cols,
                                              native.dtype_code(xc.dtype), native.stream_ptr()),
                     "lb_layer_norm_bwd")
        native.count_launch(2)
        if dscale is not None:
            sh.mark_ready()
        if dbias is not None:
            bh.mark_ready()
        return dx, None, None, None, None, None, None


def layer_norm(x, normalized_size: int, sh=None, bh=None, eps: float = 1e-5):
    """Normalise over the trailing ``normalized_size`` elements of every sample."""
    if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16, torch.float32):
        return _LayerNorm.apply(x, sh.master if sh else None, bh.master if bh else None, sh, bh,
                                int(normalized_size), eps)
    shape = x.shape
    x2 = x.reshape(-1, normalized_size).float()
    mean = x2.mean(1, keepdim=True)
    var = (x2 * x2).mean(1, keepdim=True) - mean * mean
    y = (x2 - mean) * torch.rsqrt(torch.clamp(var, min=0) + eps)
    if sh is not None:
        y = y * sh.master.reshape(1, -1)
    if bh is not None:
        y = y + bh.master.reshape(1, -1)
    return y.reshape(shape).to(x.dtype)


# --------------------------------------------------------------------------- softmax family
class _Softmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mode, in_scale, causal_period):
        xc = x.contiguous()
        cols = xc.shape[-1]
        rows = xc.numel() // cols
        y = torch.empty_like(xc)
        native.check(_lib().lb_softmax_fwd(xc.data_ptr(), y.data_ptr(), rows, cols, mode,
                                           float(in_scale), int(causal_period),
                                           native.dtype_code(x.dtype), native.stream_ptr()),
                     "lb_softmax_fwd")
        native.count_launch()
        ctx.save_for_backward(y)
        ctx.meta = (mode, in_scale, causal_period)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        mode, in_scale, causal_period = ctx.meta
        dyc = dy.contiguous()
        cols = y.shape[-1]
        rows = y.numel() // cols
        dx = torch.empty_like(y)
        native.check(_lib().lb_softmax_bwd(y.data_ptr(), dyc.data_ptr(), dx.data_ptr(), rows, cols,
                                           mode, float(in_scale), int(causal_period),
                                           native.dtype_code(y.dtype), native.stream_ptr()),
                     "lb_softmax_bwd")
        native.count_launch()
        return dx, None, None, None


def softmax_lastdim(x, log: bool = False, in_scale: float = 1.0, causal_period: int = 0):
    """(log-)softmax over the last dimension; optional input scale and causal masking of
    an S x S score matrix (row r sees columns <= r mod S)."""
    if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16, torch.float32):
        return _Softmax.apply(x, 1 if log else 0, in_scale, causal_period)
    z = x.float() * in_scale
    if causal_period:
        S = causal_period
        r = torch.arange(z.shape[-2], device=x.device) % S
        mask = torch.arange(z.shape[-1], device=x.device)[None, :] > r[:, None]
        z = z.masked_fill(mask, float("-inf"))
    out = F.log_softmax(z, -1) if log else F.softmax(z, -1)
    return out.to(x.dtype)


class _SoftmaxCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, labels):
        xc = x.contiguous()
        cols = xc.shape[-1]
        rows = xc.numel() // cols
        loss = torch.empty(rows, dtype=torch.float32, device=x.device)
        lse = torch.empty(rows, dtype=torch.float32, device=x.device)
        lab = labels.reshape(-1).to(torch.int64).contiguous()
        native.check(_lib().lb_softmax_ce_fwd(xc.data_ptr(), lab.data_ptr(), loss.data_ptr(),
                                              lse.data_ptr(), rows, cols,
                                              native.dtype_code(x.dtype), native.stream_ptr()),
                     "lb_softmax_ce_fwd")
        native.count_launch()
        ctx.save_for_backward(xc, lab, lse)
        return loss.reshape(x.shape[:-1])

    @staticmethod
    def backward(ctx, dloss):
        xc, lab, lse = ctx.saved_tensors
        cols = xc.shape[-1]
        rows = xc.numel() // cols
        dx = torch.empty_like(xc)
        g = dloss.reshape(-1).float().contiguous()
        native.check(_lib().lb_softmax_ce_bwd(xc.data_ptr(), lab.data_ptr(), lse.data_ptr(),
                                              g.data_ptr(), 0.0, dx.data_ptr(), rows, cols,
                                              native.dtype_code(xc.dtype), native.stream_ptr()),
                     "lb_softmax_ce_bwd")
        native.count_launch()
        return dx, None


def softmax_cross_entropy(logits, labels):
    """Per-row ``-log softmax(logits)[label]`` in fp32; rows with an out-of-range label give
    0 (value and gradient), as the reference's label-mode cross entropy does."""
    if logits.is_cuda and logits.dtype in (torch.float16, torch.bfloat16, torch.float32):
        return _SoftmaxCE.apply(logits, labels)
    C = logits.shape[-1]
    lab = labels.reshape(-1).long()
    ok = (lab >= 0) & (lab < C)
    lp = F.log_softmax(logits.float().reshape(-1, C), -1)
    picked = lp.gather(1, lab.clamp(0, C - 1)[:, None])[:, 0]
    return torch.where(ok, -picked, torch.zeros_like(picked)).reshape(logits.shape[:-1])


_LOSS_KIND = {"cross_entropy": 0, "mean_squared_error": 1, "mean_absolute_error": 2,
              "l1_norm": 3, "l2_norm2": 4}


class _SampleLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, kind):
        rows = a.shape[0]
        cols = a.numel() // max(rows, 1)
        ac = a.contiguous()
        bc = b.contiguous() if b is not None else None
        out = torch.empty(rows, dtype=torch.float32, device=a.device)
        native.check(_lib().lb_sample_loss_fwd(ac.data_ptr(), native.ptr(bc), out.data_ptr(), rows,
                                               cols, kind, native.dtype_code(a.dtype),
                                               native.stream_ptr()), "lb_sample_loss_fwd")
        native.count_launch()
        ctx.save_for_backward(ac, bc)
        ctx.meta = (kind, rows, cols)
        return out

    @staticmethod
    def backward(ctx, g):
        ac, bc = ctx.saved_tensors
        kind, rows, cols = ctx.meta
        da = torch.empty_like(ac) if ctx.needs_input_grad[0] else None
        db = torch.empty_like(bc) if (bc is not None and ctx.needs_input_grad[1]) else None
        gc = g.float().contiguous()
        native.check(_lib().lb_sample_loss_bwd(ac.data_ptr(), native.ptr(bc), gc.data_ptr(),
                                               native.ptr(da), native.ptr(db), rows, cols, kind,
                                               native.dtype_code(ac.dtype), native.stream_ptr()),
                     "lb_sample_loss_bwd")
        native.count_launch()
        return da, db, None


def sample_loss(kind: str, a, b=None):
    """One fp32 value per sample (dim 0): cross entropy on probabilities, MSE, MAE, L1, L2^2."""
    if a.is_cuda and a.dtype in (torch.float16, torch.bfloat16, torch.float32) and \
            (b is None or (b.dtype == a.dtype and b.shape == a.shape)):
        return _SampleLoss.apply(a, b, _LOSS_KIND[kind])
    n = a.shape[0]
    from ..exec.layer_base import rows2d
    af = rows2d(a.float())
    bf = rows2d(b.float()) if b is not None else None
    if kind == "cross_entropy":
        return torch.where(bf > 0, -bf * torch.log(af), torch.zeros_like(af)).sum(1)
    if kind == "mean_squared_error":
        return ((af - bf) ** 2).mean(1)
    if kind == "mean_absolute_error":
        return (af - bf).abs().mean(1)
    if kind == "l1_norm":
        return af.abs().sum(1)
    return (af * af).sum(1)


def topk_accuracy(scores, labels, k: int = 1):
    """1.0 where the label's score ranks among the k largest of its row (fp32 per row)."""
    if scores.is_cuda and scores.dtype in (torch.float16, torch.bfloat16, torch.float32):
        sc = scores.contiguous()
        cols = sc.shape[-1]
        rows = sc.numel() // cols
        lab = labels.reshape(-1).to(torch.int64).contiguous()
        out = torch.empty(rows, dtype=torch.float32, device=scores.device)
        native.check(_lib().lb_topk_accuracy(sc.data_ptr(), lab.data_ptr(), out.data_ptr(), rows,
                                             cols, int(k), native.dtype_code(sc.dtype),
                                             native.stream_ptr()), "lb_topk_accuracy")
        native.count_launch()
        return out.reshape(scores.shape[:-1])
    C = scores.shape[-1]
    lab = labels.reshape(-1).long()
    s = scores.float().reshape(-1, C)
    v = s.gather(1, lab.clamp(0, C - 1)[:, None])
    idx = torch.arange(C, device=s.device)[None, :]
    rank = ((s > v) | ((s == v) & (idx < lab[:, None]))).sum(1)
    return ((rank < k) & (lab >= 0) & (lab < C)).float().reshape(scores.shape[:-1])
