"""Sharded fully-connected layers on the fused GEMM + collective kernels.

Three differentiable building blocks (``x`` is ``[tokens, features]``, weights are
``[out_features, in_features]`` like the reference's fully-connected layer):

``ColumnParallelLinear``  weights split by OUTPUT rows, activations split by tokens on
    entry (sequence-parallel): forward all-gather -> GEMM, the result ``[tokens, out/P]``
    stays split by features.
``RowParallelLinear``     weights split by INPUT columns, activations split by features on
    entry: forward GEMM -> reduce-scatter, the result ``[tokens/P, out]`` is split by tokens
    again.  A column-parallel layer followed by a row-parallel one is the transformer
    FFN / attention projection pair; it reproduces what the reference obtains from a
    model-parallel (MC,MR-distributed) fully connected layer
    (src/layers/learning/fully_connected.cpp:638-808) without ever materialising a
    gathered activation or an unreduced output.
``ShardedLinear``         FSDP-style weights (split by output rows, optimizer state only for
    the local rows; src/weights/data_type_weights.cpp:244-266,456-462): forward gathers
    the weight tile by tile inside the GEMM, backward multiplies by the staged copy and
    reduce-scatters the weight gradient straight into the local fp32 gradient shard
    (include/lbann/optimizers/optimizer_impl.hpp:113-169 does all-reduce + copy).

All of them run on the symmetric-memory kernels on GPUs and on torch.distributed
collectives on CPU (gloo), so the same code is covered by the CPU tests.
"""
from __future__ import annotations

from typing import Optional

import torch

from .fused import FusedGemm
from .symm import SymmetricBuffer, SymmetricGroup


class _ModelParallelLinear(torch.autograd.Function):
    """y = x W^T with the OUTPUT rows of W dealt to the ranks of a process-grid column:
    every rank multiplies by its row block and the blocks are all-gathered; backward
    all-reduces the partial input gradient and leaves the weight gradient of the other
    ranks' rows at zero (the data-parallel gradient all-reduce completes it)."""

    @staticmethod
    def forward(ctx, x, w, b, tp):
        P, r = tp.size, tp.rank
        n = w.shape[0]
        lo, hi = tp.bounds(n)
        ctx.tp, ctx.bounds, ctx.has_bias = tp, (lo, hi, n), b is not None
        ctx.save_for_backward(x, w)
        y_loc = torch.nn.functional.linear(x, w[lo:hi].to(x.dtype),
                                           None if b is None else b[lo:hi].to(x.dtype))
        return tp.all_gather_cols(y_loc, n)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        lo, hi, n = ctx.bounds
        dy_loc = dy[:, lo:hi]
        dx = dy_loc.float() @ w[lo:hi].float()
        tp.all_reduce(dx)
        dw = torch.zeros_like(w, dtype=torch.float32)
        dw[lo:hi] = dy_loc.float().t() @ x.float()
        db = None
        if ctx.has_bias:
            db = torch.zeros(n, dtype=torch.float32, device=dy.device)
            db[lo:hi] = dy_loc.float().sum(0)
        # Only this rank produces these rows while replicated layers are produced by every
        # rank of the column; the trainer-wide gradient sum is divided by the column size,
        # so the row block is pre-multiplied by it.
        dw.mul_(tp.size)
        if db is not None:
            db.mul_(tp.size)
        return dx.to(x.dtype), dw.to(w.dtype), db, None


class _ModelParallelLinearFused(torch.autograd.Function):
    """The same layer on this library's kernels (GPUs, 16-bit activations): the forward
    product is ONE tcgen05 GEMM whose epilogue stores every finished tile of this rank's
    column block into the output of all ranks of the column (peer stores over NVLink: GEMM
    -> all-gather fused, ``lb_gemm_bcast_tc``); backward multiplies on the tensor cores,
    sums the partial input gradients with the two-shot all-reduce kernel in symmetric
    memory and writes the weight gradient of the own rows straight into the arena."""

    @staticmethod
    def forward(ctx, x, w_leaf, b_leaf, tp, layer):
        import ctypes
        from ..ops import native
        from ..ops.gemm import _lib as gemm_lib
        wh = layer.w.handle
        bh = layer.b.handle if layer.b is not None else None
        P = tp.size
        n, k = wh.master.shape
        lo, hi = tp.bounds(n)
        tokens = x.shape[0]
        dt = x.dtype
        es = _esize(dt)
        x = x.contiguous()
        ybuf = tp.ws.get(("y", layer.name, tokens, n, dt), tokens * n * es)
        y = ybuf.view(dt, tokens * n).view(tokens, n)
        w_loc = wh.cast(dt)[lo:hi]
        bias = bh.master.detach()[lo:hi].float().contiguous() if bh is not None else None
        ptrs = (native.c_void_p * P)(*[ybuf.peer_ptr(q, lo * es) for q in range(P)])
        lib = gemm_lib()
        lib.lb_gemm_bcast_tc.restype = native.c_int
        lib.lb_gemm_bcast_tc.argtypes = lib.lb_gemm_tc.argtypes[:-1] + [
            ctypes.POINTER(native.c_void_p), native.c_int, native.c_void_p]
        tp.sg.barrier_device(2)            # every rank is done reading the previous output
        rc = lib.lb_gemm_bcast_tc(x.data_ptr(), w_loc.data_ptr(), ybuf.ptr + lo * es, native.ptr(bias),
                                  tokens, hi - lo, k, 1, k, k, n, 0, 0, 0, 0, 0, native.dtype_code(dt),
                                  native.dtype_code(dt), 1.0, 0.0, 1 if bias is not None else 0, 0, 0.0, 0,
                                  ptrs, P, native.stream_ptr())
        native.check(rc, "lb_gemm_bcast_tc")
        native.count_launch()
        tp.sg.barrier_device(3)            # all column blocks have landed everywhere
        ctx.save_for_backward(x)
        ctx.meta = (tp, layer, lo, hi, n, k)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm
        from ..ops.nn import column_sums
        (x,) = ctx.saved_tensors
        tp, layer, lo, hi, n, k = ctx.meta
        wh = layer.w.handle
        bh = layer.b.handle if layer.b is not None else None
        dt = x.dtype
        tokens = x.shape[0]
        dy_loc = dy[:, lo:hi]
        if dy_loc.stride(1) != 1 or dy_loc.stride(0) % 8 or dy_loc.data_ptr() % 16:
            dy_loc = dy_loc.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dbuf = tp.ws.get(("dx", layer.name, tokens, k), tokens * k * 4)
            part = dbuf.view(torch.float32, tokens * k).view(tokens, k)
            gemm(dy_loc, wh.cast(dt)[lo:hi], out=part)                    # [tokens, k] partial sum
            tp.sg.allreduce_(dbuf, torch.float32, tokens * k)
            dx = part.to(dt)
        if wh.grad is not None:
            # rows of the other ranks stay zero here: the data-parallel reduction, which divides
            # by the column size, completes them (hence the factor)
            gemm(dy_loc, x, trans_a=True, out=wh.grad.view(n, k)[lo:hi], alpha=float(tp.size), beta=1.0)
            wh.mark_ready()
        if bh is not None and bh.grad is not None:
            bh.grad.view(-1)[lo:hi].add_(column_sums(dy_loc.contiguous()) * float(tp.size))
            bh.mark_ready()
        return dx, None, None, None, None


class TensorParallel:
    """Model-parallel fully-connected layers on a trainer's process grid (the reference's
    ``data_layout='model_parallel'`` over an MC,MR grid, src/layers/learning/
    fully_connected.cpp:638-808).  The ranks of one grid column share the mini-batch and
    split the output neurons."""

    def __init__(self, ctx):
        import torch.distributed as dist
        self.ctx = ctx
        self.comm = ctx.comm
        self.group = self.comm.grid_col_group
        self.size = self.comm.grid_height
        self.rank = dist.get_rank(self.group) if self.size > 1 else 0
        # symmetric memory over the ranks of this grid column (GPUs only)
        self.sg = SymmetricGroup(ctx.device, pg=self.group) if (
            self.size > 1 and ctx.device.type == "cuda") else None
        self.ws = _Workspace(self.sg) if self.sg is not None else None

    def bounds(self, n: int):
        per = (n + self.size - 1) // self.size
        lo = min(n, self.rank * per)
        return lo, min(n, lo + per)

    def all_gather_cols(self, y_loc: torch.Tensor, n: int) -> torch.Tensor:
        import torch.distributed as dist
        if self.size == 1:
            return y_loc
        per = (n + self.size - 1) // self.size
        pad = torch.zeros((y_loc.shape[0], per), dtype=y_loc.dtype, device=y_loc.device)
        pad[:, :y_loc.shape[1]] = y_loc
        parts = [torch.empty_like(pad) for _ in range(self.size)]
        dist.all_gather(parts, pad, group=self.group)
        return torch.cat(parts, 1)[:, :n].contiguous()

    def all_reduce(self, t: torch.Tensor):
        import torch.distributed as dist
        if self.size > 1:
            dist.all_reduce(t, group=self.group)

    def _fused_ok(self, layer, x) -> bool:
        if self.sg is None or not self.sg.native or layer.transpose or x.dim() != 2:
            return False
        n, k = layer.w.handle.master.shape
        return (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and n % (32 * self.size) == 0
                and k % 8 == 0)

    def linear(self, layer, x: torch.Tensor) -> torch.Tensor:
        if x.dim() == 3 and self._fused_ok(layer, x.reshape(-1, x.shape[-1])):
            # per-token layers (channelwise fully connected): tokens are rows
            y = _ModelParallelLinearFused.apply(
                x.reshape(-1, x.shape[-1]), layer.w.handle.master,
                layer.b.handle.master if layer.b is not None else None, self, layer)
            return y.reshape(x.shape[0], x.shape[1], -1)
        if self._fused_ok(layer, x):
            return _ModelParallelLinearFused.apply(
                x, layer.w.handle.master, layer.b.handle.master if layer.b is not None else None,
                self, layer)
        w = layer.w.handle.master
        if layer.transpose:
            w = w.t()
        b = layer.b.handle.master if layer.b is not None else None
        return _ModelParallelLinear.apply(x, w, b, self)

    def softmax(self, x: torch.Tensor, log: bool) -> torch.Tensor:
        """Activations are whole on every rank after the gather: a local softmax."""
        fn = torch.log_softmax if log else torch.softmax
        return fn(x.float(), dim=-1).to(x.dtype)


class _Workspace:
    """Symmetric buffers of one layer, allocated collectively on first use."""

    def __init__(self, group: SymmetricGroup):
        self.group = group
        self.bufs = {}

    def get(self, key, nbytes) -> SymmetricBuffer:
        b = self.bufs.get(key)
        if b is None or b.nbytes < nbytes:
            b = self.group.alloc(nbytes)
            self.bufs[key] = b
        return b


def _esize(dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def _mm_tn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a^T @ b in fp32 (weight-gradient form) on the tcgen05 GEMM when on a GPU."""
    if a.is_cuda and a.dtype in (torch.float16, torch.bfloat16):
        from ..ops.gemm import gemm
        return gemm(a.contiguous(), b.contiguous(), trans_a=True, out_dtype=torch.float32)
    return a.float().t() @ b.float()


class _ColumnParallel(torch.autograd.Function):
    """y[:, rank's features] = gather(x) . w_local^T."""

    @staticmethod
    def forward(ctx, x_local, w_local, layer):
        g, fg, ws = layer.group, layer.fused, layer.ws
        rows, k = x_local.shape
        dt = x_local.dtype
        xbuf = ws.get(("x", rows, k, dt), rows * k * _esize(dt))
        xbuf.view(dt, rows * k).view(rows, k).copy_(x_local)
        y = fg.allgather_gemm(xbuf, rows, k, w_local.to(dt), sharded="a", dtype=dt)
        ctx.layer, ctx.shape = layer, (rows, k)
        ctx.save_for_backward(w_local)
        ctx.xbuf = xbuf
        return y

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        g, fg, ws = layer.group, layer.fused, layer.ws
        (w_local,) = ctx.saved_tensors
        rows, k = ctx.shape
        dt = dy.dtype
        P = g.world
        dy = dy.contiguous()
        # dx[tokens, k] = sum over ranks of dy[:, f_r] . w_r, scattered by tokens
        obuf = ws.get(("dx", rows, k), rows * k * 4)
        dx = fg.gemm_reduce_scatter(dy, w_local.to(dt), obuf, rows, trans_b=True).to(dt)
        # dw_r[f_r, k] = dy[:, f_r]^T . gather(x): the gathered operand is split along the
        # reduction dimension here, which the fused kernel does not take: gather, then GEMM
        full = layer.gather_rows(ctx.xbuf, rows, k, dt)
        dw = _mm_tn(dy, full)
        return dx, dw.to(w_local.dtype), None


class ColumnParallelLinear:
    def __init__(self, group: SymmetricGroup, fused: Optional[FusedGemm] = None):
        self.group = group
        self.fused = fused or FusedGemm(group)
        self.ws = _Workspace(group)

    def gather_rows(self, buf: SymmetricBuffer, rows: int, k: int, dtype) -> torch.Tensor:
        """All ranks' ``[rows, k]`` blocks of a symmetric buffer as one local tensor."""
        g = self.group
        local = buf.view(dtype, rows * k).view(rows, k)
        if g.world == 1:
            return local
        import torch.distributed as dist
        full = torch.empty((g.world * rows, k), dtype=dtype, device=local.device)
        dist.all_gather_into_tensor(full, local.contiguous(), group=g.pg)
        return full

    def __call__(self, x_local: torch.Tensor, w_local: torch.Tensor) -> torch.Tensor:
        return _ColumnParallel.apply(x_local, w_local, self)


class _RowParallel(torch.autograd.Function):
    """y[rank's tokens] = sum over ranks of x[:, f_r] . w[:, f_r]^T."""

    @staticmethod
    def forward(ctx, x_feat, w_local, layer):
        g, fg, ws = layer.group, layer.fused, layer.ws
        tokens, kl = x_feat.shape
        n = w_local.shape[0]
        P = g.world
        rows = tokens // P
        dt = x_feat.dtype
        obuf = ws.get(("y", rows, n), rows * n * 4)
        y = fg.gemm_reduce_scatter(x_feat.contiguous(), w_local.to(dt), obuf, rows).to(dt)
        ctx.layer, ctx.dims = layer, (tokens, kl, n, rows)
        ctx.save_for_backward(x_feat, w_local)
        return y

    @staticmethod
    def backward(ctx, dy_local):
        layer = ctx.layer
        g, fg, ws = layer.group, layer.fused, layer.ws
        x_feat, w_local = ctx.saved_tensors
        tokens, kl, n, rows = ctx.dims
        dt = dy_local.dtype
        # dx[:, f_r] = gather(dy)[tokens, n] . w[:, f_r]   (all-gather -> GEMM)
        dbuf = ws.get(("dy", rows, n, dt), rows * n * _esize(dt))
        dbuf.view(dt, rows * n).view(rows, n).copy_(dy_local)
        dx = fg.allgather_gemm(dbuf, rows, n, w_local.to(dt).t().contiguous(), sharded="a", dtype=dt)
        # dw[:, f_r] = gather(dy)^T . x[:, f_r]
        full = layer.gather_rows(dbuf, rows, n, dt)
        dw = _mm_tn(full, x_feat)
        return dx, dw.to(w_local.dtype), None


class RowParallelLinear(ColumnParallelLinear):
    def __call__(self, x_feat: torch.Tensor, w_local: torch.Tensor) -> torch.Tensor:
        return _RowParallel.apply(x_feat, w_local, self)


class _Sharded(torch.autograd.Function):
    """y = x . gather(w_shards)^T with the gather inside the GEMM; dW reduce-scattered."""

    @staticmethod
    def forward(ctx, x, w_shard_leaf, layer):
        g, fg = layer.group, layer.fused
        rows, k = layer.shard_rows, layer.k
        dt = x.dtype
        wbuf = layer.compute_shard(dt)
        y = fg.allgather_gemm(wbuf, rows, k, x.contiguous(), sharded="b", dtype=dt)
        ctx.layer = layer
        ctx.stage_token = fg.last_stage_token    # None when this forward did not stage
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        g, fg = layer.group, layer.fused
        (x,) = ctx.saved_tensors
        rows, k = layer.shard_rows, layer.k
        dt = dy.dtype
        dy = dy.contiguous()
        w_full = layer.gathered_weight(dt, ctx.stage_token)
        if x.is_cuda:
            from ..ops.gemm import gemm
            dx = gemm(dy, w_full)
        else:
            dx = (dy.float() @ w_full.float()).to(dt)
        # dW[n, k] = dy^T . x summed over the data-parallel ranks, rows scattered to their owners
        gbuf = layer.grad_buffer()
        dw = fg.gemm_reduce_scatter(dy, x.contiguous(), gbuf, rows, trans_a=True, trans_b=True,
                                    zero=True)
        return dx, dw.to(layer.w_shard.dtype), None


class ShardedLinear:
    """Weights ``[P * shard_rows, k]`` of which this rank owns rows
    ``[rank * shard_rows, (rank + 1) * shard_rows)`` (fp32 master ``w_shard``)."""

    def __init__(self, group: SymmetricGroup, w_shard: torch.Tensor, fused: Optional[FusedGemm] = None):
        self.group = group
        self.fused = fused or FusedGemm(group)
        self.ws = _Workspace(group)
        self.w_shard = w_shard
        self.shard_rows, self.k = w_shard.shape

    def compute_shard(self, dtype) -> SymmetricBuffer:
        """This rank's rows in the compute dtype, in symmetric memory (refreshed per call)."""
        n = self.shard_rows * self.k
        buf = self.ws.get(("w", dtype), n * _esize(dtype))
        buf.view(dtype, n).view(self.shard_rows, self.k).copy_(self.w_shard.detach())
        return buf

    def gathered_weight(self, dtype, stage_token=None) -> torch.Tensor:
        """The full weight matrix for the data-gradient product.  ``stage_token`` is what the
        matching forward call left in ``FusedGemm.last_stage_token``: the staged copy in local
        memory is used only when that forward staged (small mini-batches do not) and no other
        call of the same operand shape has overwritten the copy since; otherwise the shards
        are gathered again."""
        key = (self.shard_rows, self.k, dtype)
        st = self.fused._stage.get(key)
        g = self.group
        if (st is not None and g.native and stage_token is not None
                and self.fused._stage_token.get(key) == stage_token):
            full = st[0]
            # the local rows are read from the shard itself in the forward kernel: fill them in
            full[g.rank * self.shard_rows:(g.rank + 1) * self.shard_rows].copy_(self.w_shard.detach())
            return full
        buf = self.ws.get(("w", dtype), self.shard_rows * self.k * _esize(dtype))
        return ColumnParallelLinear.gather_rows(self, buf, self.shard_rows, self.k, dtype)

    def grad_buffer(self) -> SymmetricBuffer:
        return self.ws.get(("dw",), self.shard_rows * self.k * 4)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return _Sharded.apply(x, self.w_shard, self)
