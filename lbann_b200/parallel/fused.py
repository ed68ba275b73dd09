"""GEMM fused with its collective over NVLink peer memory (``csrc/gemm_comm_tc.cu``).

``allgather_gemm``      Y = concat_r(X_r) . W^T   or   Y = X . concat_r(W_r)^T, where the
                        shards X_r / W_r live in a symmetric buffer: the kernel's TMA loads
                        read every tile from the rank that owns it, so no all-gather pass
                        and no gathered copy exist.
``gemm_reduce_scatter`` OUT_owner += A . B^T over the ranks' K slices: the epilogue adds
                        every tile into the output shard of the rank that owns its rows.

These are the building blocks of the sharded-weights (FSDP) path and of the
tensor-parallel fully-connected layer; the reference does the same work as a gather of
the weights followed by a local GEMM (src/weights/data_type_weights.cpp:456-462) and an
all-reduce of the full gradient followed by a copy of the local shard
(include/lbann/optimizers/optimizer_impl.hpp:113-169), and as a distributed El::Gemm for
model-parallel layers (src/layers/learning/fully_connected.cpp:638-808).

On CPU / gloo (tests, fall-back) the same functions run as torch.distributed
collectives around a local matmul.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native
from .symm import SymmetricBuffer, SymmetricGroup

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_configured = False


def _lib():
    global _configured
    lib = native.cuda_lib()
    if not _configured:
        lib.lb_gemm_comm_tc.restype = c_int
        lib.lb_gemm_comm_tc.argtypes = [
            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int, c_int, c_int,
            c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
            ctypes.c_uint, c_int, c_void_p, c_int, c_int, c_void_p]
        _configured = True
    return lib


class FusedGemm:
    """Fused GEMM + collective entry points of one symmetric group."""

    def __init__(self, group: SymmetricGroup):
        self.group = group
        self._maps = None
        self._stage = {}            # (rows, k, dtype) -> (gathered, flags)
        self._stage_token = {}      # (rows, k, dtype) -> serial number of the call that staged last
        self._calls = 0
        self.last_stage_token = None
        self._epoch = 0
        self.helpers = 6            # copying CTAs of the staged all-gather -> GEMM
        self.bytes_over_nvlink = 0

    # ------------------------------------------------------------------ helpers
    def _maps_dev(self) -> int:
        if self._maps is None:
            self._maps = torch.empty(32 * 128, dtype=torch.uint8, device=self.group.device)
            lib = _lib()
            lib.lb_gemm_comm_forget.restype = None
            lib.lb_gemm_comm_forget.argtypes = [c_void_p]
            lib.lb_gemm_comm_forget(self._maps.data_ptr())   # nothing uploaded there yet
        return self._maps.data_ptr()

    def _staging(self, rows: int, k: int, dtype: torch.dtype):
        """Local gathered buffer and per-block flags for one operand shape.  The flags are
        cleared in the stream before every launch and the "block present" value is constant,
        so a launch carries no per-call value and can be replayed from a CUDA graph."""
        key = (rows, k, dtype)
        if key not in self._stage:
            P = self.group.world
            gathered = torch.empty((P * rows, k), dtype=dtype, device=self.group.device)
            flags = torch.zeros(P * rows // 128, dtype=torch.int32, device=self.group.device)
            self._stage[key] = (gathered, flags)
        gathered, flags = self._stage[key]
        flags.zero_()
        return gathered, flags, 1

    def _ptr_array(self, buf: SymmetricBuffer, offset_bytes: int = 0):
        return (c_void_p * self.group.world)(*[p + offset_bytes for p in buf.peer_ptrs])

    # ------------------------------------------------------------------ all-gather -> GEMM
    def allgather_gemm(self, shards: SymmetricBuffer, shard_rows: int, k: int, other: torch.Tensor,
                       *, sharded: str = "a", dtype: torch.dtype = torch.bfloat16,
                       out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                       alpha: float = 1.0, offset_bytes: int = 0, sync: bool = True,
                       staged: Optional[bool] = None) -> torch.Tensor:
        """``sharded='a'``: rows of the LEFT operand are spread over the ranks
        (``shards`` holds this rank's ``[shard_rows, k]`` block); returns
        ``concat(shards) @ other.T`` of shape ``[world * shard_rows, other.shape[0]]``.
        ``sharded='b'``: rows of the RIGHT operand (an ``[N, k]`` weight matrix, N split
        over the ranks) are spread; returns ``other @ concat(shards).T``.
        ``sync``: rendezvous first so that every rank's shard is complete.
        ``staged``: copy the remote shards once into local memory inside the same kernel
        (copying CTAs + per-block flags) instead of reading every tile through NVLink;
        default: whenever a remote tile would be read by more than two output tiles."""
        g = self.group
        P = g.world
        out_dtype = out_dtype or dtype
        local = shards.view(dtype, shard_rows * k, offset_bytes).view(shard_rows, k)
        if sharded == "a":
            M, N = P * shard_rows, other.shape[0]
        else:
            M, N = other.shape[0], P * shard_rows
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=other.device)
        if not g.native:
            if P > 1:
                full = torch.empty((P * shard_rows, k), dtype=dtype, device=local.device)
                dist.all_gather_into_tensor(full, local.contiguous(), group=g.pg)
            else:
                full = local
            a, b = (full, other) if sharded == "a" else (other, full)
            out.copy_((alpha * (a.float() @ b.float().t())).to(out.dtype))
            return out
        if sync:
            g.barrier_device(2)
        other = other.contiguous()
        ptrs = self._ptr_array(shards, offset_bytes)
        a_ptrs, b_ptrs = (ptrs, None) if sharded == "a" else (None, ptrs)
        reuse = (N + 255) // 256 if sharded == "a" else (M + 127) // 128
        if staged is None:
            staged = reuse > 2
        staged = bool(staged) and shard_rows % 128 == 0 and P > 1
        gathered = flags = None
        epoch = 0
        # Callers that want to reuse the gathered copy later (the data-gradient product of a
        # sharded layer) keep the token of THEIR call: the copy is theirs only while no other
        # call with the same operand shape has staged since, and only if this call staged.
        self._calls += 1
        self.last_stage_token = None
        if staged:
            gathered, flags, epoch = self._staging(shard_rows, k, dtype)
            self._stage_token[(shard_rows, k, dtype)] = self._calls
            self.last_stage_token = self._calls
        rc = _lib().lb_gemm_comm_tc(
            other.data_ptr() if sharded == "b" else None, other.data_ptr() if sharded == "a" else None,
            out.data_ptr(), M, N, k, k, k, out.stride(0), 0, 0, native.dtype_code(dtype),
            native.dtype_code(out.dtype), float(alpha), a_ptrs, shard_rows if sharded == "a" else 0,
            b_ptrs, shard_rows if sharded == "b" else 0, P, g.rank, self._maps_dev(),
            native.ptr(gathered), native.ptr(flags), epoch, self.helpers, None, 0, 0,
            native.stream_ptr())
        native.check(rc, "lb_gemm_comm_tc (all-gather -> GEMM)")
        native.count_launch()
        self.bytes_over_nvlink += (P - 1) * shard_rows * k * local.element_size()
        return out

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_reduce_scatter(self, a: torch.Tensor, b: torch.Tensor, out: SymmetricBuffer,
                            rows_per_rank: int, *, trans_a: bool = False, trans_b: bool = False,
                            alpha: float = 1.0, offset_bytes: int = 0, zero: bool = True) -> torch.Tensor:
        """Every rank holds a K slice: ``a`` is ``[M, K_local]`` (or ``[K_local, M]`` with
        ``trans_a``), ``b`` is ``[N, K_local]`` (or ``[K_local, N]`` with ``trans_b``).  The
        sum over ranks of ``a @ b.T`` is left, in fp32, distributed by rows: this rank's
        ``[rows_per_rank, N]`` block of ``out`` (returned as a view).  ``zero``: clear the
        local block first (the kernel accumulates)."""
        g = self.group
        P = g.world
        M = a.shape[1] if trans_a else a.shape[0]
        N = b.shape[1] if trans_b else b.shape[0]
        K = a.shape[0] if trans_a else a.shape[1]
        mine = out.view(torch.float32, rows_per_rank * N, offset_bytes).view(rows_per_rank, N)
        if not g.native:
            af = (a.t() if trans_a else a).float()
            bf = (b.t() if trans_b else b).float()
            full = alpha * (af @ bf.t())
            if P * rows_per_rank != M:
                full = torch.nn.functional.pad(full, (0, 0, 0, P * rows_per_rank - M))
            if P > 1:
                res = torch.empty_like(mine)
                if g.device.type == "cuda":
                    dist.reduce_scatter_tensor(res, full.contiguous(), group=g.pg)
                else:   # gloo has no reduce-scatter: all-reduce and keep the local rows
                    dist.all_reduce(full, group=g.pg)
                    res = full[g.rank * rows_per_rank:(g.rank + 1) * rows_per_rank]
            else:
                res = full
            if zero:
                mine.copy_(res)
            else:
                mine.add_(res)
            return mine
        a = a.contiguous()
        b = b.contiguous()
        shard_elems = rows_per_rank * N
        use_slots = zero and P > 1 and shard_elems % 4 == 0
        if use_slots:
            # Every source rank owns a slot at every other rank: the epilogue writes partial
            # tiles there with plain (posted, coalesced) stores - own rows go straight into
            # the output shard - and a short kernel adds the P - 1 slots after the rendezvous.
            # Remote fp32 atomics would need one NVLink transaction per 16 bytes.
            key = ("rs", shard_elems)
            slots = self._stage.get(key)
            if slots is None:
                slots = g.alloc((P - 1) * shard_elems * 4)
                self._stage[key] = slots
            ptr_list = []
            for r in range(P):
                if r == g.rank:
                    ptr_list.append(out.peer_ptr(r, offset_bytes))
                else:
                    slot = (g.rank - r - 1) % P
                    ptr_list.append(slots.peer_ptr(r, slot * shard_elems * 4))
            ptrs = (c_void_p * P)(*ptr_list)
        else:
            if zero:
                mine.zero_()
            ptrs = self._ptr_array(out, offset_bytes)
        g.barrier_device(2)           # destinations are ready (cleared / no longer being read)
        rc = _lib().lb_gemm_comm_tc(
            a.data_ptr(), b.data_ptr(), None, M, N, K, a.stride(0), b.stride(0), N,
            1 if trans_a else 0, 1 if trans_b else 0, native.dtype_code(a.dtype), native.DT_F32,
            float(alpha), None, 0, None, 0, P, g.rank, None, None, None, 0, 0, ptrs, rows_per_rank,
            1 if use_slots else 0, native.stream_ptr())
        native.check(rc, "lb_gemm_comm_tc (GEMM -> reduce-scatter)")
        native.count_launch()
        g.barrier_device(3)           # every rank's contributions have landed
        if use_slots:
            lib = _lib()
            lib.lb_rs_reduce.restype = c_int
            lib.lb_rs_reduce.argtypes = [c_void_p, c_void_p, c_int, c_ll, c_ll, c_void_p]
            rc = lib.lb_rs_reduce(mine.data_ptr(), slots.ptr, P - 1, shard_elems, shard_elems,
                                  native.stream_ptr())
            native.check(rc, "lb_rs_reduce")
            native.count_launch()
        self.bytes_over_nvlink += (P - 1) * rows_per_rank * N * 4
        return mine
