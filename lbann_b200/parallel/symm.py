"""Symmetric (peer-mapped) buffers and the device-side collectives built on them.

``SymmetricGroup`` covers a set of ranks on one NVSwitch domain.  ``alloc`` gives every
rank a buffer of the same size and the peer-mapped addresses of all the others; the
collectives (two-shot / one-shot all-reduce, row puts for halos and shuffles, group
barrier) are this library's kernels (``csrc/comm_kernels.cu``) working on those addresses
with peer loads and stores.  On CPU ranks (gloo) and single-rank groups the same methods
fall back to ``torch.distributed`` / local copies so host-side logic can be tested
without GPUs.
"""
from __future__ import annotations

import ctypes
import weakref
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import native
from ..ops.native import c_float, c_int, c_ll, c_void_p

_configured = False


def _lib():
    global _configured
    lib = native.cuda_lib()
    if not _configured:
        vpp = ctypes.POINTER(c_void_p)
        lib.lb_symm_alloc.restype = c_void_p
        lib.lb_symm_alloc.argtypes = [c_ll]
        lib.lb_symm_free.argtypes = [c_void_p]
        lib.lb_ipc_handle_bytes.restype = c_int
        lib.lb_ipc_get_handle.restype = c_int
        lib.lb_ipc_get_handle.argtypes = [c_void_p, c_void_p]
        lib.lb_ipc_open.restype = c_void_p
        lib.lb_ipc_open.argtypes = [c_void_p]
        lib.lb_ipc_close.argtypes = [c_void_p]
        lib.lb_comm_pad_bytes.restype = c_int
        lib.lb_allreduce_two_shot.restype = c_int
        lib.lb_allreduce_two_shot.argtypes = [vpp, vpp, c_int, c_int, c_ll, c_float, c_void_p,
                                              c_int, c_int, c_void_p]
        lib.lb_reduce_scatter_owned.restype = c_int
        lib.lb_reduce_scatter_owned.argtypes = [vpp, vpp, c_int, c_int, c_ll, c_ll, c_ll, c_float,
                                                c_void_p, c_int, c_int, c_void_p]
        lib.lb_allreduce_one_shot.restype = c_int
        lib.lb_allreduce_one_shot.argtypes = [vpp, vpp, c_int, c_int, c_void_p, c_void_p, c_int,
                                              c_int, c_ll, c_void_p, c_void_p]
        lib.lb_put_rows.restype = c_int
        lib.lb_put_rows.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_ll, c_ll, c_void_p]
        lib.lb_halo_exchange_fwd.restype = c_int
        lib.lb_halo_exchange_fwd.argtypes = [vpp, vpp, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_ll,
                                             c_ll, c_ll, c_float, c_int, c_void_p, c_void_p]
        lib.lb_halo_exchange_bwd.restype = c_int
        lib.lb_halo_exchange_bwd.argtypes = [vpp, vpp, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                             c_ll, c_ll, c_ll, c_ll, c_int, c_void_p, c_void_p]
        lib.lb_alltoall_slabs.restype = c_int
        lib.lb_alltoall_slabs.argtypes = [vpp, vpp, c_int, c_int, c_void_p, c_ll, c_ll, c_void_p, c_void_p]
        lib.lb_scatter_rows.restype = c_int
        lib.lb_scatter_rows.argtypes = [vpp, vpp, c_int, c_int, c_void_p, c_void_p, c_void_p, c_ll, c_ll,
                                        c_void_p, c_void_p]
        lib.lb_group_barrier.restype = c_int
        lib.lb_group_barrier.argtypes = [vpp, vpp, c_int, c_int, c_int, c_void_p, c_void_p]
        _configured = True
    return lib


class _DevMem:
    """Exposes a raw device allocation to PyTorch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 3, "strides": None}


def tensor_from_ptr(ptr: int, nbytes: int, device) -> torch.Tensor:
    t = torch.as_tensor(_DevMem(ptr, nbytes), device=device)
    t._lb_keepalive = True
    return t


class SymmetricBuffer:
    """One allocation per rank; ``local`` is this rank's bytes, ``peer_ptrs[r]`` the address
    of rank r's bytes as mapped into this process."""

    def __init__(self, group: "SymmetricGroup", nbytes: int):
        self.group = group
        self.nbytes = int(nbytes)
        dev = group.device
        if group.native:
            lib = _lib()
            ptr = lib.lb_symm_alloc(self.nbytes)
            if not ptr:
                raise native.NativeError(f"symmetric allocation of {nbytes} bytes failed")
            self.ptr = ptr
            hb = lib.lb_ipc_handle_bytes()
            handle = ctypes.create_string_buffer(hb)
            native.check(lib.lb_ipc_get_handle(ptr, handle), "lb_ipc_get_handle")
            handles = group.gather_object(bytes(handle.raw))
            self.peer_ptrs: List[int] = []
            for r, h in enumerate(handles):
                if r == group.rank:
                    self.peer_ptrs.append(ptr)
                else:
                    p = lib.lb_ipc_open(ctypes.create_string_buffer(h, hb))
                    if not p:
                        raise native.NativeError(f"cannot map the symmetric buffer of rank {r}")
                    self.peer_ptrs.append(p)
            self.local = tensor_from_ptr(ptr, self.nbytes, dev)
        else:
            self.local = torch.zeros(self.nbytes, dtype=torch.uint8, device=dev)
            self.ptr = self.local.data_ptr()
            self.peer_ptrs = [self.ptr] * group.world
        self._c_ptrs = (c_void_p * group.world)(*self.peer_ptrs)

    def view(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        es = torch.empty((), dtype=dtype).element_size()
        n = (self.nbytes - offset_bytes) // es if numel is None else numel
        return self.local[offset_bytes:offset_bytes + n * es].view(dtype)

    def peer_ptr(self, r: int, offset_bytes: int = 0) -> int:
        return self.peer_ptrs[r] + offset_bytes


_live_groups = weakref.WeakSet()


def _poison_groups(code: int) -> None:
    """A wait on another rank ran out somewhere on this device: the kernels involved left
    before their closing rendezvous, so the use counters of the flag rows no longer agree
    between the ranks and later rendezvous could pass on stale flags.  Every group of this
    process refuses further collectives (restart from a checkpoint)."""
    if code == 5:
        for g in list(_live_groups):
            g.poisoned = True


native.on_status(_poison_groups)


class SymmetricGroup:
    """Collectives of one group launch on ONE stream at a time and in the same order on every
    rank: the rendezvous rows (phases 0/1 all-reduce and reduce-scatter, 2/3 everything else)
    are shared by all kernels of the group and count their uses on the device."""

    def __init__(self, device, ranks: Optional[Sequence[int]] = None, pg=None):
        self.device = torch.device(device)
        self.pg = pg
        self.distributed = dist.is_initialized() and (pg is not None or ranks is None or len(ranks) > 1)
        if self.distributed:
            self.world = dist.get_world_size(pg) if pg is not None else dist.get_world_size()
            self.rank = dist.get_rank(pg) if pg is not None else dist.get_rank()
        else:
            self.world, self.rank = 1, 0
        self.native = self.device.type == "cuda" and self.world > 1
        self.poisoned = False
        _live_groups.add(self)
        self.epoch = 0
        self.ctr = None          # use counters of the flag rows (this rank's own memory)
        self.ctr_ptr = None
        self.pad = None
        self.staging = None
        self.bytes_moved = 0
        if self.native:
            self.pad = SymmetricBuffer(self, _lib().lb_comm_pad_bytes())
            self.ctr = torch.zeros(_lib().lb_comm_pad_bytes() // 4, dtype=torch.int32, device=self.device)
            self.ctr_ptr = self.ctr.data_ptr()
            self.staging = SymmetricBuffer(self, self.world * 4096 * 4)   # one-shot slots
            self.barrier_host()

    def _guard(self):
        if self.poisoned:
            raise native.NativeError("this group saw a rendezvous time out: its ranks are no longer "
                                     "in step; restart from the last checkpoint")

    def gather_object(self, obj):
        if not self.distributed:
            return [obj]
        out = [None] * self.world
        dist.all_gather_object(out, obj, group=self.pg)
        return out

    def barrier_host(self):
        if self.distributed:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            dist.barrier(group=self.pg)

    def alloc(self, nbytes: int) -> SymmetricBuffer:
        b = SymmetricBuffer(self, nbytes)
        self.barrier_host()
        return b

    def _next_epoch(self) -> int:
        self.epoch = (self.epoch + 1) & 0x7FFFFFFF or 1
        return self.epoch

    # ------------------------------------------------------------------ collectives
    def allreduce_(self, buf: SymmetricBuffer, dtype: torch.dtype, numel: int, scale: float = 1.0,
                   offset_bytes: int = 0, blocks: int = 32):
        """In-place sum over the group of ``numel`` elements at ``offset_bytes`` of ``buf``."""
        self._guard()
        if self.world == 1:
            if scale != 1.0:
                buf.view(dtype, numel, offset_bytes).mul_(scale)
            return
        if not self.native:
            t = buf.view(dtype, numel, offset_bytes)
            dist.all_reduce(t, group=self.pg)
            if scale != 1.0:
                t.mul_(scale)
            return
        ptrs = (c_void_p * self.world)(*[p + offset_bytes for p in buf.peer_ptrs])
        rc = _lib().lb_allreduce_two_shot(ptrs, self.pad._c_ptrs, self.rank, self.world, numel,
                                          float(scale), self.ctr_ptr,
                                          native.dtype_code(dtype), blocks, native.stream_ptr())
        native.check(rc, "lb_allreduce_two_shot")
        native.count_launch()
        es = torch.empty((), dtype=dtype).element_size()
        self.bytes_moved += 2 * numel * es * (self.world - 1) // self.world

    def reduce_scatter_owned_(self, buf: SymmetricBuffer, dtype: torch.dtype, e0: int, e1: int,
                              own_elems: int, scale: float = 1.0, blocks: int = 48):
        """Elements [e0, e1) of ``buf``: every ownership block (``own_elems`` elements, block b
        owned by rank b % world) ends up summed over the group, times ``scale``, in its
        owner's buffer.  The other ranks' copies of the block keep their own contribution.
        No closing rendezvous: call a later collective before the buffers are overwritten."""
        self._guard()
        if self.world == 1:
            if scale != 1.0:
                buf.view(dtype)[e0:e1].mul_(scale)
            return
        if not self.native:
            t = buf.view(dtype)[e0:e1]
            dist.all_reduce(t, group=self.pg)
            if scale != 1.0:
                t.mul_(scale)
            return
        rc = _lib().lb_reduce_scatter_owned(buf._c_ptrs, self.pad._c_ptrs, self.rank, self.world,
                                            e0, e1, own_elems, float(scale), self.ctr_ptr,
                                            native.dtype_code(dtype), blocks, native.stream_ptr())
        native.check(rc, "lb_reduce_scatter_owned")
        native.count_launch()
        es = torch.empty((), dtype=dtype).element_size()
        self.bytes_moved += (e1 - e0) * es * (self.world - 1) // self.world

    def allreduce_small_(self, t: torch.Tensor, op: str = "sum"):
        """In-place all-reduce of a short fp32 tensor (<= 4096 elements) in one kernel."""
        self._guard()
        if self.world == 1:
            return
        if not self.native or t.dtype != torch.float32 or t.numel() > 4096 or not t.is_contiguous():
            o = dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.MAX
            if t.dtype in (torch.float32, torch.float64, torch.int32, torch.int64):
                dist.all_reduce(t, o, group=self.pg)
            else:
                f = t.float()
                dist.all_reduce(f, o, group=self.pg)
                t.copy_(f)
            return
        rc = _lib().lb_allreduce_one_shot(self.staging._c_ptrs, self.pad._c_ptrs, self.rank, self.world,
                                          t.data_ptr(), t.data_ptr(), t.numel(),
                                          0 if op == "sum" else 1, 4096, self.ctr_ptr,
                                          native.stream_ptr())
        native.check(rc, "lb_allreduce_one_shot")
        native.count_launch()
        self.bytes_moved += t.numel() * 4 * (self.world - 1)

    def put_rows(self, src: torch.Tensor, dst_buf: SymmetricBuffer, dst_rank: int, dst_offset_bytes: int,
                 rows: int, row_bytes: int, src_pitch: int, dst_pitch: int):
        """Copy ``rows`` rows from a local tensor into rank ``dst_rank``'s buffer."""
        self._guard()
        rc = _lib().lb_put_rows(src.data_ptr(), src_pitch, dst_buf.peer_ptr(dst_rank, dst_offset_bytes),
                                dst_pitch, rows, row_bytes, native.stream_ptr())
        native.check(rc, "lb_put_rows")
        native.count_launch()
        self.bytes_moved += rows * row_bytes

    def halo_forward(self, x: torch.Tensor, ext: SymmetricBuffer, n: int, dl: int, h: int,
                     plane_bytes: int, fill: float) -> bool:
        """One kernel: ``x`` [n, dl, plane] -> interior of this rank's extended buffer, boundary
        planes -> the neighbours' halo planes, with the two rendezvous inside.  Returns False
        when the shape is not covered (the caller then uses separate puts and barriers)."""
        self._guard()
        up = self.rank - 1 if self.rank > 0 else -1
        down = self.rank + 1 if self.rank < self.world - 1 else -1
        rc = _lib().lb_halo_exchange_fwd(ext._c_ptrs, self.pad._c_ptrs, self.rank, self.world, up, down,
                                         x.data_ptr(), n, dl, h, plane_bytes, float(fill),
                                         native.dtype_code(x.dtype), self.ctr_ptr,
                                         native.stream_ptr())
        if rc == -2:
            return False
        native.check(rc, "lb_halo_exchange_fwd")
        native.count_launch()
        self.bytes_moved += n * h * plane_bytes * ((up >= 0) + (down >= 0))
        return True

    def halo_backward(self, g: torch.Tensor, recv: SymmetricBuffer, dx: torch.Tensor, n: int, dl: int,
                      h: int, plane_bytes: int) -> bool:
        """One kernel: halo-plane gradients -> the neighbours' receive areas, and
        ``dx`` = interior of ``g`` + what the neighbours sent."""
        self._guard()
        up = self.rank - 1 if self.rank > 0 else -1
        down = self.rank + 1 if self.rank < self.world - 1 else -1
        rc = _lib().lb_halo_exchange_bwd(recv._c_ptrs, self.pad._c_ptrs, self.rank, self.world, up, down,
                                         g.data_ptr(), dx.data_ptr(), n, dl, h, plane_bytes,
                                         native.dtype_code(g.dtype), self.ctr_ptr,
                                         native.stream_ptr())
        if rc == -2:
            return False
        native.check(rc, "lb_halo_exchange_bwd")
        native.count_launch()
        self.bytes_moved += n * h * plane_bytes * ((up >= 0) + (down >= 0))
        return True

    def alltoall_slabs(self, src: torch.Tensor, dst: SymmetricBuffer, count: int, slab_bytes: int) -> bool:
        """One kernel: slab i of ``src`` (``count`` contiguous slabs) -> rank i % world, slot
        (i // world) * world + rank of ``dst``; ends with a rendezvous of the group.  Returns
        False when the slabs are not multiples of 16 bytes (the caller falls back to puts)."""
        self._guard()
        rc = _lib().lb_alltoall_slabs(dst._c_ptrs, self.pad._c_ptrs, self.rank, self.world,
                                      src.data_ptr(), count, slab_bytes, self.ctr_ptr,
                                      native.stream_ptr())
        if rc == -2:
            return False
        native.check(rc, "lb_alltoall_slabs")
        native.count_launch()
        self.bytes_moved += count * slab_bytes * (self.world - 1) // self.world
        return True

    def scatter_rows(self, src: Optional[torch.Tensor], dst: SymmetricBuffer, dst_rank: torch.Tensor,
                     dst_row: torch.Tensor, rows: int, row_bytes: int) -> bool:
        """One kernel: row j of ``src`` -> row ``dst_row[j]`` of rank ``dst_rank[j]``'s ``dst``
        (int32 device tensors), closed by a rendezvous of the group.  Every rank of the group
        calls it, also with ``rows == 0``.  False when rows are not multiples of 16 bytes."""
        self._guard()
        rc = _lib().lb_scatter_rows(dst._c_ptrs, self.pad._c_ptrs, self.rank, self.world,
                                    src.data_ptr() if (src is not None and rows) else None,
                                    dst_rank.data_ptr() if rows else None,
                                    dst_row.data_ptr() if rows else None, rows, row_bytes,
                                    self.ctr_ptr, native.stream_ptr())
        if rc == -2:
            return False
        native.check(rc, "lb_scatter_rows")
        native.count_launch()
        self.bytes_moved += rows * row_bytes
        return True

    def barrier_device(self, phase: int = 3):
        """Stream-ordered rendezvous of the group (no host synchronisation)."""
        self._guard()
        if self.world == 1:
            return
        if not self.native:
            dist.barrier(group=self.pg)
            return
        rc = _lib().lb_group_barrier(self.pad._c_ptrs, self.pad._c_ptrs, self.rank, self.world, phase,
                                     self.ctr_ptr, native.stream_ptr())
        native.check(rc, "lb_group_barrier")
        native.count_launch()
