"""Flat parameter arena and the fused (single-launch) optimizer step.

``ParameterArena`` lays every weight tensor of a model out in one fp32 buffer (each tensor
padded to the optimizer's chunk size), with a parallel gradient arena, two optimizer-state
arenas and an optional 16-bit compute copy.  ``step()`` updates all tensors with one
kernel launch on CUDA; on CPU it applies the same formulas tensor by tensor.  The update
rules are the reference's (src/optimizers/{sgd,adam,adagrad,rmsprop}.cu); its per-tensor
launch structure (one kernel per weight tensor) is not kept.
"""
from __future__ import annotations

import math
import struct
from typing import Dict, List, Optional

import torch

from . import native
from .native import c_float, c_int, c_ll, c_void_p

# hypergradient Adam is applied tensor by tensor after the fused launch (``_step_hypergradient``):
# the fused kernel sees those tensors as frozen
KIND = {"sgd": 0, "adam": 1, "adagrad": 2, "rmsprop": 3, "none": -1, "hypergradient_adam": -1}
_SEG_FMT = "<qqiiffffffffff"  # 64 bytes, mirrors OptSegment in csrc/optim.cu
assert struct.calcsize(_SEG_FMT) == 64
_configured = False


def _lib():
    global _configured
    lib = native.cuda_lib()
    if not _configured:
        lib.lb_fused_optimizer.restype = c_int
        lib.lb_fused_optimizer.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int, c_ll, c_float, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.lb_unscale_check.restype = c_int
        lib.lb_unscale_check.argtypes = [c_void_p, c_ll, c_float, c_void_p, c_int, c_void_p, c_int, c_void_p]
        lib.lb_unscale_check_owned.restype = c_int
        lib.lb_unscale_check_owned.argtypes = [c_void_p, c_ll, c_float, c_void_p, c_int, c_void_p, c_int,
                                               c_int, c_int, c_int, c_void_p]
        lib.lb_fused_optimizer_sharded.restype = c_int
        lib.lb_fused_optimizer_sharded.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_int, c_ll, c_float, c_void_p, c_void_p,
                                                   c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                   c_void_p, c_void_p]
        lib.lb_fused_optimizer_sharded2.restype = c_int
        lib.lb_fused_optimizer_sharded2.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                    c_void_p, c_int, c_ll, c_float, c_void_p, c_void_p,
                                                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                    c_void_p, c_int, c_void_p]
        lib.lb_amp_update.restype = c_int
        lib.lb_amp_update.argtypes = [c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_void_p]
        lib.lb_sqnorm.restype = c_int
        lib.lb_sqnorm.argtypes = [c_void_p, c_ll, c_void_p, c_int, c_void_p]
        lib.lb_cast_scale.restype = c_int
        lib.lb_cast_scale.argtypes = [c_void_p, c_void_p, c_ll, c_float, c_int, c_int, c_void_p]
        lib.lb_opt_chunk.restype = c_int
        _configured = True
    return lib


CHUNK = 1024
OWN_CHUNKS = 16        # chunks per ownership block of a sharded update (64 KiB of fp32)


class ArenaShard:
    """Ownership of an arena whose optimizer update is sharded over the ranks of a group:
    blocks of ``OWN_CHUNKS`` chunks are dealt round-robin, block b belongs to rank b % world.
    Gradients of a block are reduced onto its owner, only the owner keeps optimizer state for
    it and updates it, and the new values are stored into every rank's master arena
    (``peer_master``: the peer-mapped addresses of the master arenas).  ``after_step`` runs
    once the update has been launched (a rendezvous of the group)."""

    def __init__(self, rank: int, world: int, peer_master, after_step=None):
        self.rank, self.world = int(rank), int(world)
        self.own_chunks = OWN_CHUNKS
        self.own_elems = OWN_CHUNKS * CHUNK
        self.peer_master = peer_master
        self.after_step = after_step
        self.state_whole = True      # False once a sharded step has run since the last gather

    def owner_mask(self, numel: int, device) -> torch.Tensor:
        """bool[numel]: elements whose block this rank owns."""
        nb = (numel + self.own_elems - 1) // self.own_elems
        own = (torch.arange(nb, device=device) % self.world) == self.rank
        return own.repeat_interleave(self.own_elems)[:numel]


class Slot:
    """One weight tensor's place in the arena plus its optimizer hyper-parameters."""

    def __init__(self, name: str, shape, offset: int):
        self.name = name
        self.shape = tuple(shape)
        self.count = int(math.prod(self.shape)) if self.shape else 1
        self.offset = offset
        self.kind = "none"
        self.hp: Dict[str, float] = {}
        self.step_count = 0
        self.l2 = 0.0
        self.extra: Dict[str, torch.Tensor] = {}     # optimizer state beyond the two arenas

    def segment_bytes(self) -> bytes:
        hp = self.hp
        kind = KIND[self.kind]
        lr = float(hp.get("learn_rate", 0.0))
        p0 = p1 = eps = wd = corr = 0.0
        nesterov = 0
        if self.kind == "sgd":
            p0 = float(hp.get("momentum", 0.0))
            nesterov = int(bool(hp.get("nesterov", False)))
        elif self.kind == "adam":
            p0, p1 = float(hp.get("beta1", 0.9)), float(hp.get("beta2", 0.99))
            eps = float(hp.get("eps", 1e-8))
            wd = float(hp.get("adamw_weight_decay", 0.0))
        elif self.kind == "adagrad":
            eps = float(hp.get("eps", 1e-8))
        elif self.kind == "rmsprop":
            p0 = float(hp.get("decay_rate", 0.9))
            eps = float(hp.get("eps", 1e-8))
        return struct.pack(_SEG_FMT, self.offset, self.count, kind, nesterov, lr, p0, p1, eps, wd,
                           corr, float(self.l2), 0.0, 0.0, 0.0)


class ParameterArena:
    def __init__(self, device: torch.device, compute_dtype: Optional[torch.dtype] = None,
                 grad_dtype: torch.dtype = torch.float32, allocator=None):
        self.device = torch.device(device)
        self.compute_dtype = compute_dtype
        self.grad_dtype = grad_dtype
        self.slots: List[Slot] = []
        self.total = 0
        self.allocator = allocator  # callable(nelem, dtype) -> tensor (e.g. symmetric memory)
        self.master = self.grad = self.state0 = self.state1 = self.compute = None
        self._seg_dev = None
        self._seg_stage = []
        self._seg_key = None
        self.step_dev = None      # int32[1] on the device: optimizer step number
        self.lr_scale_dev = None  # float32[1] on the device: global learning-rate multiplier
        self.shard: Optional[ArenaShard] = None   # set when the update is sharded over ranks
        self.state_compact = False    # optimizer state stored for the owned blocks only
        self._full_state = None       # [state0, state1] at full size while a gathered copy is in use

    # ---- layout
    def reserve(self, name: str, shape) -> Slot:
        if self.master is not None:
            raise RuntimeError("arena already materialised")
        slot = Slot(name, shape, self.total)
        self.slots.append(slot)
        self.total += (slot.count + CHUNK - 1) // CHUNK * CHUNK
        return slot

    def _alloc(self, dtype):
        n = max(self.total, CHUNK)
        if self.allocator is not None:
            t = self.allocator(n, dtype)
            t.zero_()
            return t
        return torch.zeros(n, dtype=dtype, device=self.device)

    def materialise(self):
        self.master = self._alloc(torch.float32)
        self.grad = self._alloc(self.grad_dtype)
        self.state0 = torch.zeros_like(self.master)
        self.state1 = None
        if self.compute_dtype in (torch.float16, torch.bfloat16):
            self.compute = torch.zeros(self.master.numel(), dtype=self.compute_dtype,
                                       device=self.device)
        return self

    def ensure_state1(self):
        if self.state1 is None:
            self.state1 = torch.zeros_like(self.state0)       # full size, or the owned share when compact

    # ---- optimizer state for the owned blocks only (memory sharded over the ranks)
    def _block_counts(self):
        sh = self.shard
        nchunks = (self.total + CHUNK - 1) // CHUNK
        nblocks = (nchunks + sh.own_chunks - 1) // sh.own_chunks
        mine = (nblocks - sh.rank + sh.world - 1) // sh.world
        return nblocks, mine

    def _pack_state(self, full: torch.Tensor) -> torch.Tensor:
        """Owned blocks of a full-size state tensor, densely, in block order."""
        sh = self.shard
        nblocks, mine = self._block_counts()
        padded = torch.zeros(nblocks * sh.own_elems, dtype=full.dtype, device=full.device)
        padded[:min(full.numel(), padded.numel())] = full.reshape(-1)[:padded.numel()]
        return padded.view(nblocks, sh.own_elems)[sh.rank::sh.world].reshape(-1).clone()

    def _unpack_state(self, compact: torch.Tensor) -> torch.Tensor:
        """Full-size tensor with this rank's blocks filled in and zeros elsewhere."""
        sh = self.shard
        nblocks, mine = self._block_counts()
        padded = torch.zeros(nblocks * sh.own_elems, dtype=compact.dtype, device=compact.device)
        padded.view(nblocks, sh.own_elems)[sh.rank::sh.world] = compact.view(mine, sh.own_elems)
        return padded[:self.master.numel()] if padded.numel() >= self.master.numel() else \
            torch.cat([padded, padded.new_zeros(self.master.numel() - padded.numel())])

    def compact_state(self) -> None:
        """Keep optimizer state for the blocks this rank owns only: the moments of a sharded
        update are never read elsewhere, so 8 of Adam's 18 bytes per parameter shrink to 8 / world
        (what the reference's sharded weights do for their optimizer state,
        src/weights/data_type_weights.cpp:244-283).  Call once, after the shard is installed and
        before the first step (the storage must not move once a step has been captured)."""
        if self.shard is None or self.shard.world <= 1 or self.state_compact or self.state0 is None:
            return
        old0, old1 = self.state0, self.state1
        self.state0 = self._pack_state(old0)
        self.state1 = self._pack_state(old1) if old1 is not None else None
        self.state_compact = True
        self._full_state = None

    def state_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.state0, self.state1) if t is not None)

    def state_view(self, which: int, slot: Slot) -> torch.Tensor:
        """A weight tensor's slice of optimizer state ``which`` (0 / 1).  With compact state this
        is a view of the gathered full-size copy (``gather_sharded_state`` makes it whole across
        the ranks; ``commit_state`` writes changes back into the owned share)."""
        if not self.state_compact:
            return self.view(self.state0 if which == 0 else self.state1, slot)
        if self._full_state is None:
            self._full_state = [self._unpack_state(self.state0),
                                self._unpack_state(self.state1) if self.state1 is not None else None]
        if which == 1 and self._full_state[1] is None:
            self.ensure_state1()
            self._full_state[1] = self._unpack_state(self.state1)
        return self.view(self._full_state[which], slot)

    def commit_state(self) -> None:
        """Write a gathered full-size copy that was modified (checkpoint restart, model
        exchange) back into the owned share, in place, and drop the copy."""
        if not self.state_compact or self._full_state is None:
            return
        self.state0.copy_(self._pack_state(self._full_state[0]))
        if self._full_state[1] is not None:
            self.ensure_state1()
            self.state1.copy_(self._pack_state(self._full_state[1]))
        self._full_state = None

    def view(self, buf: torch.Tensor, slot: Slot) -> torch.Tensor:
        return buf[slot.offset:slot.offset + slot.count].view(slot.shape if slot.shape else (1,))

    def refresh_compute(self):
        """Re-derive the 16-bit compute copy from the master weights (after init / load)."""
        if self.compute is None:
            return
        if self.master.is_cuda:
            rc = _lib().lb_cast_scale(self.master.data_ptr(), self.compute.data_ptr(),
                                      self.master.numel(), 1.0, native.DT_F32,
                                      native.dtype_code(self.compute.dtype), native.stream_ptr())
            native.check(rc, "lb_cast_scale")
            native.count_launch()
        else:
            self.compute.copy_(self.master)

    def zero_grad(self):
        self.grad.zero_()

    def gather_sharded_state(self, allreduce_sum) -> None:
        """Make the optimizer state whole on every rank after sharded steps (checkpoints,
        model exchange): each rank clears the blocks it does not own and the ranks sum.
        ``allreduce_sum(tensor)`` sums in place over the group.  Collective."""
        sh = self.shard
        if self.state_compact:
            # every rank contributes its blocks to a full-size copy; the sum is the whole state
            self._full_state = [self._unpack_state(self.state0),
                                self._unpack_state(self.state1) if self.state1 is not None else None]
            for st in self._full_state:
                if st is not None:
                    allreduce_sum(st)
            sh.state_whole = True
            return
        # (no short cut on ``state_whole``: a replayed graph steps without passing through here)
        if sh is None:
            return
        mask = sh.owner_mask(self.state0.numel(), self.state0.device)
        for st in (self.state0, self.state1):
            if st is None:
                continue
            st.mul_(mask)
            allreduce_sum(st)
        sh.state_whole = True

    # ---- optimizer
    def _segments(self):
        blob = b"".join(s.segment_bytes() for s in self.slots)
        if blob != self._seg_key:
            self._seg_key = blob
            if self._seg_dev is None or self._seg_dev.numel() != len(blob):
                self._seg_dev = torch.empty(len(blob), dtype=torch.uint8, device=self.device)
                self._seg_stage = []
            # pinned staging buffers are rotated so an upload in flight is never overwritten
            if len(self._seg_stage) < 4:
                stage = (torch.empty(len(blob), dtype=torch.uint8).pin_memory(), torch.cuda.Event())
                self._seg_stage.append(stage)
            else:
                stage = self._seg_stage.pop(0)
                stage[1].synchronize()
                self._seg_stage.append(stage)
            stage[0].copy_(torch.frombuffer(bytearray(blob), dtype=torch.uint8))
            self._seg_dev.copy_(stage[0], non_blocking=True)
            stage[1].record()
        return self._seg_dev

    def step(self, inv_scale: float = 1.0, skip_flag: Optional[torch.Tensor] = None,
             inv_scale_dev: Optional[torch.Tensor] = None):
        """Advance every slot's step counter and apply its optimizer.  ``inv_scale_dev``: a
        one-element fp32 CUDA tensor multiplied into the gradients as they are read."""
        for s in self.slots:
            if s.kind != "none":
                s.step_count += 1
        if any(s.kind in ("adam", "hypergradient_adam") for s in self.slots):
            self.ensure_state1()
        if any(s.kind == "hypergradient_adam" for s in self.slots):
            self._step_hypergradient(inv_scale, skip_flag, inv_scale_dev)
        if self.master.is_cuda:
            segs = self._segments()
            if self.step_dev is None:
                self.step_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
                self.lr_scale_dev = torch.ones(1, dtype=torch.float32, device=self.device)
            self.step_dev.add_(1)
            if skip_flag is not None:
                self.step_dev.sub_(skip_flag.to(torch.int32))   # a skipped step is not counted
            s1 = self.state1 if self.state1 is not None else self.state0
            sh = self.shard
            if self._full_state is not None and not torch.cuda.is_current_stream_capturing():
                self.commit_state()      # a gathered copy may have been written to (restart, exchange)
            rc = _lib().lb_fused_optimizer_sharded2(
                self.master.data_ptr(), self.grad.data_ptr(), self.state0.data_ptr(),
                s1.data_ptr(), native.ptr(self.compute), segs.data_ptr(), len(self.slots),
                self.total, float(inv_scale), native.ptr(skip_flag), self.step_dev.data_ptr(),
                self.lr_scale_dev.data_ptr(), native.ptr(inv_scale_dev), native.dtype_code(self.grad.dtype),
                native.dtype_code(self.compute.dtype) if self.compute is not None else native.DT_BF16,
                sh.rank if sh else 0, sh.world if sh else 1, sh.own_chunks if sh else 1,
                sh.peer_master if sh else None, 1 if self.state_compact else 0, native.stream_ptr())
            native.check(rc, "lb_fused_optimizer_sharded")
            native.count_launch()
            if sh is not None:
                # every rank's stores must have landed before anybody reads the new weights;
                # the 16-bit copy is then cast from the (whole) master arena
                sh.state_whole = False
                if sh.after_step is not None:
                    sh.after_step()
                self.refresh_compute()
            return
        self._step_cpu(inv_scale)

    @torch.no_grad()
    def _step_hypergradient(self, inv_scale, skip_flag, inv_scale_dev):
        """Adam whose learning rate follows its own gradient
        (src/optimizers/hypergradient_adam.cpp:137-185): lr += hyper_lr * <g, previous update
        direction>, then a bias-corrected Adam step on g + eps whose direction is remembered."""
        if skip_flag is not None and bool(int(skip_flag.item())):
            return
        scale = float(inv_scale) * (float(inv_scale_dev.item()) if inv_scale_dev is not None else 1.0)
        for s in self.slots:
            if s.kind != "hypergradient_adam":
                continue
            hp = s.hp
            b1, b2 = float(hp.get("beta1", 0.9)), float(hp.get("beta2", 0.99))
            eps = float(hp.get("eps", 1e-8))
            x = self.view(self.master, s)
            g = self.view(self.grad, s).float() * scale
            if s.l2:
                g = g + s.l2 * x
            old = s.extra.get("old_gradient")
            if old is None:
                old = s.extra["old_gradient"] = torch.zeros_like(x)
            lr = float(hp.get("learn_rate", 0.0)) + float(hp.get("hyper_learning_rate", 1e-7)) * \
                float((g * old).sum())
            hp["learn_rate"] = lr
            t = s.step_count
            corr = math.sqrt(1.0 - b2 ** t) / (1.0 - b1 ** t)
            g = g + eps
            m1, m2 = self.view(self.state0, s), self.view(self.state1, s)
            m1.mul_(b1).add_(g, alpha=1 - b1)
            m2.mul_(b2).addcmul_(g, g, value=1 - b2)
            old.copy_(corr * m1 / (m2.sqrt() + eps))
            x.sub_(lr * old)
            if self.compute is not None:
                self.view(self.compute, s).copy_(x)

    @torch.no_grad()
    def _step_cpu(self, inv_scale: float):
        for s in self.slots:
            if s.kind == "none":
                continue
            x = self.view(self.master, s)
            g = self.view(self.grad, s).float() * inv_scale
            if s.l2:
                g = g + s.l2 * x
            hp = s.hp
            lr = float(hp.get("learn_rate", 0.0))
            if s.kind == "sgd":
                mu = float(hp.get("momentum", 0.0))
                if mu != 0.0:
                    v = self.view(self.state0, s)
                    v.mul_(mu).add_(g)
                    x.sub_(lr * (mu * v + g) if hp.get("nesterov") else lr * v)
                else:
                    x.sub_(lr * g)
            elif s.kind == "adam":
                b1, b2 = float(hp.get("beta1", 0.9)), float(hp.get("beta2", 0.99))
                eps = float(hp.get("eps", 1e-8))
                wd = float(hp.get("adamw_weight_decay", 0.0))
                t = s.step_count
                corr = lr * math.sqrt(1.0 - b2 ** t) / (1.0 - b1 ** t)
                m1, m2 = self.view(self.state0, s), self.view(self.state1, s)
                ok = torch.isfinite(g)
                gz = torch.where(ok, g, torch.zeros_like(g))
                nm1 = b1 * m1 + (1 - b1) * gz
                nm2 = b2 * m2 + (1 - b2) * gz * gz
                m1.copy_(torch.where(ok, nm1, m1))
                m2.copy_(torch.where(ok, nm2, m2))
                upd = corr * (m1 / (m2.sqrt() + eps)) + lr * wd * x
                x.sub_(torch.where(ok, upd, torch.zeros_like(upd)))
            elif s.kind == "adagrad":
                c = self.view(self.state0, s)
                c.add_(g * g)
                x.sub_(lr * g / (c.sqrt() + float(hp.get("eps", 1e-8))))
            elif s.kind == "rmsprop":
                d = float(hp.get("decay_rate", 0.9))
                c = self.view(self.state0, s)
                c.mul_(d).add_((1 - d) * g * g)
                x.sub_(lr * g / (c.sqrt() + float(hp.get("eps", 1e-8))))
        if self.compute is not None:
            self.compute.copy_(self.master)

    # ---- reductions used by AMP / clipping / L2 reporting
    def grad_sqnorm(self, buf: Optional[torch.Tensor] = None) -> torch.Tensor:
        buf = self.grad if buf is None else buf
        if buf.is_cuda:
            out = torch.zeros(1, dtype=torch.float32, device=buf.device)
            rc = _lib().lb_sqnorm(buf.data_ptr(), buf.numel(), out.data_ptr(),
                                  native.dtype_code(buf.dtype), native.stream_ptr())
            native.check(rc, "lb_sqnorm")
            native.count_launch()
            return out
        return (buf.float() ** 2).sum().reshape(1)

    def unscale_and_check(self, inv_scale: float, flag: torch.Tensor, write_back: bool = True,
                          inv_scale_dev: Optional[torch.Tensor] = None):
        """grad *= inv_scale (optionally) and flag[0] |= any non-finite value.  With
        ``inv_scale_dev`` (a one-element fp32 CUDA tensor) the factor is read on the device."""
        if self.grad.is_cuda:
            sh = self.shard     # sharded update: every rank checks the chunks it owns
            rc = _lib().lb_unscale_check_owned(self.grad.data_ptr(), self.grad.numel(), float(inv_scale),
                                               native.ptr(inv_scale_dev), 1 if write_back else 0,
                                               flag.data_ptr(), native.dtype_code(self.grad.dtype),
                                               sh.rank if sh else 0, sh.world if sh else 1,
                                               sh.own_chunks if sh else 1, native.stream_ptr())
            native.check(rc, "lb_unscale_check_owned")
            native.count_launch()
            return
        g = self.grad.float() * inv_scale
        if not torch.isfinite(g).all():
            flag.fill_(1)
        if write_back:
            self.grad.copy_(g)


def amp_update(state: torch.Tensor, reduced, flag: torch.Tensor, growth: float, backoff: float,
               interval: int) -> None:
    """One step of the loss-scale schedule on the device (``state``: scale, 1 / scale, clean
    steps, consecutive skipped steps; ``reduced``: overflow flag after the reduction over the
    ranks or None; ``flag``: int32 flag that the fused optimizer reads)."""
    rc = _lib().lb_amp_update(state.data_ptr(), native.ptr(reduced), flag.data_ptr(), float(growth),
                              float(backoff), float(interval), native.stream_ptr())
    native.check(rc, "lb_amp_update")
    native.count_launch()
