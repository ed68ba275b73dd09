"""Process topology and host-side collectives: the ``lbann_comm`` of this framework.

One process per GPU.  The world is split into equally sized *trainers* by contiguous blocks
of ranks (src/comm.cpp:99-139); ranks with the same position in different trainers form the
*inter-trainer* communicator; each trainer may further carry a 2-D grid (rows x columns, the
reference's ``--trainer_grid_height``) for sharded weights / model-parallel layers, and
sub-grids for sub-graph parallelism (src/comm.cpp:141-321).  ``torch.distributed`` (NCCL on
GPUs, gloo on CPU ranks) provides bootstrap and the baseline collectives; the device-side
collectives of the hot paths live in ``parallel/symm.py`` and ``csrc/comm_kernels.cu``.
Byte and barrier counters mirror include/lbann/comm.hpp:834-860.
"""
from __future__ import annotations

import os
import socket
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class LbannComm:
    def __init__(self, procs_per_trainer: int = 0, grid_height: int = 1, backend: Optional[str] = None,
                 device: Optional[torch.device] = None, init: bool = True, timeout_s: float = 600.0):
        self.device = device or torch.device("cpu")
        env_world = int(os.environ.get("WORLD_SIZE", "1"))
        if init and env_world > 1 and not dist.is_initialized():
            import datetime
            backend = backend or ("nccl" if self.device.type == "cuda" else "gloo")
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
            kw = {}
            if backend == "nccl":
                kw["device_id"] = self.device
            dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
        self.distributed = dist.is_initialized()
        self.world_size = dist.get_world_size() if self.distributed else 1
        self.rank_in_world = dist.get_rank() if self.distributed else 0
        self.local_rank = int(os.environ.get("LOCAL_RANK", self.rank_in_world))
        self.bytes_sent = 0
        self.bytes_received = 0
        self.num_barriers = 0
        self.num_collectives = 0
        self.trainer_group = None
        self.intertrainer_group = None
        self.node_group = None
        self.grid_row_group = self.grid_col_group = None
        self.subgrid_groups = {}
        self._split_trainers(procs_per_trainer or self.world_size)
        self._split_grid(grid_height)

    # ---------------------------------------------------------------- topology
    def _split_trainers(self, ppt: int):
        if self.world_size % ppt:
            raise ValueError(f"world size {self.world_size} is not a multiple of procs_per_trainer {ppt}")
        self.procs_per_trainer = ppt
        self.num_trainers = self.world_size // ppt
        self.trainer_rank = self.rank_in_world // ppt
        self.rank_in_trainer = self.rank_in_world % ppt
        if not self.distributed:
            return
        if self.num_trainers == 1:
            self.trainer_group = dist.group.WORLD
            self.trainer_ranks = list(range(self.world_size))
        else:
            for t in range(self.num_trainers):
                ranks = list(range(t * ppt, (t + 1) * ppt))
                g = dist.new_group(ranks)
                if t == self.trainer_rank:
                    self.trainer_group, self.trainer_ranks = g, ranks
            for r in range(ppt):
                ranks = [t * ppt + r for t in range(self.num_trainers)]
                g = dist.new_group(ranks)
                if r == self.rank_in_trainer:
                    self.intertrainer_group, self.intertrainer_ranks = g, ranks

    def _split_grid(self, height: int):
        """Trainer grid of ``height`` rows; a rank's (row, col) = (r mod height, r div height),
        the column-major order of an Elemental grid."""
        ppt = self.procs_per_trainer
        height = max(1, int(height))
        if ppt % height:
            raise ValueError(f"trainer grid height {height} does not divide {ppt}")
        self.grid_height, self.grid_width = height, ppt // height
        self.grid_row = self.rank_in_trainer % height
        self.grid_col = self.rank_in_trainer // height
        if not self.distributed:
            return
        base = self.trainer_rank * ppt
        if height > 1 and self.grid_width > 1:
            for t in range(self.num_trainers):
                b = t * ppt
                for c in range(self.grid_width):     # ranks of one grid column (vary row)
                    ranks = [b + c * height + r for r in range(height)]
                    g = dist.new_group(ranks)
                    if t == self.trainer_rank and c == self.grid_col:
                        self.grid_col_group, self.grid_col_ranks = g, ranks
                for r in range(height):              # ranks of one grid row (vary col)
                    ranks = [b + c * height + r for c in range(self.grid_width)]
                    g = dist.new_group(ranks)
                    if t == self.trainer_rank and r == self.grid_row:
                        self.grid_row_group, self.grid_row_ranks = g, ranks
        elif height > 1:
            self.grid_col_group, self.grid_col_ranks = self.trainer_group, list(range(base, base + ppt))
        else:
            self.grid_row_group, self.grid_row_ranks = self.trainer_group, list(range(base, base + ppt))

    def split_subgrids(self, num: int):
        """Split the trainer into ``num`` contiguous sub-grids (block order,
        src/utils/lbann_library.cpp:310-346); returns this rank's sub-grid index."""
        ppt = self.procs_per_trainer
        if ppt % num:
            raise ValueError(f"cannot split {ppt} ranks into {num} sub-grids")
        size = ppt // num
        mine = self.rank_in_trainer // size
        if self.distributed:
            base = self.trainer_rank * ppt
            for t in range(self.num_trainers):
                for s in range(num):
                    ranks = [t * ppt + s * size + i for i in range(size)]
                    g = dist.new_group(ranks)
                    if t == self.trainer_rank:
                        self.subgrid_groups[s] = (g, ranks)
            # peers: same position in every sub-grid
            for t in range(self.num_trainers):
                for i in range(size):
                    ranks = [t * ppt + s * size + i for s in range(num)]
                    g = dist.new_group(ranks)
                    if t == self.trainer_rank and i == self.rank_in_trainer % size:
                        self.subgrid_peer_group, self.subgrid_peer_ranks = g, ranks
        self.num_subgrids, self.subgrid_index, self.subgrid_size = num, mine, size
        return mine

    def new_group(self, ranks: Sequence[int]):
        return dist.new_group(list(ranks)) if self.distributed else None

    # ---------------------------------------------------------------- queries
    def am_world_master(self) -> bool:
        return self.rank_in_world == 0

    def am_trainer_master(self) -> bool:
        return self.rank_in_trainer == 0

    def hostname_hash(self) -> int:
        return hash(socket.gethostname()) & 0x7FFFFFFF

    # ---------------------------------------------------------------- collectives (host API)
    def _count(self, t: torch.Tensor, peers: int):
        n = t.numel() * t.element_size()
        self.bytes_sent += n * max(peers - 1, 0)
        self.bytes_received += n * max(peers - 1, 0)
        self.num_collectives += 1

    def _grp(self, which):
        return {"world": dist.group.WORLD if self.distributed else None,
                "trainer": self.trainer_group, "intertrainer": self.intertrainer_group,
                "row": self.grid_row_group, "col": self.grid_col_group}.get(which, which)

    def allreduce(self, t: torch.Tensor, group="trainer", op="sum", async_op=False):
        g = self._grp(group)
        if not self.distributed or g is None:
            return None
        ops = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN,
               "prod": dist.ReduceOp.PRODUCT}
        self._count(t, dist.get_world_size(g))
        return dist.all_reduce(t, ops[op], group=g, async_op=async_op)

    def broadcast(self, t: torch.Tensor, root_in_group: int = 0, group="trainer"):
        g = self._grp(group)
        if not self.distributed or g is None:
            return
        self._count(t, dist.get_world_size(g))
        dist.broadcast(t, dist.get_global_rank(g, root_in_group), group=g)

    def trainer_broadcast(self, t, root=0):
        self.broadcast(t, root, "trainer")

    def all_gather(self, t: torch.Tensor, group="trainer") -> List[torch.Tensor]:
        g = self._grp(group)
        if not self.distributed or g is None:
            return [t]
        n = dist.get_world_size(g)
        out = [torch.empty_like(t) for _ in range(n)]
        self._count(t, n)
        dist.all_gather(out, t, group=g)
        return out

    def reduce_scatter(self, out: torch.Tensor, inp: torch.Tensor, group="trainer"):
        g = self._grp(group)
        if not self.distributed or g is None:
            out.copy_(inp.reshape(out.shape))
            return
        self._count(inp, dist.get_world_size(g))
        dist.reduce_scatter_tensor(out, inp, group=g)

    def all_to_all(self, out: torch.Tensor, inp: torch.Tensor, group="trainer"):
        g = self._grp(group)
        if not self.distributed or g is None:
            out.copy_(inp)
            return
        self._count(inp, dist.get_world_size(g))
        dist.all_to_all_single(out, inp, group=g)

    def send(self, t, dst_world_rank):
        self.bytes_sent += t.numel() * t.element_size()
        dist.send(t, dst_world_rank)

    def recv(self, t, src_world_rank):
        self.bytes_received += t.numel() * t.element_size()
        dist.recv(t, src_world_rank)

    def sendrecv(self, send_t, recv_t, peer_world_rank):
        """Pairwise exchange with ``peer`` (both sides call with each other's rank)."""
        if peer_world_rank == self.rank_in_world:
            recv_t.copy_(send_t)
            return
        ops = [dist.P2POp(dist.isend, send_t, peer_world_rank),
               dist.P2POp(dist.irecv, recv_t, peer_world_rank)]
        for r in dist.batch_isend_irecv(ops):
            r.wait()
        n = send_t.numel() * send_t.element_size()
        self.bytes_sent += n
        self.bytes_received += n

    def barrier(self, group="world"):
        g = self._grp(group)
        self.num_barriers += 1
        if self.distributed and g is not None:
            dist.barrier(group=g)

    def trainer_barrier(self):
        self.barrier("trainer")

    def intertrainer_barrier(self):
        self.barrier("intertrainer")

    def global_barrier(self):
        self.barrier("world")

    # ---------------------------------------------------------------- python objects
    def gather_object(self, obj, group="trainer"):
        g = self._grp(group)
        if not self.distributed or g is None:
            return [obj]
        out = [None] * dist.get_world_size(g)
        dist.all_gather_object(out, obj, group=g)
        return out

    def trainer_gather_object(self, obj):
        return self.gather_object(obj, "trainer")

    def intertrainer_gather_object(self, obj):
        if self.num_trainers == 1:
            return [obj]
        return self.gather_object(obj, "intertrainer")

    def world_gather_object(self, obj):
        return self.gather_object(obj, "world")

    def broadcast_object(self, obj, root_in_group=0, group="trainer"):
        g = self._grp(group)
        if not self.distributed or g is None:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, dist.get_global_rank(g, root_in_group), group=g)
        return box[0]

    def reset_stats(self):
        self.bytes_sent = self.bytes_received = self.num_barriers = self.num_collectives = 0

    def finalize(self):
        if self.distributed and dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass
