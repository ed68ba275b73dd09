"""K-FAC: Kronecker-factored approximate curvature preconditioning around SGD.

For every fully-connected, channelwise fully-connected and convolution layer with an
optimizer the algorithm keeps running averages of the two Kronecker factors

    A = E[a a^T]  (layer inputs; unfolded patches for convolutions)
    G = E[g g^T]  (gradients w.r.t. the layer outputs, rescaled to per-sample values)

and replaces the weight gradient dW by  (G + pi^-1 sqrt(damping_err) I)^-1 dW
(A + pi sqrt(damping_act) I)^-1  before the first-order optimizer step (Martens and
Grosse 2015; the reference: src/execution_algorithms/kfac.cpp:122-860 and
src/execution_algorithms/kfac/kfac_block_fc_conv.cpp).  Factors are averaged over the
data-parallel ranks; inverses are recomputed every ``update_interval`` steps with a
Cholesky solve (``torch.linalg``; not a hot path) or, with ``use_eigen_decomposition``,
from the eigen-decompositions of both factors.

Batch-norm layers get the reference's dense block (kfac_block_bn.cpp): the Fisher matrix of
the stacked (scale, bias) gradient, F = E_n[g_n g_n^T] with g_n = [sum_x dy x_hat ; sum_x dy]
per sample, damped with ``damping_bn_err`` and inverted like the other factors.

With ``distribute_precondition_compute`` (or ``inverse_strategy: "each"``) block i is
inverted by data-parallel rank i mod P only and the inverses travel to the others (the
reference spreads inverses over ranks the same way, kfac.cpp:480-620).

Asynchronous inverses (``--trainer_enable_subgrid_async_comm``, the reference's switch for its
secondary grid, kfac.cpp:283-390,1109-1180: ranks set aside for the inversions hand their
results to the training ranks one step late).  Here no GPU is set aside: at a refresh step the
owner of a block starts the inversion of the current factors beside the training step (a side
CUDA stream on a GPU, a worker thread on the host), the step itself preconditions with the
inverses it already has, and the NEXT K-FAC step waits for the job, exchanges the result and
installs it.  Every rank installs at the same step, so the ranks stay identical; only a
block's very first inversion is synchronous.

GRU layers (kfac_block_gru.cpp): per stacked layer and per product (input -> gates, hidden ->
gates) one activation factor over samples x time steps and one error factor per gate; see
``_precondition_gru``.
"""
from __future__ import annotations

import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List

import torch
import torch.nn.functional as F

from .algorithms import SGDTrainingAlgorithm, Termination


def _floats(s, default):
    vals = [float(v) for v in str(s).split()] if s else []
    return vals or [default]


class _Block:
    """Factor state of one layer."""

    def __init__(self, layer):
        self.layer = layer
        self.A = self.G = self.Ainv = self.Ginv = None
        self.inp = self.out = self.grad_out = None
        self.hook = None

    # inputs as a [rows, features] matrix (bias handled by an appended column of ones)
    def activations(self) -> torch.Tensor:
        l, x = self.layer, self.inp.detach().float()
        if l.type == "convolution":
            nd = l.nd
            if nd == 2:
                cols = F.unfold(x, l.ksize, dilation=l.dil, padding=l.pad, stride=l.stride)
                a = cols.transpose(1, 2).reshape(-1, cols.shape[1])
            else:       # 3-D: patches through a direct gather (small problems only)
                xp = F.pad(self.inp.detach().float(), [p for q in reversed(l.pad) for p in (q, q)])
                u = xp.unfold(2, l.ksize[0], l.stride[0]).unfold(3, l.ksize[1], l.stride[1])
                u = u.unfold(4, l.ksize[2], l.stride[2])
                a = u.permute(0, 2, 3, 4, 1, 5, 6, 7).reshape(-1, l.cin * l.ksize[0] * l.ksize[1] * l.ksize[2])
        elif l.type == "channelwise_fully_connected":
            a = x.reshape(-1, l.in_size)
        else:
            a = x.reshape(x.shape[0], -1)
        if l.b is not None:
            a = torch.cat([a, torch.ones(a.shape[0], 1, device=a.device)], 1)
        return a

    def bn_sample_gradients(self, batch: int) -> torch.Tensor:
        """[samples, 2C]: every sample's gradient of (scale, bias)."""
        l = self.layer
        x, g = self.inp.detach().float(), self.grad_out.detach().float() * batch
        dims = [0] + list(range(2, x.dim()))
        mean = x.mean(dims, keepdim=True)
        count = x.numel() // x.shape[1]
        var = x.var(dims, unbiased=bool(getattr(l, "bessel", False)) and count > 1, keepdim=True)
        xhat = (x - mean) / torch.sqrt(var + l.eps)
        sp = list(range(2, x.dim()))
        d_scale = (g * xhat).sum(sp) if sp else g * xhat
        d_bias = g.sum(sp) if sp else g
        return torch.cat([d_scale, d_bias], 1)

    def errors(self, batch: int) -> torch.Tensor:
        l, g = self.layer, self.grad_out.detach().float()
        if l.type == "convolution":
            g = g.reshape(g.shape[0], g.shape[1], -1).transpose(1, 2).reshape(-1, g.shape[1])
        elif l.type == "channelwise_fully_connected":
            g = g.reshape(-1, l.out_size)
        else:
            g = g.reshape(g.shape[0], -1)
        return g * batch       # the objective is a mean over the mini-batch


class KFAC(SGDTrainingAlgorithm):
    def __init__(self, name, sgd: SGDTrainingAlgorithm, msg):
        super().__init__(name, sgd.termination, sgd.suppress_timer)
        self.damping_act = _floats(msg.damping_act, 1e-2)
        self.damping_err = _floats(msg.damping_err, 1e-2)
        self.damping_warmup_steps = int(msg.damping_warmup_steps) or 0
        self.decay = float(msg.kronecker_decay) or 0.99
        self.use_pi = bool(msg.use_pi)
        iv = [int(v) for v in str(msg.update_intervals).split()] if msg.update_intervals else [1]
        self.update_intervals = iv
        self.update_interval_steps = int(msg.update_interval_steps) or 1
        self.compute_interval = int(msg.compute_interval) or 1
        self.disable_layers = set(str(msg.disable_layers).split()) if msg.disable_layers else set()
        self.lr_factor = float(msg.learning_rate_factor) or 1.0
        self.lr_factor_gru = float(msg.learning_rate_factor_gru) or self.lr_factor
        # "a b c": plain SGD in epochs [0, a), K-FAC in [a, b), SGD in [b, c), K-FAC afterwards
        # (factors keep being updated; only the preconditioned gradient is not applied)
        self.use_epochs = self._parse_use_interval(str(msg.kfac_use_interval or ""))
        self.print_time = bool(msg.print_time)
        self.print_matrix_summary = bool(msg.print_matrix_summary) or bool(msg.print_matrix)
        self.damping_bn_act = _floats(msg.damping_bn_act, self.damping_act[0])
        self.damping_bn_err = _floats(msg.damping_bn_err, self.damping_err[0])
        self.use_eigen = bool(msg.use_eigen_decomposition)
        self.distribute = bool(msg.distribute_precondition_compute) or \
            str(msg.inverse_strategy).lower() in ("each", "root")
        self.root_only = str(msg.inverse_strategy).lower() == "root"
        self.inverses_computed = 0          # on this rank (tests read it)
        self.blocks: Dict[str, _Block] = {}
        from ..utils import options as _opts
        self.async_inverses = _opts.current().get_bool("trainer_enable_subgrid_async_comm")
        self._pending: Dict[object, tuple] = {}     # block key -> job started at the last refresh
        self._pool = None
        self._side = None
        self.async_installs = 0             # inverses that arrived one step late (tests read it)

    # ---------------------------------------------------------------- schedules
    @staticmethod
    def _parse_use_interval(s: str) -> List[bool]:
        marks = [int(v) for v in s.split()]
        flags, use = [], False
        for epoch in range(marks[-1] if marks else 0):
            if epoch in marks:
                use = not use
            flags.append(use)
        return flags

    def _applies(self, epoch: int) -> bool:
        return self.use_epochs[epoch] if epoch < len(self.use_epochs) else True

    def _damping(self, vals: List[float], step: int) -> float:
        if len(vals) == 1 or self.damping_warmup_steps <= 0:
            return vals[0]
        t = min(1.0, step / self.damping_warmup_steps)
        return vals[0] * (1 - t) + vals[1] * t

    def _update_interval(self, step: int) -> int:
        if len(self.update_intervals) == 1:
            return max(1, self.update_intervals[0])
        t = min(1.0, step / max(1, self.update_interval_steps))
        return max(1, int(round(self.update_intervals[0] * (1 - t) + self.update_intervals[1] * t)))

    # ---------------------------------------------------------------- set-up
    def _setup(self, model):
        for l in model.layers:
            l.fuse_pool_layer = None          # the blocks need every layer's own output
            if l.type == "batch_normalization":
                if l.name not in self.disable_layers and l.scale.has_optimizer() and l.bias.has_optimizer() \
                        and not getattr(l, "fused_into_parent", False):
                    self.blocks[l.name] = _Block(l)
                continue
            if l.type == "gru":
                if l.name not in self.disable_layers and all(w.has_optimizer() for grp in l.ws for w in grp):
                    l.kfac_capture = True
                    self.blocks[l.name] = _Block(l)
                continue
            if l.type not in ("fully_connected", "channelwise_fully_connected", "convolution"):
                continue
            if l.name in self.disable_layers or not l.w.has_optimizer():
                continue
            if getattr(l, "transpose", False) or getattr(l, "groups", 1) != 1:
                continue
            self.blocks[l.name] = _Block(l)

    def _capture(self, model):
        """Remember every block's input and hook its output for the error signal."""
        for name, blk in self.blocks.items():
            l = blk.layer
            parent = l.parents[0]
            blk.inp = model.acts[parent.name][model._slot(parent, l)]
            out = model.acts[name][0]
            blk.out = out
            if out.requires_grad:
                out.register_hook(lambda g, b=blk: setattr(b, "grad_out", g))

    # ---------------------------------------------------------------- the step
    def train_mini_batch(self, trainer, model, ctx, batch, cbs):
        if not self.blocks and not getattr(self, "_ready", False):
            self._ready = True
            self._setup(model)
        for cb in cbs:
            if ctx.step % cb.batch_interval == 0:
                cb.on_batch_begin(model)
        model.clear_gradients()
        model.forward_prop(batch.tensors, "training", batch.global_size, batch.offset)
        self._capture(model)
        obj = model.local_objective()
        model.last_objective = obj.detach()
        model.record_statistics("training", obj)
        model.backward_prop(obj)
        if ctx.step % self.compute_interval == 0:
            self._apply = self._applies(ctx.epoch)
            t0 = time.perf_counter() if self.print_time else 0.0
            self._precondition(model, ctx.step, batch.global_size)
            if self.print_time and trainer.comm.rank_in_trainer == 0:
                if model.device.type == "cuda":
                    torch.cuda.synchronize()
                print(f"K-FAC step {ctx.step}: preconditioning {1e3 * (time.perf_counter() - t0):.3f} ms"
                      f"{'' if self._apply else ' (factors only)'}", flush=True)
        model.update_weights()
        ctx.step += 1
        ctx.step_in_epoch += 1
        for cb in cbs:
            if (ctx.step - 1) % cb.batch_interval == 0:
                cb.on_batch_end(model)

    def _invert(self, M: torch.Tensor, damping: float) -> torch.Tensor:
        eye = torch.eye(M.shape[0], device=M.device)
        self.inverses_computed += 1
        if self.use_eigen:
            w, V = torch.linalg.eigh(M)
            return (V / (w.clamp_min(0.0) + damping)) @ V.t()
        return torch.cholesky_inverse(torch.linalg.cholesky(M + damping * eye))

    def _inverses(self, par, index: int, mats, dampings):
        """Inverses of ``mats``; with the distributed strategy one rank computes them and the
        others receive (a sum over the ranks in which only the owner's term is non-zero)."""
        if not self.distribute or par is None or par.dp_size <= 1:
            return [self._invert(M, d) for M, d in zip(mats, dampings)]
        owner = 0 if self.root_only else index % par.dp_size
        mine = par.dp_rank == owner
        out = []
        for M, d in zip(mats, dampings):
            inv = self._invert(M, d) if mine else torch.zeros_like(M)
            par.allreduce_sum_inplace(inv)
            out.append(inv)
        return out

    # ---------------------------------------------------------------- asynchronous inverses
    def _start_job(self, par, index: int, mats, dampings):
        """Start the inversion of ``mats`` beside the training step; returns the job."""
        distributed = self.distribute and par is not None and par.dp_size > 1
        owner = 0 if (self.root_only or not distributed) else index % par.dp_size
        mine = (not distributed) or par.dp_rank == owner
        mats = [M.clone() for M in mats]
        if not mine:
            return ("none", mats, None, distributed)
        if mats[0].is_cuda:
            if self._side is None:
                self._side = torch.cuda.Stream()
            side, cur = self._side, torch.cuda.current_stream()
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                out = [self._invert(M, d) for M, d in zip(mats, dampings)]
                for t in mats + out:
                    t.record_stream(side)
            ev = torch.cuda.Event()
            ev.record(side)
            return ("stream", mats, (out, ev), distributed)
        if self._pool is None:
            self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="kfac-inverse")
        fut = self._pool.submit(lambda: [self._invert(M, d) for M, d in zip(mats, dampings)])
        return ("thread", mats, fut, distributed)

    def _finish_job(self, par, job):
        kind, mats, handle, distributed = job
        if kind == "none":
            out = [torch.zeros_like(M) for M in mats]
        elif kind == "stream":
            out, ev = handle
            cur = torch.cuda.current_stream()
            cur.wait_event(ev)
            for t in out:                  # allocated on the side stream, used on this one from now on
                t.record_stream(cur)
        else:
            out = handle.result()
        if distributed:
            for inv in out:
                par.allreduce_sum_inplace(inv)
        self.async_installs += len(out)
        return out

    def _refresh(self, key, have, refresh: bool, par, index: int, mats, dampings):
        """The inverses to precondition with at this step.  ``have``: the installed ones (None
        before the first inversion)."""
        if not self.async_inverses:
            return self._inverses(par, index, mats, dampings) if (refresh or have is None) else have
        job = self._pending.pop(key, None)
        if job is not None:
            have = self._finish_job(par, job)
        if have is None:
            return self._inverses(par, index, mats, dampings)
        if refresh:
            self._pending[key] = self._start_job(par, index, mats, dampings)
        return have

    def shutdown(self):
        for job in self._pending.values():
            if job[0] == "thread":
                job[2].result()
        self._pending.clear()
        if self._pool is not None:
            self._pool.shutdown(wait=True)
            self._pool = None

    def _precondition_gru(self, blk, par, dp, index, global_batch, refresh, d_act, d_err):
        """GRU block (src/execution_algorithms/kfac/kfac_block_gru.cpp): for every stacked
        layer and each of its two products (input -> gates, hidden -> gates) one activation
        factor A over (samples x time steps) of [input | 1] resp. [previous hidden | 1], and one
        error factor G per gate (reset, update, new) from the gradient at that gate's
        pre-activation; the gate's rows of the matrix and bias become G^-1 [dW | db] A^-1."""
        l = blk.layer
        H = l.hidden
        caches = getattr(l, "kfac_cache", None) or []
        if blk.A is None:
            blk.A, blk.G, blk.Ainv, blk.Ginv = {}, {}, {}, {}
        for li, (cap, (wih, whh, bih, bhh)) in enumerate(zip(caches, l.ws)):
            if cap["g_gi"] is None or any(g is None for g in cap["g_gh"]):
                continue
            ones = lambda a: torch.cat([a, torch.ones(a.shape[0], 1, device=a.device)], 1)   # noqa: E731
            prods = (("ih", ones(cap["x"].float().reshape(-1, cap["x"].shape[-1])),
                      cap["g_gi"].float().reshape(-1, 3 * H), wih, bih),
                     ("hh", ones(torch.stack(cap["h_prev"], 1).float().reshape(-1, H)),
                      torch.stack(cap["g_gh"], 1).float().reshape(-1, 3 * H), whh, bhh))
            for tag, a, g, W, b in prods:
                if W.handle.grad is None:
                    continue
                g = g * global_batch                       # the objective is a mean over the mini-batch
                key = (li, tag)
                A = a.t() @ a / a.shape[0]
                Gs = [g[:, k * H:(k + 1) * H].t() @ g[:, k * H:(k + 1) * H] / g.shape[0] for k in range(3)]
                if dp > 1:
                    for M in [A] + Gs:
                        par.allreduce_sum_inplace(M)
                        M /= dp
                if key not in blk.A:
                    blk.A[key], blk.G[key] = A, Gs
                else:
                    blk.A[key] = self.decay * blk.A[key] + (1 - self.decay) * A
                    blk.G[key] = [self.decay * o + (1 - self.decay) * n for o, n in zip(blk.G[key], Gs)]
                have = [blk.Ainv[key]] + list(blk.Ginv[key]) if key in blk.Ainv else None
                invs = self._refresh((l.name, key), have, refresh, par, index, [blk.A[key]] + blk.G[key],
                                     [d_act ** 0.5] + [d_err ** 0.5] * 3)
                blk.Ainv[key], blk.Ginv[key] = invs[0], invs[1:]
                gw = W.handle.grad.float().reshape(3 * H, -1)
                gb = b.handle.grad.float().reshape(3 * H, 1) if b.handle.grad is not None else \
                    torch.zeros(3 * H, 1, device=gw.device)
                full = torch.cat([gw, gb], 1)
                nat = torch.cat([blk.Ginv[key][k] @ full[k * H:(k + 1) * H] @ blk.Ainv[key] for k in range(3)], 0)
                nat = nat * self.lr_factor_gru
                if not getattr(self, "_apply", True):
                    continue
                W.handle.grad.copy_(nat[:, :-1].reshape(W.handle.grad.shape))
                if b.handle.grad is not None:
                    b.handle.grad.copy_(nat[:, -1].reshape(b.handle.grad.shape))

    def _summary(self, name: str, **mats):
        """``print_matrix_summary``: size, mean and extreme values of a block's factors and
        inverses (kfac_util.cpp prints the same figures)."""
        if not self.print_matrix_summary:
            return
        parts = [f"{k} {tuple(M.shape)} mean {float(M.mean()):.3e} min {float(M.min()):.3e} "
                 f"max {float(M.max()):.3e}" for k, M in mats.items() if M is not None]
        print(f"K-FAC {name}: " + "; ".join(parts), flush=True)

    @torch.no_grad()
    def _precondition(self, model, step: int, global_batch: int):
        d_act = self._damping(self.damping_act, step)
        d_err = self._damping(self.damping_err, step)
        d_bn = self._damping(self.damping_bn_err, step)
        refresh = step % self._update_interval(step) == 0
        par = model.parallel
        dp = par.dp_size if par is not None else 1
        for index, blk in enumerate(self.blocks.values()):
            l = blk.layer
            if blk.grad_out is None:
                continue
            if l.type == "gru":
                self._precondition_gru(blk, par, dp, index, global_batch, refresh, d_act, d_err)
                blk.grad_out = None
                continue
            if l.type == "batch_normalization":
                if l.scale.handle.grad is None or l.bias.handle.grad is None:
                    continue
                gs = blk.bn_sample_gradients(global_batch)
                Fm = gs.t() @ gs / gs.shape[0]
                if dp > 1:
                    par.allreduce_sum_inplace(Fm)
                    Fm /= dp
                blk.G = Fm if blk.G is None else self.decay * blk.G + (1 - self.decay) * Fm
                (blk.Ginv,) = self._refresh(l.name, None if blk.Ginv is None else [blk.Ginv], refresh, par,
                                            index, [blk.G], [d_bn])
                c = l.scale.handle.grad.numel()
                g = torch.cat([l.scale.handle.grad.float().reshape(-1), l.bias.handle.grad.float().reshape(-1)])
                nat = blk.Ginv @ g * self.lr_factor
                if getattr(self, "_apply", True):
                    l.scale.handle.grad.copy_(nat[:c].reshape(l.scale.handle.grad.shape))
                    l.bias.handle.grad.copy_(nat[c:].reshape(l.bias.handle.grad.shape))
                self._summary(l.name, G=blk.G, Ginv=blk.Ginv)
                blk.grad_out = None
                continue
            if l.w.handle.grad is None:
                continue
            a = blk.activations()
            g = blk.errors(global_batch)
            A = a.t() @ a / a.shape[0]
            G = g.t() @ g / g.shape[0]
            if dp > 1:
                par.allreduce_sum_inplace(A)
                par.allreduce_sum_inplace(G)
                A /= dp
                G /= dp
            blk.A = A if blk.A is None else self.decay * blk.A + (1 - self.decay) * A
            blk.G = G if blk.G is None else self.decay * blk.G + (1 - self.decay) * G
            pi = 1.0
            if self.use_pi and (refresh or blk.Ainv is None):
                pi = float(torch.sqrt((blk.A.trace() / blk.A.shape[0]) /
                                      (blk.G.trace() / blk.G.shape[0]).clamp_min(1e-30)).clamp(1e-3, 1e3))
            blk.Ainv, blk.Ginv = self._refresh(l.name, None if blk.Ainv is None else [blk.Ainv, blk.Ginv],
                                               refresh, par, index, [blk.A, blk.G],
                                               [pi * d_act ** 0.5, d_err ** 0.5 / pi])
            gw = l.w.handle.grad.float().reshape(blk.G.shape[0], -1)
            if l.b is not None and l.b.handle.grad is not None:
                gw = torch.cat([gw, l.b.handle.grad.float().reshape(-1, 1)], 1)
            # (the patch matrix is ordered (channel, kernel...) like the kernel's trailing dims)
            nat = blk.Ginv @ gw @ blk.Ainv * self.lr_factor
            self._summary(l.name, A=blk.A, G=blk.G, Ainv=blk.Ainv, Ginv=blk.Ginv)
            blk.grad_out = None
            if not getattr(self, "_apply", True):
                continue
            if l.b is not None and l.b.handle.grad is not None:
                l.b.handle.grad.copy_(nat[:, -1].reshape(l.b.handle.grad.shape))
                nat = nat[:, :-1]
            l.w.handle.grad.copy_(nat.reshape(l.w.handle.grad.shape))
