"""Worker run under torch.distributed.run by the multi-rank tests (CPU ranks over gloo, or
one GPU per rank when CUDA is available and LBANN_TEST_DEVICE=cuda)."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import lbann_b200 as lbann  # noqa: E402
from lbann_b200.exec.trainer import ExecTrainer  # noqa: E402
from lbann_b200.models.cosmoflow import construct_cosmoflow_model, synthetic_reader  # noqa: E402
from lbann_b200.utils import options as opts  # noqa: E402


def cosmoflow(depth_groups, steps, dtype, width=32, channels=(8, 16, 16), graph=False):
    o = opts.reset()
    o.set("default_dtype", dtype)
    if os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cpu":
        o.set("disable_cuda", True)
    if graph:
        o.set("use_cuda_graph", True)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    height_groups = int(os.environ.get("LBANN_TEST_HEIGHT_GROUPS", "1"))
    width_groups = int(os.environ.get("LBANN_TEST_WIDTH_GROUPS", "1"))
    ps = lbann.get_parallel_strategy_args(depth_groups=depth_groups, height_groups=height_groups,
                                          width_groups=width_groups) \
        if depth_groups * height_groups * width_groups > 1 else None
    model = construct_cosmoflow_model(width, 4, 4, num_epochs=1, channels=tuple(channels), pool_mode="max",
                                      conv_bias=False, fc_sizes=(32, 16), parallel_strategy=ps)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=int(os.environ.get("LBANN_TEST_MINI_BATCH", "4")), random_seed=5),
        model=model, data_reader=synthetic_reader(16, width, 4, 4),
        optimizer=lbann.SGD(learn_rate=float(os.environ.get("LBANN_TEST_LR", "0.01")), momentum=0.9))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    losses = []
    dc = tr.data_coordinator
    dc.start_epoch("training")
    for _ in range(steps):
        b = dc.next_batch("training")
        if b is None:                       # end of the epoch: the next one reshuffles nothing
            dc.start_epoch("training")
            b = dc.next_batch("training")
        m.train_step(b.tensors, b.global_size)
        v = m.last_objective.detach().float().reshape(1).clone()
        if tr.parallel is not None:
            tr.comm.allreduce(v, "trainer", "sum")
        losses.append(float(v))
    w = {x.name: float(x.values.detach().float().norm()) for x in m.weights}
    res = {"losses": losses, "weight_norms": w, "world": world}
    if tr.distconv is not None:
        res["interior_copies"] = tr.distconv.interior_copies
        res["halo_bytes"] = tr.distconv.halo_bytes
        res["halo_tensors"] = len(tr.distconv._halo_tensors)
    if torch.cuda.is_available() and os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cuda":
        from lbann_b200.ops import native
        torch.cuda.synchronize()
        res["status"] = native.consume_status(False)
        res["launches"] = native.launches()
        res["sharded_update"] = m.arena.shard is not None
        res["graph"] = bool(getattr(m, "_graph_mode", False))
    tr.shutdown()
    return res


def unet(depth_groups, height_groups, steps, volume=16, base=4, levels=2):
    """Small 3-D U-Net (convolution + batch norm + ReLU, max pooling, 2x up-convolutions,
    skip concatenations, per-voxel softmax cross-entropy) on a depth x height grid."""
    from lbann_b200.models import construct_unet3d_model
    o = opts.reset()
    o.set("default_dtype", "float")
    if os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cpu":
        o.set("disable_cuda", True)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ps = lbann.get_parallel_strategy_args(depth_groups=depth_groups, height_groups=height_groups) \
        if depth_groups * height_groups > 1 else None
    model = construct_unet3d_model(num_classes=3, base_channels=base, levels=levels, parallel_strategy=ps)
    v = volume
    r = lbann.reader_pb2.Reader()
    r.name, r.role, r.shuffle, r.fraction_of_data_to_use = "synthetic", "train", False, 1.0
    r.synth_dimensions = f"1 {v} {v} {v}"
    r.synth_response_dimensions = f"{v} {v} {v}"
    r.synth_distribution = "samples:normal responses:randint:3"
    r.num_samples = 4
    r.synth_pool_size = 4
    dr = lbann.reader_pb2.DataReader()
    dr.reader.append(r)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=2, random_seed=3), model=model, data_reader=dr,
        optimizer=lbann.SGD(learn_rate=float(os.environ.get("LBANN_TEST_LR", "1e-5")), momentum=0.9))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    losses = []
    dc = tr.data_coordinator
    dc.start_epoch("training")
    for _ in range(steps):
        b = dc.next_batch("training")
        if b is None:
            dc.start_epoch("training")
            b = dc.next_batch("training")
        m.train_step(b.tensors, b.global_size)
        losses.append(float(m.last_objective.detach().float()))
    w = {x.name: float(x.values.detach().float().norm()) for x in m.weights}
    res = {"losses": losses, "weight_norms": w, "world": world,
           "halo_bytes": tr.distconv.halo_bytes if tr.distconv is not None else 0}
    tr.shutdown()
    return res


def comm_kernels():
    """Device collectives of parallel/symm.py against closed-form expectations."""
    from lbann_b200.ops import native
    from lbann_b200.parallel.comm import LbannComm
    from lbann_b200.parallel.symm import SymmetricGroup
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    comm = LbannComm(device=dev)
    g = SymmetricGroup(dev, pg=comm.trainer_group)
    P = g.world
    res = {"world": P, "native": g.native}
    n = 3 * 1024 * 1024 + 37
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        buf = g.alloc(n * 4)
        t = buf.view(dt, n)
        base = torch.arange(n, device=dev, dtype=torch.float32) % 97 / 97.0
        t.copy_((base + rank).to(dt))
        g.barrier_host()
        g.allreduce_(buf, dt, n, scale=0.5)
        torch.cuda.synchronize()
        expect = 0.5 * (P * base + sum(range(P)))
        res[f"allreduce_{dt}"] = float((t.float() - expect).abs().max()) <= tol * P * 2
    v = torch.arange(100, device=dev, dtype=torch.float32) + rank
    g.allreduce_small_(v, "sum")
    m = torch.full((5,), float(rank), device=dev)
    g.allreduce_small_(m, "max")
    torch.cuda.synchronize()
    res["one_shot_sum"] = bool(torch.allclose(v, P * torch.arange(100, device=dev, dtype=torch.float32) + sum(range(P))))
    res["one_shot_max"] = bool((m == P - 1).all())
    # neighbour put + barrier
    rows, rb = 4, 256
    buf = g.alloc(P * rows * rb)
    src = torch.full((rows, rb), rank + 1, dtype=torch.uint8, device=dev)
    g.barrier_host()
    g.put_rows(src, buf, (rank + 1) % P, rank * rows * rb, rows, rb, rb, rb)
    g.barrier_device(3)
    torch.cuda.synchronize()
    got = buf.local.view(P, rows * rb)[(rank - 1) % P]
    res["put_rows"] = bool((got == ((rank - 1) % P) + 1).all())
    res["status"] = native.consume_status(False)
    oks = comm.world_gather_object({k: v for k, v in res.items() if k not in ("world", "native")})
    res["all_ranks_ok"] = all(all(bool(x) if k != "status" else x == 0 for k, x in o.items()) for o in oks)
    return res


def fused_gemm():
    """All-gather -> GEMM and GEMM -> reduce-scatter against fp32 references."""
    from lbann_b200.ops import native
    from lbann_b200.parallel.comm import LbannComm
    from lbann_b200.parallel.fused import FusedGemm
    from lbann_b200.parallel.symm import SymmetricGroup
    rank = int(os.environ.get("RANK", "0"))
    use_cuda = os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cuda"
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
    comm = LbannComm(device=dev)
    g = SymmetricGroup(dev, pg=comm.trainer_group)
    P = g.world
    fg = FusedGemm(g)
    dt = torch.bfloat16
    res = {"world": P, "native": g.native}
    gen = torch.Generator().manual_seed(1234)
    rows, K, N = (256, 512, 384) if use_cuda else (16, 32, 24)
    X = torch.randn(P * rows, K, generator=gen).to(dt)         # the same on every rank
    W = torch.randn(N, K, generator=gen).to(dt)
    # --- left operand sharded by rows
    buf = g.alloc(rows * K * 2)
    buf.view(dt, rows * K).view(rows, K).copy_(X[rank * rows:(rank + 1) * rows])
    y = fg.allgather_gemm(buf, rows, K, W.to(dev), sharded="a", dtype=dt, out_dtype=torch.float32)
    ref = X.float() @ W.float().t()
    res["ag_a"] = bool(torch.allclose(y.cpu(), ref, rtol=2e-2, atol=2e-1))
    for rep in range(2):     # staged through copying CTAs; twice: the flags carry epochs
        y = fg.allgather_gemm(buf, rows, K, W.to(dev), sharded="a", dtype=dt, out_dtype=torch.float32,
                              staged=True)
        res[f"ag_a_staged{rep}"] = bool(torch.allclose(y.cpu(), ref, rtol=2e-2, atol=2e-1))
    # --- right operand (weights) sharded by rows
    wrows = N // P if (N // P) % (64 if use_cuda else 1) == 0 else N
    if use_cuda:
        wrows = 128
    Wf = torch.randn(P * wrows, K, generator=gen).to(dt)
    wbuf = g.alloc(wrows * K * 2)
    wbuf.view(dt, wrows * K).view(wrows, K).copy_(Wf[rank * wrows:(rank + 1) * wrows])
    xin = torch.randn(160 if use_cuda else 8, K, generator=gen).to(dt)
    y2 = fg.allgather_gemm(wbuf, wrows, K, xin.to(dev), sharded="b", dtype=dt, out_dtype=torch.float32)
    res["ag_b"] = bool(torch.allclose(y2.cpu(), xin.float() @ Wf.float().t(), rtol=2e-2, atol=2e-1))
    y2 = fg.allgather_gemm(wbuf, wrows, K, xin.to(dev), sharded="b", dtype=dt, out_dtype=torch.float32,
                           staged=True)
    res["ag_b_staged"] = bool(torch.allclose(y2.cpu(), xin.float() @ Wf.float().t(), rtol=2e-2, atol=2e-1))
    # --- K-sliced product, result scattered by rows
    M2, N2, Kl = (P * 128, 320, 256) if use_cuda else (P * 4, 12, 16)
    A = torch.randn(M2, P * Kl, generator=gen).to(dt)
    B = torch.randn(N2, P * Kl, generator=gen).to(dt)
    obuf = g.alloc((M2 // P) * N2 * 4)
    a_loc = A[:, rank * Kl:(rank + 1) * Kl].contiguous().to(dev)
    b_loc = B[:, rank * Kl:(rank + 1) * Kl].contiguous().to(dev)
    mine = fg.gemm_reduce_scatter(a_loc, b_loc, obuf, M2 // P)
    full = A.float() @ B.float().t()
    want = full[rank * (M2 // P):(rank + 1) * (M2 // P)]
    res["rs"] = bool(torch.allclose(mine.cpu(), want, rtol=2e-2, atol=5e-1))
    # transposed operands (weight-gradient form: dW = dY^T . X over the sample slices)
    mine2 = fg.gemm_reduce_scatter(a_loc.t().contiguous(), b_loc.t().contiguous(), obuf, M2 // P,
                                   trans_a=True, trans_b=True)
    res["rs_t"] = bool(torch.allclose(mine2.cpu(), want, rtol=2e-2, atol=5e-1))
    if use_cuda:
        torch.cuda.synchronize()
        res["status"] = native.consume_status(False)
    oks = comm.world_gather_object({k: v for k, v in res.items() if k not in ("world", "native")})
    res["all_ranks_ok"] = all(all(bool(x) if k != "status" else x == 0 for k, x in o.items()) for o in oks)
    return res


def tensor_parallel():
    """Column/row-parallel and sharded (FSDP) linear layers against dense autograd."""
    from lbann_b200.parallel.comm import LbannComm
    from lbann_b200.parallel.symm import SymmetricGroup
    from lbann_b200.parallel.tensor_parallel import (ColumnParallelLinear, RowParallelLinear,
                                                     ShardedLinear)
    rank = int(os.environ.get("RANK", "0"))
    use_cuda = os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cuda"
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
    comm = LbannComm(device=dev)
    g = SymmetricGroup(dev, pg=comm.trainer_group)
    P = g.world
    dt = torch.bfloat16 if use_cuda else torch.float32
    tol = dict(rtol=3e-2, atol=3e-1) if use_cuda else dict(rtol=1e-4, atol=1e-4)
    gen = torch.Generator().manual_seed(7)
    T, D, F = (P * 128, 256, P * 256) if use_cuda else (P * 4, 8, P * 6)
    X = torch.randn(T, D, generator=gen).to(dt)
    W1 = (torch.randn(F, D, generator=gen) / D ** 0.5).to(dt)
    W2 = (torch.randn(D, F, generator=gen) / F ** 0.5).to(dt)
    DY = torch.randn(T, D, generator=gen).to(dt)
    # dense reference (fp32 autograd)
    xr, w1r, w2r = (t.float().clone().detach().requires_grad_(True) for t in (X, W1, W2))
    yr = (xr @ w1r.t()) @ w2r.t()
    yr.backward(DY.float())
    res = {"world": P}
    rows, fl = T // P, F // P
    x = X[rank * rows:(rank + 1) * rows].to(dev).clone().detach().requires_grad_(True)
    w1 = W1[rank * fl:(rank + 1) * fl].to(dev).clone().detach().requires_grad_(True)   # output rows
    w2 = W2[:, rank * fl:(rank + 1) * fl].contiguous().to(dev).clone().detach().requires_grad_(True)   # input columns
    col, row = ColumnParallelLinear(g), RowParallelLinear(g)
    h = col(x, w1)                    # [T, F/P]
    y = row(h, w2)                    # [T/P, D]
    y.backward(DY[rank * rows:(rank + 1) * rows].to(dev))
    sl = slice(rank * rows, (rank + 1) * rows)
    res["tp_fwd"] = bool(torch.allclose(y.detach().float().cpu(), yr[sl].detach(), **tol))
    res["tp_dx"] = bool(torch.allclose(x.grad.float().cpu(), xr.grad[sl], **tol))
    res["tp_dw1"] = bool(torch.allclose(w1.grad.float().cpu(), w1r.grad[rank * fl:(rank + 1) * fl], **tol))
    res["tp_dw2"] = bool(torch.allclose(w2.grad.float().cpu(), w2r.grad[:, rank * fl:(rank + 1) * fl], **tol))
    # sharded weights, data-parallel activations: every rank has its own tokens
    Xs = torch.randn(P, rows, D, generator=gen).to(dt)
    DYs = torch.randn(P, rows, F, generator=gen).to(dt)
    w_master = W1[rank * fl:(rank + 1) * fl].float().to(dev).clone().detach().requires_grad_(True)
    lin = ShardedLinear(g, w_master)
    xs = Xs[rank].to(dev).clone().detach().requires_grad_(True)
    ys = lin(xs)
    ys.backward(DYs[rank].to(dev))
    wd = W1.float().clone().detach().requires_grad_(True)
    xd = Xs.float().clone().detach().requires_grad_(True)
    yd = xd @ wd.t()
    yd.backward(DYs.float())
    res["fsdp_fwd"] = bool(torch.allclose(ys.detach().float().cpu(), yd[rank].detach(), **tol))
    res["fsdp_dx"] = bool(torch.allclose(xs.grad.float().cpu(), xd.grad[rank], **tol))
    res["fsdp_dw"] = bool(torch.allclose(w_master.grad.float().cpu(), wd.grad[rank * fl:(rank + 1) * fl], **tol))
    res["fsdp_dw_err"] = float((w_master.grad.float().cpu() - wd.grad[rank * fl:(rank + 1) * fl]).abs().max())
    if use_cuda:
        from lbann_b200.ops import native
        torch.cuda.synchronize()
        res["status"] = native.consume_status(False)
    oks = comm.world_gather_object({k: v for k, v in res.items() if k != "world"})
    res["all_ranks_ok"] = all(all((bool(x) if k != "status" else x == 0) for k, x in o.items() if not k.endswith("_err")) for o in oks)
    res["detail"] = oks
    return res


def model_parallel_fc(grid_height, steps, sharded=False):
    """MLP whose hidden layers are model-parallel over a process-grid column (or, with
    ``sharded``, whose first layer has weights flagged sharded on a data-parallel trainer)."""
    o = opts.reset()
    on_gpu = os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cuda"
    if on_gpu:
        o.set("default_dtype", "bf16")
    else:
        o.set("disable_cuda", True)
    if grid_height > 1:
        o.set("trainer_grid_height", grid_height)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n1, n2, n3, nin = (128, 64, 64, 64) if on_gpu else (24, 10, 3, 12)
    x = lbann.Input(data_field="samples")
    t = lbann.Input(data_field="responses")
    layout = "model_parallel" if not sharded else "data_parallel"
    if sharded:
        w = lbann.Weights(initializer=lbann.HeNormalInitializer(), sharded=True, name="fc1_w")
        h = lbann.Relu(lbann.FullyConnected(x, num_neurons=256, has_bias=True, weights=[w], name="fc1"))
    else:
        h = lbann.Relu(lbann.FullyConnected(x, num_neurons=n1, has_bias=True, data_layout=layout, name="fc1"))
    h = lbann.Relu(lbann.FullyConnected(h, num_neurons=n2, has_bias=True, name="fc2"))
    y = lbann.FullyConnected(h, num_neurons=n3, has_bias=False, data_layout=layout, name="fc3")
    loss = lbann.MeanSquaredError(y, t, name="mse")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x, t])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    from test_models_cpu import _reader
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=8, random_seed=11), model=model,
        data_reader=_reader(16, [nin], "normal", response_dims=[n3]),
        optimizer=lbann.SGD(learn_rate=0.05 if not on_gpu else 0.01, momentum=0.9))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    losses = []
    for _ in range(steps):
        b = dc.next_batch("training")
        if b is None:
            dc.start_epoch("training")
            b = dc.next_batch("training")
        m.train_step(b.tensors, b.global_size)
        v = m.last_objective.detach().float().reshape(1).clone()
        if tr.parallel is not None and tr.parallel.dp_size > 1:
            tr.comm.allreduce(v, "trainer", "sum")       # local objectives are partial sums
        losses.append(float(v))
    w = {x.name: float(x.values.detach().float().norm()) for x in m.weights}
    res = {"losses": losses, "weight_norms": w, "world": world}
    if tr.distconv is not None:
        res["interior_copies"] = tr.distconv.interior_copies
        res["halo_bytes"] = tr.distconv.halo_bytes
        res["halo_tensors"] = len(tr.distconv._halo_tensors)
    if torch.cuda.is_available() and os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cuda":
        from lbann_b200.ops import native
        torch.cuda.synchronize()
        res["status"] = native.consume_status(False)
        res["sharded_update"] = m.arena.shard is not None
        res["graph"] = bool(getattr(m, "_graph_mode", False))
    tr.shutdown()
    return res


def dist_embedding(steps):
    """Embedding layer with its own sparse SGD: on several ranks the table is partitioned
    (GPU ranks: one-sided row gather / gradient scatter; CPU ranks: replicated with gathered
    gradients).  Returns the losses and the trained table."""
    o = opts.reset()
    if os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cpu":
        o.set("disable_cuda", True)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    x = lbann.Input(data_field="samples")
    t = lbann.Input(data_field="responses")
    e = lbann.DistEmbedding(x, num_embeddings=21, embedding_dim=8, sparse_sgd=True, learning_rate=0.01,
                            name="table")
    y = lbann.Reduction(lbann.Reshape(e, dims=[6, 8]), mode="sum")
    loss = lbann.MeanSquaredError(lbann.Reshape(y, dims=[1]), t, name="mse")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x, t])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    from test_models_cpu import _reader
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=8, random_seed=11), model=model,
        data_reader=_reader(16, [6], "samples:randint:23 responses:normal", response_dims=[1]),
        optimizer=lbann.SGD(learn_rate=0.05))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    losses = []
    for _ in range(steps):
        b = dc.next_batch("training")
        if b is None:
            dc.start_epoch("training")
            b = dc.next_batch("training")
        m.train_step(b.tensors, b.global_size)
        v = m.last_objective.detach().float().reshape(1).clone()
        if tr.parallel is not None and tr.parallel.dp_size > 1:
            tr.comm.allreduce(v, "trainer", "sum")
        losses.append(float(v))
    if torch.cuda.is_available() and not o.get_bool("disable_cuda"):
        torch.cuda.synchronize()
    from lbann_b200.io.checkpoint import model_state
    tensors, _ = model_state(m)
    table = next(v for k, v in tensors.items() if k.endswith("/values") and v.numel() == 21 * 8)
    from lbann_b200.ops import native
    status = native.consume_status(False) if torch.cuda.is_available() and not o.get_bool("disable_cuda") else 0
    tr.shutdown()
    return {"losses": losses, "table": table.reshape(-1).tolist(), "world": world, "status": int(status)}


def data_store(preload):
    """Ranks of one trainer draw differently shuffled epochs through the data store: every
    sample is read from the reader once, later epochs are served by owner -> consumer sends."""
    import numpy as np
    import torch.distributed as dist
    from lbann_b200.data.readers import ArrayReader
    from lbann_b200.data.store import DataStore
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    n = 24
    arrays = {"samples": np.arange(n * 6, dtype=np.float32).reshape(n, 2, 3),
              "responses": -np.arange(n, dtype=np.float32).reshape(n, 1)}
    reader = ArrayReader(arrays).setup(0)
    store = DataStore(reader, rank, world, DataStore.make_group(), preload=preload)
    ok = True
    for epoch in range(3):
        order = np.random.RandomState(epoch).permutation(n)
        for pos in range(0, n, 8):
            gidx = order[pos:pos + 8]
            mine = gidx[rank::world]
            got = store.fetch_batch_global(gidx, rank, world, ["samples", "responses"])
            ok = ok and np.array_equal(got["samples"].numpy(), arrays["samples"][mine])
            ok = ok and np.array_equal(got["responses"].numpy(), arrays["responses"][mine])
    stats = [None] * world
    dist.all_gather_object(stats, dict(store.stats, ok=bool(ok), cached=len(store.cache)))
    return {"world": world, "stats": stats, "samples": n}


def ltfb(strategy):
    """Two trainers of one rank each run LTFB tournaments on an MLP regression."""
    o = opts.reset()
    if os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cpu":
        o.set("disable_cuda", True)
    o.set("procs_per_trainer", 1)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    x = lbann.Input(data_field="samples")
    t = lbann.Input(data_field="responses")
    h = lbann.Tanh(lbann.FullyConnected(x, num_neurons=12, has_bias=True, name="fc1"))
    y = lbann.FullyConnected(h, num_neurons=2, has_bias=True, name="fc2")
    loss = lbann.MeanSquaredError(y, t, name="mse")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x, t])),
                        objective_function=lbann.ObjectiveFunction([loss]),
                        metrics=[lbann.Metric(loss, name="mse")])
    RPE = lbann.RandomPairwiseExchange
    if strategy == "truncation":
        meta = lbann.TruncationSelectionExchange({"mse": RPE.MetricStrategy.LOWER_IS_BETTER}, truncation_k=1)
    else:
        meta = RPE({"mse": RPE.MetricStrategy.LOWER_IS_BETTER}, RPE.ExchangeStrategy(strategy))
    algo = lbann.LTFB("ltfb", lbann.BatchedIterativeOptimizer("local", num_iterations=3), meta,
                      metalearning_steps=3)
    from test_models_cpu import _reader
    rd = _reader(32, [6], "normal", response_dims=[2])
    r2 = rd.reader.add()
    r2.CopyFrom(rd.reader[0])
    r2.role = "tournament"
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=8, random_seed=3, training_algo=algo), model=model,
        data_reader=rd, optimizer=lbann.SGD(learn_rate=0.05 if rank == 0 else 0.0))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tr.train(m, num_epochs=1)
    w = {x.name: float(x.values.detach().float().norm()) for x in m.weights}
    allw = tr.comm.world_gather_object(w)
    tr.shutdown()
    return {"world": world, "weights": allw, "num_trainers": tr.comm.num_trainers}


def kfac_job(distribute, steps, asynchronous=0):
    """K-FAC on a small MLP with batch norm; optionally the inverses are spread over the ranks
    and computed beside the next step."""
    o = opts.reset()
    o.set("disable_cuda", True)
    if asynchronous:
        o.set("trainer_enable_subgrid_async_comm", True)
    x = lbann.Input(data_field="samples")
    t = lbann.Input(data_field="responses")
    h = lbann.FullyConnected(x, num_neurons=12, has_bias=True, name="fc1")
    h = lbann.BatchNormalization(h, name="bn1", epsilon=1e-5, statistics_group_size=0)
    y = lbann.FullyConnected(lbann.Tanh(h), num_neurons=3, has_bias=True, name="fc2")
    loss = lbann.MeanSquaredError(y, t, name="mse")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x, t])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    sgd = lbann.BatchedIterativeOptimizer("sgd", epoch_count=1)
    algo = lbann.KFAC("kfac", sgd, damping_act="1e-2", damping_err="1e-2", damping_bn_err="3e-2",
                      kronecker_decay=0.9, update_intervals="1", compute_interval=1,
                      distribute_precondition_compute=bool(distribute))
    from test_models_cpu import _reader
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=16, random_seed=9, training_algo=algo), model=model,
        data_reader=_reader(64, [8], "normal", response_dims=[3]),
        optimizer=lbann.SGD(learn_rate=0.05, momentum=0.0))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tr.train(m, num_batches=steps)
    w = {x_.name: float(x_.values.detach().double().norm()) for x_ in m.weights}
    tr.algorithm.shutdown()                       # asynchronous jobs still running are counted too
    counts = torch.tensor([float(tr.algorithm.inverses_computed)])
    per_rank = [float(counts)]
    all_w = [w]
    if tr.parallel is not None:
        per_rank = [float(v) for v in tr.comm.all_gather(counts, "trainer")]
        all_w = tr.comm.world_gather_object(w)
    obj, _, _ = m.reduce_statistics("training")
    res = {"weight_norms": w, "world": int(os.environ.get("WORLD_SIZE", "1")), "inverses": per_rank,
           "all_weight_norms": all_w, "installs": tr.algorithm.async_installs, "objective": float(obj)}
    tr.shutdown()
    return res


def subgraph_transformer(num_subgrids, steps):
    """Encoder whose attention heads sit on two sub-grids (two heads each)."""
    from lbann_b200.models.subgraph import TransformerAllSubgraph
    o = opts.reset()
    on_gpu = os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cuda"
    if not on_gpu:
        o.set("disable_cuda", True)
    if num_subgrids > 1:
        o.set("num_subgrids", num_subgrids)
    S, E = 6, 16
    x = lbann.Input(data_field="samples")
    t = lbann.Input(data_field="responses")
    seq = lbann.Reshape(x, dims=[S, E])
    enc = TransformerAllSubgraph(2, hidden_size=E, num_heads=4, num_encoder_layers=2, num_decoder_layers=0,
                                 feedforward_size=32, dropout=0.0, name="sgt")
    y = enc(seq, None)
    y = lbann.FullyConnected(lbann.Reshape(y, dims=[S * E]), num_neurons=4, has_bias=False, name="head")
    loss = lbann.MeanSquaredError(y, t, name="mse")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x, t])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    from test_models_cpu import _reader
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=8, random_seed=17), model=model,
        data_reader=_reader(16, [S * E], "normal", response_dims=[4]),
        optimizer=lbann.SGD(learn_rate=0.05, momentum=0.9))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tags = sorted({l.grid_tag for l in m.layers})
    head_tags = {l.name: l.grid_tag for l in m.layers if l.name.endswith("_matmul") and "encoder0" in l.name}
    dc = tr.data_coordinator
    dc.start_epoch("training")
    losses = []
    for _ in range(steps):
        b_ = dc.next_batch("training")
        if b_ is None:
            dc.start_epoch("training")
            b_ = dc.next_batch("training")
        m.train_step(b_.tensors, b_.global_size)
        v = m.last_objective.detach().float().reshape(1).clone()
        if tr.parallel is not None:
            tr.comm.allreduce(v, "trainer", "sum")
        losses.append(float(v))
    w = {x_.name: float(x_.values.detach().double().norm()) for x_ in m.weights}
    res = {"losses": losses, "weight_norms": w, "world": int(os.environ.get("WORLD_SIZE", "1")),
           "tags": tags, "head_tags": head_tags}
    tr.shutdown()
    return res


def layer_parallel_gpt(num_subgrids, steps):
    """A small GPT whose blocks are placed on sub-grids in order (blocks 0-1 on grid 1,
    blocks 2-3 on grid 2): layer parallelism as placement, the grids run one after the other."""
    from types import SimpleNamespace
    from lbann_b200.models.parallelism import apply_layer_parallelism
    from lbann_b200.models.transformer import construct_gpt_model
    o = opts.reset()
    if os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cpu":
        o.set("disable_cuda", True)
    model = construct_gpt_model(vocab_size=24, seq_len=8, d_model=16, num_heads=2, num_layers=4, ffn_dim=32)
    grids = 0
    if num_subgrids > 1:
        grids = apply_layer_parallelism(model, SimpleNamespace(layer_parallel=True, lp_count=num_subgrids))
        o.set("num_subgrids", grids)
    from test_models_cpu import _reader
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=8, random_seed=23), model=model,
        data_reader=_reader(16, [9], "randint:24"), optimizer=lbann.SGD(learn_rate=0.05, momentum=0.9))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tags = sorted({l.grid_tag for l in m.layers})
    dc = tr.data_coordinator
    dc.start_epoch("training")
    losses = []
    for _ in range(steps):
        b_ = dc.next_batch("training")
        if b_ is None:
            dc.start_epoch("training")
            b_ = dc.next_batch("training")
        m.train_step(b_.tensors, b_.global_size)
        v = m.last_objective.detach().float().reshape(1).clone()
        if tr.parallel is not None:
            tr.comm.allreduce(v, "trainer", "sum")
        losses.append(float(v))
    w = {x_.name: float(x_.values.detach().double().norm()) for x_ in m.weights}
    res = {"losses": losses, "weight_norms": w, "world": int(os.environ.get("WORLD_SIZE", "1")),
           "tags": tags, "grids": grids}
    tr.shutdown()
    return res


def token_parallel(channel_groups, steps):
    """One attention + MLP block over [S, E] token tensors with the tokens split over the
    ranks (channel_groups): projections and the MLP are channel-wise and stay local, the
    score and context products gather keys and values, everything after the block runs
    sample-parallel."""
    o = opts.reset()
    if os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cpu":
        o.set("disable_cuda", True)
    S, E = 8, 16
    ps = lbann.get_parallel_strategy_args(channel_groups=channel_groups) if channel_groups > 1 else {}
    x = lbann.Input(data_field="samples")
    t = lbann.Input(data_field="responses")
    seq = lbann.Identity(lbann.Reshape(x, dims=[S, E]), name="tokens", parallel_strategy=ps)

    def cfc(h, n, name):
        return lbann.ChannelwiseFullyConnected(h, output_channel_dims=[n], name=name, parallel_strategy=ps)
    q, k, v = cfc(seq, E, "q"), cfc(seq, E, "k"), cfc(seq, E, "v")
    scores = lbann.MatMul(q, k, transpose_b=True, name="scores", parallel_strategy=ps)
    probs = lbann.ChannelwiseSoftmax(lbann.Scale(scores, constant=E ** -0.5, name="scaled", parallel_strategy=ps),
                                     name="probs", parallel_strategy=ps)
    ctx = lbann.MatMul(probs, v, name="context", parallel_strategy=ps)
    h = lbann.Add(seq, ctx, name="res1", parallel_strategy=ps)
    m = cfc(lbann.Relu(cfc(h, 32, "up"), name="act", parallel_strategy=ps), E, "down")
    h = lbann.Add(h, m, name="res2", parallel_strategy=ps)
    y = lbann.FullyConnected(lbann.Reshape(h, dims=[S * E]), num_neurons=4, has_bias=False, name="head")
    loss = lbann.MeanSquaredError(y, t, name="mse")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x, t])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    from test_models_cpu import _reader
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=6, random_seed=29), model=model,
        data_reader=_reader(12, [S * E], "normal", response_dims=[4]),
        optimizer=lbann.SGD(learn_rate=0.005, momentum=0.9))
    tr = ExecTrainer(exp)
    mdl = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    losses = []
    for _ in range(steps):
        b_ = dc.next_batch("training")
        if b_ is None:
            dc.start_epoch("training")
            b_ = dc.next_batch("training")
        mdl.train_step(b_.tensors, b_.global_size)
        vv = mdl.last_objective.detach().float().reshape(1).clone()
        if tr.parallel is not None:
            tr.comm.allreduce(vv, "trainer", "sum")
        losses.append(float(vv))
    w = {x_.name: float(x_.values.detach().double().norm()) for x_ in mdl.weights}
    spatial = sorted(n for n, d in (tr.distconv.dist.items() if tr.distconv is not None else []) if d == "spatial")
    res = {"losses": losses, "weight_norms": w, "world": int(os.environ.get("WORLD_SIZE", "1")),
           "partitioned": spatial, "sample_groups": tr.distconv.num_sample_groups if tr.distconv is not None else 1}
    tr.shutdown()
    return res


def filter_parallel(channel_groups, steps):
    """Two 3-D convolutions with bias, leaky ReLU and max pooling whose channels / filters are
    split over the ranks (channel_groups == filter_groups), a batch norm (not partitioned: runs
    sample-parallel after a redistribution) and a fully-connected head."""
    o = opts.reset()
    if os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cpu":
        o.set("disable_cuda", True)
    ps = lbann.get_parallel_strategy_args(channel_groups=channel_groups, filter_groups=channel_groups) \
        if channel_groups > 1 else {}
    x = lbann.Input(data_field="samples")
    t = lbann.Input(data_field="responses")
    vol = lbann.Identity(lbann.Reshape(x, dims=[4, 8, 8, 8]), name="volume", parallel_strategy=ps)

    def conv(h, n, name):
        return lbann.Convolution(h, num_dims=3, out_channels=n, kernel_size=3, padding=1, stride=1, has_bias=True,
                                 name=name, parallel_strategy=ps)

    def pool(h, name):
        return lbann.Pooling(h, num_dims=3, pool_dims_i=2, pool_strides_i=2, pool_pads_i=0, pool_mode="max",
                             name=name, parallel_strategy=ps)
    h = pool(lbann.LeakyRelu(conv(vol, 8, "conv1"), negative_slope=0.1, name="act1", parallel_strategy=ps), "pool1")
    h = lbann.BatchNormalization(h, name="bn", epsilon=1e-5, statistics_group_size=-1)
    h = pool(lbann.LeakyRelu(conv(h, 12, "conv2"), negative_slope=0.1, name="act2", parallel_strategy=ps), "pool2")
    y = lbann.FullyConnected(h, num_neurons=4, has_bias=True, name="head")
    loss = lbann.MeanSquaredError(y, t, name="mse")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x, t])),
                        objective_function=lbann.ObjectiveFunction([loss]))
    from test_models_cpu import _reader
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=6, random_seed=31), model=model,
        data_reader=_reader(12, [4 * 8 * 8 * 8], "normal", response_dims=[4]),
        optimizer=lbann.SGD(learn_rate=0.01, momentum=0.9))
    tr = ExecTrainer(exp)
    mdl = tr.build_model(exp.model)
    dc = tr.data_coordinator
    dc.start_epoch("training")
    losses = []
    for _ in range(steps):
        b_ = dc.next_batch("training")
        if b_ is None:
            dc.start_epoch("training")
            b_ = dc.next_batch("training")
        mdl.train_step(b_.tensors, b_.global_size)
        vv = mdl.last_objective.detach().float().reshape(1).clone()
        if tr.parallel is not None:
            tr.comm.allreduce(vv, "trainer", "sum")
        losses.append(float(vv))
    w = {x_.name: float(x_.values.detach().double().norm()) for x_ in mdl.weights if "running" not in x_.name}
    spatial = sorted(n for n, d in (tr.distconv.dist.items() if tr.distconv is not None else []) if d == "spatial")
    res = {"losses": losses, "weight_norms": w, "world": int(os.environ.get("WORLD_SIZE", "1")),
           "partitioned": spatial, "sample_groups": tr.distconv.num_sample_groups if tr.distconv is not None else 1}
    tr.shutdown()
    return res


def subgraph_branches(num_subgrids, steps):
    """Two branches of a small network on two sub-grids (grid tags 1 and 2), joined by a sum on
    the whole trainer; a third output goes through a sum across the grids."""
    o = opts.reset()
    on_gpu = os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cuda"
    if not on_gpu:
        o.set("disable_cuda", True)
    if num_subgrids > 1:
        o.set("num_subgrids", num_subgrids)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    x = lbann.Input(data_field="samples")
    t = lbann.Input(data_field="responses")
    a = lbann.Sin(x, grid_tag=1, name="branch1_sin")
    a = lbann.FullyConnected(a, num_neurons=8, has_bias=True, name="branch1_fc")        # inherits grid 1
    b = lbann.Cos(x, parallel_strategy={"grid_tag": 2}, name="branch2_cos")
    b = lbann.FullyConnected(b, num_neurons=8, has_bias=True, name="branch2_fc")        # inherits grid 2
    y = lbann.Sum(a, b, name="join")                                                       # parents differ: grid 0
    y = lbann.FullyConnected(lbann.Tanh(y), num_neurons=4, has_bias=False, name="head")
    loss = lbann.MeanSquaredError(y, t, name="mse")
    model = lbann.Model(1, layers=list(lbann.traverse_layer_graph([x, t])),
                        objective_function=lbann.ObjectiveFunction([loss]),
                        metrics=[lbann.Metric(loss, name="mse")])
    from test_models_cpu import _reader
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=8, random_seed=13), model=model,
        data_reader=_reader(32, [16], "normal", response_dims=[4]),
        optimizer=lbann.SGD(learn_rate=0.05, momentum=0.9))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    tags = {l.name: l.grid_tag for l in m.layers if l.name in ("branch1_sin", "branch1_fc", "branch2_cos",
                                                                "branch2_fc", "join", "head")}
    dc = tr.data_coordinator
    dc.start_epoch("training")
    losses = []
    for _ in range(steps):
        b_ = dc.next_batch("training")
        if b_ is None:
            dc.start_epoch("training")
            b_ = dc.next_batch("training")
        m.train_step(b_.tensors, b_.global_size)
        v = m.last_objective.detach().float().reshape(1).clone()
        if tr.parallel is not None:
            tr.comm.allreduce(v, "trainer", "sum")
        losses.append(float(v))
    w = {x_.name: float(x_.values.detach().double().norm()) for x_ in m.weights}
    moved = tr.parallel.subgrid.bytes_moved if (tr.parallel is not None and tr.parallel.subgrid) else 0
    tr.shutdown()
    return {"world": world, "losses": losses, "weight_norms": w, "tags": tags, "bytes_moved": moved}


def abort_and_restart(ckpt_dir, fail_step, epochs):
    """LeNet on the ranks of one trainer with a shared checkpoint after every epoch.  With
    fail_step >= 0 rank 1 raises between two steps (after step ``fail_step``); the driver's
    abort semantics then end this process with a non-zero code and the launcher tears the
    other rank down.  A later run with the same checkpoint directory resumes."""
    from lbann_b200 import driver
    from lbann_b200.callbacks import ExecCallback
    from test_lenet_cpu import build_lenet, make_reader
    o = opts.reset()
    if os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cpu":
        o.set("disable_cuda", True)
    images, labels, loss, acc = build_lenet()
    cbs = [lbann.CallbackCheckpoint(checkpoint_dir=ckpt_dir, checkpoint_epochs=1)]
    model = lbann.Model(epochs, layers=[images, labels], objective_function=loss,
                        metrics=[lbann.Metric(acc, name="accuracy", unit="%")], callbacks=cbs)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=64, random_seed=7), model=model,
        data_reader=make_reader(256), optimizer=lbann.SGD(learn_rate=0.01, momentum=0.9))
    rank = int(os.environ.get("RANK", "0"))

    class FailAt(ExecCallback):
        def on_batch_end(self, m):
            if fail_step >= 0 and rank == 1 and m.ctx.step >= fail_step:
                raise RuntimeError(f"injected failure on rank {rank} after step {m.ctx.step}")

    orig = ExecTrainer.build_model

    def build_with_failure(self, proto):
        m = orig(self, proto)
        m.callbacks.append(FailAt())
        return m
    ExecTrainer.build_model = build_with_failure
    try:
        tr, m = driver.run_experiment(exp, return_trainer=True)
    finally:
        ExecTrainer.build_model = orig
    w = {x.name: float(x.values.detach().double().norm()) for x in m.weights}
    res = {"world": int(os.environ.get("WORLD_SIZE", "1")), "weights": w, "epoch": m.ctx.epoch,
           "step": m.ctx.step, "state_compact": bool(getattr(m.arena, "state_compact", False)),
           "state_bytes": int(m.arena.state_bytes()), "master_bytes": int(m.arena.master.numel() * 4)}
    tr.shutdown()
    return res


if __name__ == "__main__":
    what, out = sys.argv[1], sys.argv[2]
    if what == "comm":
        res = comm_kernels()
    elif what == "fused":
        res = fused_gemm()
    elif what == "tp":
        res = tensor_parallel()
    elif what == "ltfb":
        res = ltfb(sys.argv[3])
    elif what == "distembed":
        res = dist_embedding(int(sys.argv[3]))
    elif what == "store":
        res = data_store(sys.argv[3] == "preload")
    elif what == "mpfc":
        res = model_parallel_fc(int(sys.argv[3]), int(sys.argv[4]), len(sys.argv) > 5 and sys.argv[5] == "sharded")
    elif what == "subgraph":
        res = subgraph_branches(int(sys.argv[3]), int(sys.argv[4]))
    elif what == "kfac":
        res = kfac_job(int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5]) if len(sys.argv) > 5 else 0)
    elif what == "filter_parallel":
        res = filter_parallel(int(sys.argv[3]), int(sys.argv[4]))
    elif what == "token_parallel":
        res = token_parallel(int(sys.argv[3]), int(sys.argv[4]))
    elif what == "layer_parallel":
        res = layer_parallel_gpt(int(sys.argv[3]), int(sys.argv[4]))
    elif what == "subgraph_transformer":
        res = subgraph_transformer(int(sys.argv[3]), int(sys.argv[4]))
    elif what == "abort_restart":
        res = abort_and_restart(sys.argv[3], int(sys.argv[4]), int(sys.argv[5]))
    elif what == "unet":
        res = unet(int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5]))
    elif what == "cosmoflow":
        res = cosmoflow(int(sys.argv[3]), int(sys.argv[4]), sys.argv[5] if len(sys.argv) > 5 else "float",
                        int(sys.argv[6]) if len(sys.argv) > 6 else 32,
                        tuple(int(c) for c in sys.argv[7].split(",")) if len(sys.argv) > 7 else (8, 16, 16),
                        len(sys.argv) > 8 and sys.argv[8] == "graph")
    else:
        raise SystemExit(f"unknown job {what}")
    if int(os.environ.get("RANK", "0")) == 0:
        with open(out, "w") as f:
            json.dump(res, f)
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
