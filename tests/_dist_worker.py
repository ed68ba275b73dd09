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


def cosmoflow(depth_groups, steps, dtype, width=32):
    o = opts.reset()
    o.set("default_dtype", dtype)
    if os.environ.get("LBANN_TEST_DEVICE", "cpu") == "cpu":
        o.set("disable_cuda", True)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ps = lbann.get_parallel_strategy_args(depth_groups=depth_groups) if depth_groups > 1 else None
    model = construct_cosmoflow_model(width, 4, 4, num_epochs=1, channels=(8, 16, 16), pool_mode="max",
                                      conv_bias=False, fc_sizes=(32, 16), parallel_strategy=ps)
    exp = lbann.proto.serialize.build_experiment(
        trainer=lbann.Trainer(mini_batch_size=4, random_seed=5), model=model,
        data_reader=synthetic_reader(16, width, 4, 4),
        optimizer=lbann.SGD(learn_rate=0.01, momentum=0.9))
    tr = ExecTrainer(exp)
    m = tr.build_model(exp.model)
    losses = []
    dc = tr.data_coordinator
    dc.start_epoch("training")
    for _ in range(steps):
        b = dc.next_batch("training")
        m.train_step(b.tensors, b.global_size)
        v = m.last_objective.detach().float().reshape(1).clone()
        if tr.parallel is not None:
            tr.comm.allreduce(v, "trainer", "sum")
        losses.append(float(v))
    w = {x.name: float(x.values.detach().float().norm()) for x in m.weights}
    tr.shutdown()
    return {"losses": losses, "weight_norms": w, "world": world}


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


if __name__ == "__main__":
    what, out = sys.argv[1], sys.argv[2]
    if what == "comm":
        res = comm_kernels()
    elif what == "cosmoflow":
        res = cosmoflow(int(sys.argv[3]), int(sys.argv[4]), sys.argv[5] if len(sys.argv) > 5 else "float",
                        int(sys.argv[6]) if len(sys.argv) > 6 else 32)
    else:
        raise SystemExit(f"unknown job {what}")
    if int(os.environ.get("RANK", "0")) == 0:
        with open(out, "w") as f:
            json.dump(res, f)
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
