"""CosmoFlow 3-D CNN with the volumes split along depth over the GPUs of the job
(applications/physics/cosmology/cosmoflow of the reference).

    torchrun --nnodes=1 --nproc-per-node 4 examples/cosmoflow.py --depth-groups 4 --in-process
    python examples/cosmoflow.py --procs-per-node 8 --depth-groups 8        # through the launcher
"""
import argparse

import lbann
import lbann.contrib.args
import lbann.contrib.launcher
from lbann.models.cosmoflow import construct_cosmoflow_model, synthetic_reader


def build(args, world):
    depth = args.depth_groups or world
    ps = lbann.get_parallel_strategy_args(depth_groups=depth) if depth > 1 else None
    model = construct_cosmoflow_model(args.width, 4, 4, num_epochs=args.num_epochs, pool_mode="max",
                                      parallel_strategy=ps)
    model.callbacks.extend([lbann.CallbackPrint(), lbann.CallbackTimer()])
    reader = synthetic_reader(args.num_samples, args.width, 4, 4, pool=2 * args.mini_batch_size)
    trainer = lbann.Trainer(mini_batch_size=args.mini_batch_size)
    return trainer, model, reader, lbann.Adam(learn_rate=args.learning_rate, beta1=0.9, beta2=0.99, eps=1e-8)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    lbann.contrib.args.add_scheduler_arguments(ap, "cosmoflow")
    lbann.contrib.args.add_training_arguments(ap, default_minibatch_size=8, default_epochs=1)
    ap.add_argument("--width", type=int, default=128, help="edge of the cubic volumes")
    ap.add_argument("--num-samples", type=int, default=64)
    ap.add_argument("--depth-groups", type=int, default=0, help="ranks along depth (default: all)")
    ap.add_argument("--learning-rate", type=float, default=1e-3)
    ap.add_argument("--in-process", action="store_true", help="this process is a rank started by torchrun")
    a = ap.parse_args()
    kw = lbann.contrib.args.get_scheduler_kwargs(a)
    world = (kw.get("nodes") or 1) * (kw.get("procs_per_node") or 1)
    if a.in_process:
        import os
        from lbann_b200 import driver
        world = int(os.environ.get("WORLD_SIZE", "1"))
        trainer, model, reader, opt = build(a, world)
        exp = lbann.proto.serialize.build_experiment(trainer=trainer, model=model, data_reader=reader, optimizer=opt)
        from lbann_b200.utils import options
        o = options.current()
        o.set("default_dtype", "fp16")
        o.set("use_cuda_graph", True)
        driver.run_experiment(exp)
        raise SystemExit(0)
    trainer, model, reader, opt = build(a, world)
    raise SystemExit(lbann.contrib.launcher.run(trainer, model, reader, opt,
                                                lbann_args=["--default_dtype=fp16", "--use_cuda_graph"], **kw))
