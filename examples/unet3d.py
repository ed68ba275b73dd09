"""3-D U-Net segmentation with batch norm on a depth x height grid of GPUs
(applications/segmentation of the reference).

    python examples/unet3d.py --procs-per-node 8 --depth-groups 4 --height-groups 2 --volume 256
"""
import argparse

import lbann
import lbann.contrib.args
import lbann.contrib.launcher
from lbann.models import construct_unet3d_model


def build(args, world):
    hg = max(1, args.height_groups)
    dg = args.depth_groups or max(1, world // hg)
    ps = lbann.get_parallel_strategy_args(depth_groups=dg, height_groups=hg) if dg * hg > 1 else None
    model = construct_unet3d_model(num_classes=3, base_channels=args.base_channels, levels=args.levels,
                                   num_epochs=args.num_epochs, parallel_strategy=ps)
    model.callbacks.extend([lbann.CallbackPrint(), lbann.CallbackTimer()])
    v = args.volume
    reader = lbann.reader_pb2.DataReader()
    r = reader.reader.add()
    r.name, r.role, r.shuffle, r.fraction_of_data_to_use = "synthetic", "train", False, 1.0
    r.synth_dimensions, r.synth_response_dimensions = f"1 {v} {v} {v}", f"{v} {v} {v}"
    r.synth_distribution, r.num_samples = "samples:normal responses:randint:3", args.num_samples
    r.synth_pool_size = 2 * args.mini_batch_size
    return lbann.Trainer(mini_batch_size=args.mini_batch_size), model, reader


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    lbann.contrib.args.add_scheduler_arguments(ap, "unet3d")
    lbann.contrib.args.add_training_arguments(ap, default_minibatch_size=1, default_epochs=1)
    ap.add_argument("--volume", type=int, default=128)
    ap.add_argument("--num-samples", type=int, default=16)
    ap.add_argument("--base-channels", type=int, default=32)
    ap.add_argument("--levels", type=int, default=4)
    ap.add_argument("--depth-groups", type=int, default=0)
    ap.add_argument("--height-groups", type=int, default=1)
    a = ap.parse_args()
    kw = lbann.contrib.args.get_scheduler_kwargs(a)
    world = (kw.get("nodes") or 1) * (kw.get("procs_per_node") or 1)
    trainer, model, reader = build(a, world)
    raise SystemExit(lbann.contrib.launcher.run(trainer, model, reader,
                                                lbann.Adam(learn_rate=1e-3, beta1=0.9, beta2=0.99, eps=1e-8),
                                                lbann_args=["--default_dtype=bf16"], **kw))
