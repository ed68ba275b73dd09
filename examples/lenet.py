"""LeNet-5 on MNIST (applications/vision/lenet.py of the reference).

    python examples/lenet.py --synthetic --num-epochs 2
    python examples/lenet.py --data-dir /data/MNIST --nodes 1 --procs-per-node 4
"""
import argparse

import lbann
import lbann.contrib.args
import lbann.contrib.launcher


def build(args):
    images = lbann.Input(data_field="samples", name="images")
    labels = lbann.Input(data_field="labels", name="labels")
    x = lbann.Reshape(images, dims=[1, 28, 28])
    probs = lbann.Softmax(lbann.models.LeNet(10)(x), name="probs")
    loss = lbann.CrossEntropy(probs, labels, name="cross_entropy")
    acc = lbann.CategoricalAccuracy(probs, labels, name="accuracy")
    callbacks = [lbann.CallbackPrintModelDescription(), lbann.CallbackPrint(), lbann.CallbackTimer()]
    if args.checkpoint_dir:
        callbacks.append(lbann.CallbackCheckpoint(checkpoint_dir=args.checkpoint_dir, checkpoint_epochs=1))
    model = lbann.Model(args.num_epochs, layers=list(lbann.traverse_layer_graph([images, labels])),
                        objective_function=lbann.ObjectiveFunction([loss, lbann.L2WeightRegularization(scale=1e-4)]),
                        metrics=[lbann.Metric(acc, name="accuracy", unit="%")], callbacks=callbacks)
    reader = lbann.reader_pb2.DataReader()
    for role, images_file, labels_file in (("train", "train-images-idx3-ubyte", "train-labels-idx1-ubyte"),
                                           ("test", "t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte")):
        r = reader.reader.add()
        r.role, r.shuffle, r.fraction_of_data_to_use = role, role == "train", 1.0
        if args.synthetic:
            r.name, r.num_samples, r.num_labels = "synthetic", 512 if role == "train" else 128, 10
            r.synth_dimensions, r.synth_distribution = "1 28 28", "uniform"
        else:
            r.name, r.data_filedir, r.num_labels = "mnist", args.data_dir, 10
            r.data_filename, r.label_filename = images_file, labels_file
        if role == "train":
            r.validation_fraction = 0.1
    return lbann.Trainer(mini_batch_size=args.mini_batch_size), model, reader


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    lbann.contrib.args.add_scheduler_arguments(ap, "lenet")
    lbann.contrib.args.add_training_arguments(ap, default_minibatch_size=64, default_epochs=5)
    lbann.contrib.args.add_optimizer_arguments(ap, default_optimizer="momentum", default_learning_rate=0.01)
    ap.add_argument("--data-dir", default="/data/MNIST")
    ap.add_argument("--synthetic", action="store_true", help="random digits instead of the MNIST files")
    ap.add_argument("--checkpoint-dir", default="")
    a = ap.parse_args()
    trainer, model, reader = build(a)
    raise SystemExit(lbann.contrib.launcher.run(trainer, model, reader, lbann.contrib.args.create_optimizer(a),
                                                **lbann.contrib.args.get_scheduler_kwargs(a)))
