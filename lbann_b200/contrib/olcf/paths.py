"""Data set locations at this centre (python/lbann/contrib/olcf/paths.py): taken from the
environment (``LBANN_DATA_ROOT``), since the centre's project directories differ per allocation."""
import os


def parallel_file_system_path(system=None):
    return os.environ.get("LBANN_DATA_ROOT", os.path.expanduser("~/datasets")).rstrip("/") + "/"


def mnist_dir(system=None):
    return parallel_file_system_path(system) + "MNIST"


def cifar10_dir(system=None):
    return parallel_file_system_path(system) + "cifar10-bin"


def imagenet_dir(system=None, data_set="training", num_classes=1000):
    sub = {"train": "train/", "training": "train/", "val": "val/", "validation": "val/", "evaluation": "val/"}
    if data_set not in sub:
        raise RuntimeError(f"unknown ImageNet data set ({data_set})")
    return parallel_file_system_path(system) + "imagenet/" + sub[data_set]


def imagenet_labels(system=None, data_set="training", num_classes=1000):
    name = "train" if data_set in ("train", "training") else "val"
    return parallel_file_system_path(system) + f"imagenet/labels/{name}.txt"
