"""Where the common data sets live on Livermore Computing file systems
(python/lbann/contrib/lc/paths.py).  Paths are returned, not checked: the file systems are
only mounted on the centre's machines."""
from . import systems as _sys

_ROOT = {"default": "/p/lustre2/brainusr/datasets", "lassen": "/p/gpfs1/brainusr/datasets",
         "sierra": "/p/gpfs1/brainusr/datasets", "rzansel": "/p/gpfs1/brainusr/datasets"}


def parallel_file_system_path(system=None):
    return _ROOT.get(system or _sys.system(), _ROOT["default"]) + "/"


def mnist_dir(system=None):
    return parallel_file_system_path(system) + "MNIST"


def cifar10_dir(system=None):
    return parallel_file_system_path(system) + "cifar10-bin"


def imagenet_dir(system=None, data_set="training", num_classes=1000):
    base = parallel_file_system_path(system) + "ILSVRC2012/original/"
    sub = {"train": "train/", "training": "train/", "val": "val/", "validation": "val/", "evaluation": "val/"}
    if data_set not in sub:
        raise RuntimeError(f"unknown ImageNet data set ({data_set})")
    return base + sub[data_set]


def imagenet_labels(system=None, data_set="training", num_classes=1000):
    base = parallel_file_system_path(system) + "ILSVRC2012/original/labels/"
    name = {"train": "train", "training": "train", "val": "val", "validation": "val", "evaluation": "val"}
    if data_set not in name:
        raise RuntimeError(f"unknown ImageNet data set ({data_set})")
    suffix = "" if num_classes == 1000 else f"_c0-{num_classes - 1}"
    return f"{base}{name[data_set]}{suffix}.txt"
