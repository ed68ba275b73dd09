"""Machines of this centre (python/lbann/contrib/riken/systems.py); the table lives in
``lbann.contrib.systems``."""
from .. import systems as _all

SITE = "riken"


def system():
    """Name of the machine this process runs on (host name without the node number)."""
    site, name = _all.detect()
    return name if site == SITE else _all.host_system()


def is_riken_system(name=None):
    return (name or system()) in _all.SITES[SITE]


def _p(name=None):
    return _all.params(SITE, name or system())


def gpus_per_node(name=None):
    return _p(name).gpus_per_node


def has_gpu(name=None):
    return gpus_per_node(name) > 0


def cores_per_node(name=None):
    return _p(name).cores_per_node


def scheduler(name=None):
    return _p(name).scheduler


def procs_per_node(name=None):
    return _all.procs_per_node(SITE, name or system())
