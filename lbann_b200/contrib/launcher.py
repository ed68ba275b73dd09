"""Site-aware launcher front (python/lbann/contrib/launcher.py): recognises the computing
centre from the host name or its environment, takes the scheduler, the processes per node
and the centre's environment settings from ``lbann.contrib.systems``, and forwards to
:func:`lbann.run`.  On an unknown machine the scheduler is guessed from the job environment."""
from __future__ import annotations

import os

from .. import launcher as _launcher
from . import systems as _systems

# environment each centre's machines want for one-process-per-GPU jobs
SITE_ENVIRONMENT = {
    "lc": {"OMP_NUM_THREADS": None, "MV2_USE_RDMA_CM": "0", "AL_PROGRESS_RANKS_PER_NUMA_NODE": "2"},
    "nersc": {"OMP_NUM_THREADS": None, "MPICH_GPU_SUPPORT_ENABLED": "1"},
    "olcf": {"OMP_NUM_THREADS": None, "MPICH_GPU_SUPPORT_ENABLED": "1", "NCCL_SOCKET_IFNAME": "hsn0"},
    "riken": {"OMP_NUM_THREADS": None},
}


def detect_scheduler() -> str:
    site, system = _systems.detect()
    if site is not None:
        return _systems.params(site, system).scheduler
    if "SLURM_JOB_ID" in os.environ:
        return "slurm"
    if "LSB_JOBID" in os.environ:
        return "lsf"
    if "FLUX_URI" in os.environ:
        return "flux"
    return "local"


def site_defaults(site: str, system=None, kwargs=None) -> dict:
    """Fill scheduler / procs_per_node / environment defaults for a machine of ``site``."""
    kw = dict(kwargs or {})
    if system is None:
        s, system = _systems.detect()
        if s != site:
            system = None
    if system is not None:
        p = _systems.params(site, system)
        kw.setdefault("scheduler", p.scheduler)
        kw.setdefault("procs_per_node", _systems.procs_per_node(site, system))
        env = dict(kw.get("environment") or {})
        for k, v in SITE_ENVIRONMENT.get(site, {}).items():
            if v is None:          # threads per process: the node's cores over its processes
                v = str(max(1, p.cores_per_node // max(1, kw["procs_per_node"]) - 1))
            env.setdefault(k, v)
        kw["environment"] = env
    else:
        kw.setdefault("scheduler", detect_scheduler())
    return kw


def site_run(site, *args, system=None, **kwargs):
    return _launcher.run(*args, **site_defaults(site, system, kwargs))


def site_make_batch_script(site, *args, system=None, **kwargs):
    from ..launcher.batch_script import make_batch_script as _mk
    kw = site_defaults(site, system, kwargs)
    return _mk(*args, **kw)


def run(*args, **kwargs):
    site, system = _systems.detect()
    if site is not None:
        return site_run(site, *args, system=system, **kwargs)
    kwargs.setdefault("scheduler", detect_scheduler())
    return _launcher.run(*args, **kwargs)


def make_batch_script(*args, **kwargs):
    site, system = _systems.detect()
    if site is not None:
        return site_make_batch_script(site, *args, system=system, **kwargs)
    from ..launcher.batch_script import make_batch_script as _mk
    kwargs.setdefault("scheduler", detect_scheduler())
    return _mk(*args, **kwargs)
