"""Site-aware launcher front (python/lbann/contrib/launcher.py): picks scheduler defaults
from the environment and forwards to :func:`lbann.run`."""
from __future__ import annotations

import os

from .. import launcher as _launcher


def detect_scheduler() -> str:
    if "SLURM_JOB_ID" in os.environ:
        return "slurm"
    if "LSB_JOBID" in os.environ:
        return "lsf"
    if "FLUX_URI" in os.environ:
        return "flux"
    return "local"


def run(*args, **kwargs):
    kwargs.setdefault("scheduler", detect_scheduler())
    return _launcher.run(*args, **kwargs)


def make_batch_script(*args, **kwargs):
    from ..launcher.batch_script import make_batch_script as _mk
    kwargs.setdefault("scheduler", detect_scheduler())
    return _mk(*args, **kwargs)
