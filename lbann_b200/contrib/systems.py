"""Computing centres and their machines: what the site launchers need to pick defaults
(python/lbann/contrib/{lc,nersc,olcf,riken}/systems.py keep one such table per centre).

A machine is recognised by its host name without the trailing node number, or by the
environment variable its centre sets.  On anything else (a workstation, a cloud box with
B200s) ``detect()`` returns ``(None, None)`` and the generic launcher takes over.
"""
from __future__ import annotations

import os
import re
import socket
from typing import NamedTuple, Optional, Tuple


class System(NamedTuple):
    cores_per_node: int
    gpus_per_node: int
    scheduler: str


SITES = {
    "lc": {           # Livermore Computing
        "catalyst": System(24, 0, "slurm"), "quartz": System(36, 0, "slurm"), "pascal": System(36, 2, "slurm"),
        "lassen": System(44, 4, "lsf"), "sierra": System(44, 4, "lsf"), "rzansel": System(44, 4, "lsf"),
        "corona": System(48, 8, "flux"), "tioga": System(64, 8, "flux"), "rzvernal": System(64, 8, "flux"),
        "tuolumne": System(96, 4, "flux"), "rzadams": System(96, 4, "flux"),
    },
    "nersc": {"cgpu": System(40, 8, "slurm"), "perlmutter": System(64, 4, "slurm")},
    "olcf": {"summit": System(44, 6, "lsf"), "frontier": System(64, 8, "slurm"), "crusher": System(64, 8, "slurm")},
    "riken": {"fugaku": System(48, 0, "pjm")},
}
# environment variables that name the machine directly
_ENV_HINTS = (("NERSC_HOST", "nersc"), ("LMOD_SYSTEM_NAME", "olcf"), ("LCSCHEDCLUSTER", "lc"))


def host_system() -> str:
    """Host name with the node number and domain stripped (``lassen708.llnl.gov`` -> ``lassen``)."""
    return re.sub(r"\d+$", "", socket.gethostname().split(".")[0])


def detect(environ=None, hostname: Optional[str] = None) -> Tuple[Optional[str], Optional[str]]:
    """``(site, system)`` of the machine this process runs on, or ``(None, None)``."""
    env = os.environ if environ is None else environ
    for var, site in _ENV_HINTS:
        name = (env.get(var) or "").lower()
        if name in SITES[site]:
            return site, name
    name = hostname if hostname is not None else host_system()
    name = re.sub(r"\d+$", "", name.split(".")[0]).lower()
    for site, table in SITES.items():
        if name in table:
            return site, name
    return None, None


def params(site: str, system: Optional[str] = None) -> System:
    if system is None:
        s, system = detect()
        if s != site:
            raise RuntimeError(f"not running on a known {site} system ({host_system()})")
    try:
        return SITES[site][system]
    except KeyError:
        raise RuntimeError(f"unknown {site} system ({system})") from None


def procs_per_node(site: str, system: Optional[str] = None) -> int:
    """One process per GPU; on CPU machines one per socket (two sockets per node)."""
    p = params(site, system)
    return p.gpus_per_node if p.gpus_per_node > 0 else 2
