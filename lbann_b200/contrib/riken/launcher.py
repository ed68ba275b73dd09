"""``run`` / ``make_batch_script`` with this centre's defaults
(python/lbann/contrib/riken/launcher.py): scheduler and processes per node from the machine
table, the centre's environment settings, then the generic launcher."""
from ..launcher import site_make_batch_script, site_run

SITE = "riken"


def run(*args, **kwargs):
    return site_run(SITE, *args, **kwargs)


def make_batch_script(*args, **kwargs):
    return site_make_batch_script(SITE, *args, **kwargs)
