"""The lsf flavour of the batch script (python/lbann/launcher/lsf.py): header directives,
parallel launch prefix and submit command of that scheduler; the class lives in
``batch_script.py`` with the others."""
from .batch_script import LSFBatchScript  # noqa: F401


def make_batch_script(**kwargs) -> LSFBatchScript:
    return LSFBatchScript(**kwargs)
