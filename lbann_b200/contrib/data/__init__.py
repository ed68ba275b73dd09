"""Data sets for the Python-dataset reader (python/lbann/contrib/data)."""
from . import chem_tokenizers, molecule_dataset  # noqa: F401
