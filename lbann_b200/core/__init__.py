"""``lbann.core``: the front-end object model, grouped like the reference's package
(python/lbann/core/*.py); everything is defined in ``lbann_b200.frontend``."""
from . import (callback, evaluate, layer, metric, model, objective_function, operator_layers,  # noqa: F401
               operators, optimizer, trainer, training_algorithm, util, weights)
