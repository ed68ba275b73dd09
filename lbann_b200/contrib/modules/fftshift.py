"""``numpy.fft.fftshift`` over the spatial dimensions of a [channel, ...] tensor, as one
gather with constant indices (python/lbann/contrib/modules/fftshift.py)."""
from __future__ import annotations

import numpy as np

from ...frontend import core as L
from ...modules import Module


class FFTShift(Module):
    """Moves the zero-frequency component to the centre of the spectrum, independently per
    channel (dimension 0).  ``inverse=True`` gives ``ifftshift`` (the two differ for odd sizes)."""

    def __init__(self, inverse: bool = False):
        super().__init__()
        self.inverse = inverse

    def forward(self, x, dims):
        dims = tuple(int(d) for d in dims)
        spatial = int(np.prod(dims[1:]))
        # where every output element comes from: shift a tensor that holds its own flat indices
        src = np.arange(spatial).reshape(dims[1:])
        src = (np.fft.ifftshift if self.inverse else np.fft.fftshift)(src).reshape(-1)
        idx = L.WeightsLayer(weights=L.Weights(initializer=L.ValueInitializer(values=[float(v) for v in src]),
                                               optimizer=L.NoOptimizer()), dims=[spatial])
        y = L.Gather(L.Reshape(x, dims=[dims[0], spatial]), idx, axis=1)
        return L.Reshape(y, dims=list(dims))
