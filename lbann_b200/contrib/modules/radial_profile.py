"""Mean pixel value as a function of the distance from the image centre, per channel
(python/lbann/contrib/modules/radial_profile.py): distances are binned with bin size 1, every
pixel is scattered into its bin with weight 1 / (pixels in the bin)."""
from __future__ import annotations

import numpy as np

from ...frontend import core as L
from ...modules import Module


class RadialProfile(Module):
    @staticmethod
    def radial_bins(spatial_dims, max_r):
        """Bin index of every pixel (distance from the centre, rounded down) and the number
        of pixels in each of the ``max_r`` bins."""
        axes = [np.arange(n) - (n - 1) / 2.0 for n in spatial_dims]
        grid = np.meshgrid(*axes, indexing="ij")
        r = np.floor(np.sqrt(sum(g * g for g in grid))).astype(np.int64)
        counts = np.bincount(r.reshape(-1), minlength=max_r)[:max_r]
        return r, counts

    def forward(self, image, dims, max_r):
        dims = tuple(int(d) for d in dims)
        c, spatial = dims[0], int(np.prod(dims[1:]))
        r, counts = self.radial_bins(dims[1:], max_r)
        weight = np.where(counts > 0, 1.0 / np.maximum(counts, 1), 0.0)
        r = r.reshape(-1)
        inside = r < max_r
        # scale every pixel by 1 / count of its bin, then add the pixels of a bin up
        scale = np.where(inside, weight[np.minimum(r, max_r - 1)], 0.0)
        const = lambda vals: L.WeightsLayer(                                         # noqa: E731
            weights=L.Weights(initializer=L.ValueInitializer(values=[float(v) for v in vals]),
                              optimizer=L.NoOptimizer()), dims=[len(vals)])
        x = L.Reshape(image, dims=[c, spatial])
        x = L.Multiply(x, L.Tessellate(L.Reshape(const(scale), dims=[1, spatial]), dims=[c, spatial]))
        bins = const(np.where(inside, r, -1))                                       # -1: dropped by the scatter
        return L.Scatter(x, bins, dims=[c, max_r], axis=1)
