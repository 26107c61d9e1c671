"""Two mixers side by side: both read the same input, the result is ``left_scale * left + right_scale * right``.

The two are parts of any registered kind (``left``, ``right`` in the spec, with their tensor-name prefixes below this
mixer's).  Each keeps what it needs between steps: the requirement of this mixer is the tuple of theirs, and the
cache it is handed has one part for each (``cache.parts``, in that order).  The weighted sum is taken in float32.
"""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import MIXERS, Mixer


@MIXERS.register("parallel")
class ParallelMixer(Mixer):
    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        prefixes = spec.get("prefixes", {})
        self.left = MIXERS.build(spec["left"], prefix + prefixes.get("left", "left."), dtype, device)
        self.right = MIXERS.build(spec["right"], prefix + prefixes.get("right", "right."), dtype, device)
        self.left_scale = float(spec.get("left_scale", 1.0))
        self.right_scale = float(spec.get("right_scale", 1.0))
        self.ctas_per_work_unit = max(self.left.ctas_per_work_unit, self.right.ctas_per_work_unit)

    def parts(self):
        return [self.left, self.right]

    def cache_requirement(self):
        return (self.left.cache_requirement(), self.right.cache_requirement())

    def _caches(self, cache):
        """The parts of ``cache`` in the order of (left, right); a mixer that keeps nothing gets None."""
        it = iter(cache.parts)
        return [next(it) if m.cache_requirement() is not None else None for m in (self.left, self.right)]

    # forward_pair: the two outputs and their factors as they are, for a block whose write-back takes the sum in
    # (parts.block.HyperPreNormBlock); forward: the sum itself
    produces_pairs = True

    def forward_pair(self, h, ctx, cache) -> "K.WeightedPair":
        cl, cr = self._caches(cache)
        return K.WeightedPair(self.left.forward(h, ctx, cl), self.right.forward(h, ctx, cr), self.left_scale, self.right_scale)

    def forward(self, h, ctx, cache):
        return self.forward_pair(h, ctx, cache).materialize()
