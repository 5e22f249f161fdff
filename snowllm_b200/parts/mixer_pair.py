"""Two mixers side by side on the same input (kind ``side_by_side``).

Both read the same normalised rows; each output is divided by its root mean square over the model width
and weighted with a weight of its own; the result is ``weights[0]`` times the first plus ``weights[1]``
times the second (one half each for the mean).  The two mixers are parts of any registered kinds, given as
``PartSpec``s; each keeps the cache it asks for, so the pair's ``cache_spec()`` is the tuple of theirs (pages
of one and a state slot of the other, say) and its view a tuple in the same order."""
from __future__ import annotations

from ..errors import ConfigError
from ..ops import kernels
from .base import Part
from .registry import lookup, register_mixer
from .spec import INIT_ONES, KEEP_SMALL, PartSpec, TensorSpec


class SideBySide(Part):
    def __init__(self, dtype, names, *, hidden_size: int, left: PartSpec, right: PartSpec, eps: float,
                 weights=(0.5, 0.5)):
        super().__init__(dtype, names)
        self.hidden_size, self.eps = hidden_size, float(eps)
        self.mix = (float(weights[0]), float(weights[1]))
        self.left = lookup("mixer", left.kind)(dtype, left.names, **dict(left.params))
        self.right = lookup("mixer", right.kind)(dtype, right.names, **dict(right.params))
        self.libraries = tuple(dict.fromkeys(self.left.libraries + self.right.libraries + ("streams",)))
        self._specs = (self.left.cache_spec(), self.right.cache_spec())
        for spec in self._specs:
            if isinstance(spec, (tuple, list)):
                raise ConfigError("a mixer of a pair asks for one cache at most")
        self.left_weight = self.right_weight = None

    def parts(self):
        return (self.left, self.right)

    def cache_spec(self):
        specs = tuple(s for s in self._specs if s is not None)
        return specs if len(specs) != 1 else specs[0]

    def declare(self, has):
        W, n = self.hidden_size, self.names
        return [TensorSpec("left_out", n["left_out"], (W,), INIT_ONES, KEEP_SMALL),
                TensorSpec("right_out", n["right_out"], (W,), INIT_ONES, KEEP_SMALL)]

    def bind(self, tensors):
        self.left_weight, self.right_weight = tensors["left_out"], tensors["right_out"]
        if self.left_weight.dtype != self.right_weight.dtype:
            self.left_weight, self.right_weight = self.left_weight.float(), self.right_weight.float()

    def _views(self, cache):
        """Each mixer's own view out of the pair's."""
        have = [s is not None for s in self._specs]
        if all(have):
            return cache[0], cache[1]
        return (cache if have[0] else None), (cache if have[1] else None)

    def forward(self, ctx, x, cache, owns_cache=True):
        lc, rc = self._views(cache)
        a = self.left.forward(ctx, x, lc, owns_cache)
        ctx.tap("left_out", a)
        b = self.right.forward(ctx, x, rc, owns_cache)
        ctx.tap("right_out", b)
        return kernels.pair_norm_mix(a, b, self.left_weight, self.right_weight, self.mix[0], self.mix[1], self.eps)


register_mixer("side_by_side", SideBySide)
