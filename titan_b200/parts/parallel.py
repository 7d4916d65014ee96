"""Several mixers side by side as one mixer: every branch reads the same input rows and adds its own result, times its own
factor, into the same sum.

    out += sum_b scale_b * mixer_b(h)

``MixerSpec.extra["branches"]`` is a tuple of ``MixerSpec``, any registered kinds (softmax attention beside a recurrence,
say).  A branch's factor is its own option ``output_scale`` (a branch applies it to the rows that enter its output
projection, in float32), and its tensors live under its own prefix inside this mixer's.  What the mixer asks of the cache is
the tuple of what its branches ask, in their order; the cache hands back a tuple of views in the same order.
"""
from __future__ import annotations

from typing import List

from ..weights.loader import WeightSpec
from .base import MIXERS, Mixer
from .norm import rows_of


class ParallelMixer(Mixer):
    def __init__(self, spec):
        self.spec = spec
        branches = tuple(spec.option("branches", ()))
        if not branches:
            raise ValueError("the parallel mixer needs at least one branch")
        for b in branches:
            if b.hidden_size != spec.hidden_size:
                raise ValueError(f"a branch of width {b.hidden_size} in a mixer of width {spec.hidden_size}")
            if b.cache_from is not None:
                raise ValueError("a branch of a parallel mixer keeps its own cache")
        self.branches = [MIXERS.build(b) for b in branches]

    @property
    def capturable(self):
        return all(b.capturable for b in self.branches)

    def cache_need(self):
        return tuple(b.cache_need() for b in self.branches)

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        out: List[WeightSpec] = []
        for b in self.branches:
            out += b.weight_specs(prefix + self.spec.prefix)
        return out

    def bind(self, get) -> None:
        for b in self.branches:
            b.bind(lambda name: get(self.spec.prefix + name))

    def forward(self, h, ctx, cache, out) -> None:
        if not isinstance(cache, tuple) or len(cache) != len(self.branches):
            raise TypeError("the parallel mixer takes one cache view for each of its branches")
        h = rows_of(h)
        for b, view in zip(self.branches, cache):
            b.forward(h, ctx, view, out)


MIXERS.register("parallel", ParallelMixer)
