"""Two mixers side by side on the same input: result = left_scale * left(h) + right_scale * right(h).

The spec names the two mixers (`left`, `right`: PartSpecs of registered mixer kinds) and their factors.
Each sub-mixer finds its tensors under `left.` / `right.` of the layer's mixer prefix and gets a cache or
state of its own (the layer's cache request is the pair, its view the pair of views).  The factors are
handed to the sub-mixers as their `out_scale`, so both add straight into the same buffer and nothing is
combined afterwards; a mixer kind can be used here if it declares `takes_out_scale`.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..config.specs import PartSpec
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext, part_class, register_part

SIDES = ("left", "right")


class ParallelMixers(Mixer):
    def __init__(self, spec, rt: Runtime):
        self.rt = rt
        self.subs = []
        for side in SIDES:
            ps = spec[side]
            cls = part_class("mixer", ps.kind)
            if not getattr(cls, "takes_out_scale", False):
                raise ValueError(f"mixer kind {ps.kind!r} cannot stand in a parallel pair: it takes no out_scale")
            scale = float(spec.get(side + "_scale", 1.0)) * float(ps.get("out_scale", 1.0))
            self.subs.append(cls(PartSpec(ps.kind, {**ps.params, "out_scale": scale}), rt))

    @property
    def graph_safe(self) -> bool:
        return all(getattr(m, "graph_safe", False) for m in self.subs)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {f"{side}.{name}": ts for side, m in zip(SIDES, self.subs) for name, ts in m.tensor_specs().items()}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for side, m in zip(SIDES, self.subs):
            m.load({name[len(side) + 1:]: t for name, t in tensors.items() if name.startswith(side + ".")})

    def cache_request(self):
        return tuple(m.cache_request() for m in self.subs)

    def weight_bytes(self) -> int:
        return sum(m.weight_bytes() for m in self.subs if hasattr(m, "weight_bytes"))

    def cut_by_length_key(self):
        return ("parallel",) + tuple(getattr(m, "cut_by_length_key", lambda m=m: id(m))() for m in self.subs)

    def cut_by_length(self, pos0, cache_view) -> bool:
        return cache_view is not None and any(m.cut_by_length(pos0, v) for m, v in zip(self.subs, cache_view))

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        for m, view in zip(self.subs, cache_view):
            m.forward(xn, residual, ctx, view, writes_cache)


register_part("mixer", "parallel", ParallelMixers)
