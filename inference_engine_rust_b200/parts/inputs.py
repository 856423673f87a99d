"""Step inputs: parts that run once per step on the embedded rows, before the first block."""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..weights.loader import TensorSpec
from .base import Runtime, StepContext, StepInput, part_class, register_part


class EmbedNorm(StepInput):
    """A norm on the embedded rows, in place (spec: "norm" = the norm's own spec).  Its tensors: "norm"
    (the norm's weight) and "norm.<local>" for the norm's other tensors (a bias "norm.b")."""
    graph_safe = True

    def __init__(self, spec, hidden_size: int, vocab_size: int, rt: Runtime):
        ns = spec["norm"]
        self.norm = part_class("norm", ns.kind)(ns, hidden_size, rt)

    def _names(self) -> Dict[str, str]:
        return {local: "norm" if local == "weight" else "norm." + local for local in self.norm.tensor_specs()}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = self.norm.tensor_specs()
        return {name: specs[local] for local, name in self._names().items()}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.norm.load({local: tensors[name] for local, name in self._names().items()})

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.norm.weight, getattr(self.norm, "bias", None)) if t is not None)

    def prepare(self, tokens, x, ctx: StepContext) -> None:
        self.norm.forward(x, x, ctx, rows=ctx.n_tokens)


register_part("input", "embed_norm", EmbedNorm)
