"""Two mixers side by side: both read the same input, each keeps what it needs per request, and
the layer's mixer output is ``left_scale * left(h) + right_scale * right(h)``.

The two are ordinary mixer parts (for instance causal attention beside a recurrent mixer); their
tensors live under ``left.`` and ``right.``, their caches under the same names of a composite
cache slot.  Each writes its result into float32 rows of its own, which one pass then adds,
scaled, to the output.
"""
from __future__ import annotations

import torch

from ..config.plan import PartSpec
from .base import CompositeSpec, Part, build_part, register_part

SIDES = ("left", "right")


class ParallelMixers(Part):
    category = "mixer"

    def __init__(self, hidden_size: int, left: PartSpec, right: PartSpec, left_scale: float = 1.0,
                 right_scale: float = 1.0):
        self.hidden_size = int(hidden_size)
        self.sides = {"left": build_part("mixer", left), "right": build_part("mixer", right)}
        self.scales = {"left": float(left_scale), "right": float(right_scale)}

    def weight_specs(self):
        return {f"{side}.{name}": spec for side in SIDES for name, spec in self.sides[side].weight_specs().items()}

    def load_weights(self, tensors, ops):
        for side in SIDES:
            cut = side + "."
            self.sides[side].load_weights({n[len(cut):]: t for n, t in tensors.items() if n.startswith(cut)}, ops)

    def step_lists(self):
        return [sl for side in SIDES for sl in self.sides[side].step_lists()]

    def cache_spec(self):
        return CompositeSpec(tuple((side, self.sides[side].cache_spec()) for side in SIDES))

    def forward(self, ops, h, residual, step, cache):
        rows = torch.zeros((2, h.shape[0], self.hidden_size), dtype=torch.float32, device=h.device)
        for i, side in enumerate(SIDES):
            self.sides[side].forward(ops, h, rows[i], step, cache.child(side))
        ops.add_scaled(residual, rows[0], self.scales["left"], rows[1], self.scales["right"])


register_part("mixer", "parallel_mixers", ParallelMixers)
