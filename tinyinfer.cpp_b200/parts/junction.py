"""Where the schedule enters a pass over a run of layers that is walked several times.

``loop_input``: before the first layer of pass ``t`` (``t = 0, 1, ...``) the residual stream
becomes ``x <- W [x ; x0] + s_t``, with ``x0`` the embedding output, ``W`` ``[width, 2 width]``
(tensor ``in``, the columns of ``x`` first) and ``s`` ``[passes, width]`` (tensor ``step``).  The
product reads ``[x ; x0]`` in the activation dtype and lands in float32, where ``s_t`` is added.
"""
from __future__ import annotations

import torch

from .base import MATRIX, NORM_ZERO, Part, WeightSpec, as_float32, register_part


class LoopInput(Part):
    category = "junction"

    def __init__(self, hidden_size: int, passes: int):
        self.hidden_size, self.passes = int(hidden_size), int(passes)
        if self.passes < 1:
            raise ValueError(f"a run of layers is walked at least once, got {passes} passes")
        self.w_in = self.steps = None

    def weight_specs(self):
        n = self.hidden_size
        return {"in": WeightSpec((n, 2 * n), MATRIX), "step": WeightSpec((self.passes, n), NORM_ZERO)}

    def load_weights(self, tensors, ops):
        self.w_in = ops.pack_linear(tensors["in"])
        self.steps = as_float32(tensors["step"]).contiguous()

    def forward(self, ops, x, x0, index, step):
        if not 0 <= index < self.passes:
            raise ValueError(f"pass {index} of {self.passes}")
        t, n = x.shape
        both = step.scratch.get("loop_input_rows")
        if both is None or both.shape[0] != t or both.dtype != step.act_dtype:
            both = torch.empty((t, 2 * n), dtype=step.act_dtype, device=x.device)
            step.scratch["loop_input_rows"] = both
            ops.causal_conv(x0, None, step, None, 0, both[:, n:])       # the embedding output, once a step
        ops.causal_conv(x, None, step, None, 0, both[:, :n])            # rows in the activation dtype
        ops.linear(both, self.w_in, x)
        ops.add_row(x, self.steps[index])


register_part("junction", "loop_input", LoopInput)
