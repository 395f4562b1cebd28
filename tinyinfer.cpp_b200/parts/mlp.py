"""SwiGLU feed-forward: ``residual += (silu(h Wgate^T) * (h Wup^T)) Wdown^T``.

``silu(g) = g / (1 + exp(-g))`` in float32 (reference: src/cuda/ffn.cu:13-15;
gate and up as one product over stacked rows, src/inference.cu:59-65).  How the
gate and up rows are stacked is the kernel set's choice (``ops.pack_gate_up``).

``xielu_mlp``: an ungated feed-forward with the xIELU activation (below).

``glu_mlp``: a gated feed-forward with a named activation and its constants (below).
"""
from __future__ import annotations

import math

import torch

from .base import MATRIX, Part, WeightSpec, register_part


class SwiGLU(Part):
    category = "ffn"

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def weight_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {
            "gate_proj.weight": WeightSpec((i, h), MATRIX),
            "up_proj.weight": WeightSpec((i, h), MATRIX),
            "down_proj.weight": WeightSpec((h, i), MATRIX),
        }

    def load_weights(self, tensors, ops):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        self.w_gate_up = ops.pack_gate_up(g, u)
        self.w_down = ops.pack_linear(tensors["down_proj.weight"])

    def forward(self, ops, h, residual, step):
        ops.swiglu_ffn(h, self.w_gate_up, self.w_down, residual, may_defer=True)


register_part("ffn", "swiglu", SwiGLU)


def _softplus(z: float) -> float:
    return math.log1p(math.exp(-abs(z))) + max(z, 0.0)


class XieluMlp(Part):
    """``residual += Wdown act(Wup h)`` with ``act`` = xIELU and its two stored numbers ``p, q``:
    ``softplus(p) z^2 + z/2`` for ``z > 0``, ``(1/2 + softplus(q)) (exp(z) - 1 - z) + z/2`` elsewhere.
    The two factors are made once, in double precision, when the weights are loaded."""
    category = "ffn"

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_up = self.w_down = None
        self.ap = self.aq = 0.0

    def weight_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"up": WeightSpec((i, h), MATRIX), "down": WeightSpec((h, i), MATRIX),
                "act": WeightSpec((2,), MATRIX)}

    def load_weights(self, tensors, ops):
        self.w_up, self.w_down = ops.pack_linear(tensors["up"]), ops.pack_linear(tensors["down"])
        p, q = (float(v) for v in tensors["act"].to(torch.float64).cpu())
        self.ap, self.aq = _softplus(p), 0.5 + _softplus(q)

    def forward(self, ops, h, residual, step):
        y = torch.empty((h.shape[0], self.intermediate_size), dtype=h.dtype, device=h.device)
        ops.linear_xielu(h, self.w_up, self.ap, self.aq, y)
        ops.linear(y, self.w_down, residual, accumulate=True, may_defer=True)


register_part("ffn", "xielu_mlp", XieluMlp)


class GatedMlp(Part):
    """``residual += Wdown act(Wgate h, Wup h)`` with the gated activation ``activation``:

    ``silu``     ``silu(g) u``
    ``clamped``  ``g = min(g, limit)``, ``u = clamp(u, -limit, limit)``, ``g sigmoid(alpha g) (u + 1)``

    The tensors are ``gate``, ``up`` and ``down``."""
    category = "ffn"

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "clamped", limit: float = 0.0,
                 alpha: float = 1.702):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.activation, self.limit, self.alpha = str(activation), float(limit), float(alpha)
        self.w_gate_up = self.w_down = None

    def weight_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"gate": WeightSpec((i, h), MATRIX), "up": WeightSpec((i, h), MATRIX), "down": WeightSpec((h, i), MATRIX)}

    def load_weights(self, tensors, ops):
        g, u = tensors["gate"], tensors["up"]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        self.w_gate_up = ops.pack_gate_up(g, u)
        self.w_down = ops.pack_linear(tensors["down"])

    def forward(self, ops, h, residual, step):
        ops.glu_ffn(h, self.w_gate_up, self.w_down, residual, self.activation, self.limit, self.alpha)


register_part("ffn", "glu_mlp", GatedMlp)
