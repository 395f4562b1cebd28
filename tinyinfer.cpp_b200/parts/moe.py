"""A routed feed-forward: per token the ``top`` of ``experts`` small gated feed-forwards, chosen
by a sigmoid router, plus an optional shared expert behind a sigmoid gate of its own.

* router logits ``z = Wr h`` in float32, scores ``s = sigmoid(z)``; the ``top`` largest are
  chosen (ties: the lower index) and their scores are the weights, as they are.
* a chosen expert ``e`` with weight ``w`` contributes ``Wdown_e (silu(Wgate_e x) * (Wup_e x))``
  with ``x = w h``: the weight scales the expert's input.  The kernels use
  ``Wgate_e (w h) = w (Wgate_e h)`` and apply ``w`` to both products in float32.
* the shared expert (sizes of its own) runs on ``h`` for every token and its output is
  multiplied by ``sigmoid(wsg . h)``, one number per token; ``wsg`` rides as one more row of the
  router's product.
* ``residual +=`` the sum.

Options for other designs: ``router = "softmax"`` takes the chosen experts' shares of the softmax
over all experts as weights (not renormalised); ``activation = (kind, limit, alpha)`` names another
gated activation for the experts (``parts/mlp.py``), and the weight then scales the expert's
output, ``w Wdown_e act(Wgate_e h, Wup_e h)``; ``shared_gated = False`` leaves the shared expert's
sigmoid gate out (no ``shared.sg``); ``shared_activation`` is the shared expert's own activation.

With the softmax router three more options.  ``identity = n``: the last ``n`` of the router's
``experts + n`` outputs are *identity experts* without tensors, whose output is the input ``h``
itself (times the weight).  ``correction``: a stored vector (``correction``) is added to the scores
for the choice alone; the weights are the scores without it.  ``groups = (count, keep)``: the router's
outputs, identity ones included, form ``count`` equal groups of neighbours; a group's value is its
largest score (with the correction), and only outputs of the ``keep`` best groups can be chosen.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import MATRIX, NORM_ZERO, Part, WeightSpec, as_float32, register_part


class RoutedExperts(Part):
    category = "ffn"

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int,
                 shared_size: Optional[int] = None, router: str = "sigmoid", activation=None,
                 shared_gated: bool = True, shared_activation=None, identity: int = 0, correction: bool = False,
                 groups=None):
        self.identity, self.has_correction = int(identity), bool(correction)
        self.groups = None if groups is None else (int(groups[0]), int(groups[1]))
        self.routed = int(experts) + self.identity         # the router's outputs
        if (self.identity or self.has_correction or self.groups) and router != "softmax":
            raise ValueError("identity experts, a correction and groups come with the softmax router")
        count, keep = self.groups or (1, 1)
        if self.identity < 0 or count < 1 or not 1 <= keep <= count or self.routed % count:
            raise ValueError(f"{self.routed} router outputs do not fall into {count} equal groups of which {keep} are kept")
        if not 1 <= top <= self.routed // count * keep:
            raise ValueError(f"{top} of {self.routed // count * keep} experts cannot be chosen")
        self.hidden_size, self.experts, self.top = int(hidden_size), int(experts), int(top)
        self.expert_size = int(expert_size)
        self.shared_size = None if shared_size is None else int(shared_size)
        if router not in ("sigmoid", "softmax"):
            raise ValueError(f"router kind {router!r}; known: sigmoid, softmax")
        self.router = router
        self.activation = None if activation is None else (str(activation[0]), float(activation[1]), float(activation[2]))
        self.shared_activation = None if shared_activation is None else (
            str(shared_activation[0]), float(shared_activation[1]), float(shared_activation[2]))
        self.shared_gated = bool(shared_gated)
        self.w_router = self.w_gate = self.w_up = self.w_down = None
        self.w_shared_gate_up = self.w_shared_down = None

    def weight_specs(self):
        h, f = self.hidden_size, self.expert_size
        specs = {"router": WeightSpec((self.routed, h), MATRIX)}
        if self.has_correction:
            specs["correction"] = WeightSpec((self.routed,), NORM_ZERO)
        for e in range(self.experts):
            specs[f"e{e}.gate"] = WeightSpec((f, h), MATRIX)
            specs[f"e{e}.up"] = WeightSpec((f, h), MATRIX)
            specs[f"e{e}.down"] = WeightSpec((h, f), MATRIX)
        if self.shared_size is not None:
            s = self.shared_size
            specs.update({"shared.gate": WeightSpec((s, h), MATRIX), "shared.up": WeightSpec((s, h), MATRIX),
                          "shared.down": WeightSpec((h, s), MATRIX)})
            if self.shared_gated:
                specs["shared.sg"] = WeightSpec((1, h), MATRIX)
        return specs

    def load_weights(self, tensors, ops):
        def stacked(kind):
            mats = [tensors[f"e{e}.{kind}"] for e in range(self.experts)]
            if len({m.dtype for m in mats}) > 1:
                mats = [m.to(torch.float32) for m in mats]
            return torch.stack(mats, dim=0).contiguous()

        router = [tensors["router"]]
        if self.shared_size is not None:
            if self.shared_gated:
                router.append(tensors["shared.sg"])
            g, u = tensors["shared.gate"], tensors["shared.up"]
            if g.dtype != u.dtype:
                g, u = g.to(torch.float32), u.to(torch.float32)
            self.w_shared_gate_up = ops.pack_gate_up(g, u)
            self.w_shared_down = ops.pack_linear(tensors["shared.down"])
        if len({m.dtype for m in router}) > 1:
            router = [m.to(torch.float32) for m in router]
        rows = sum(m.shape[0] for m in router)
        if rows % 16:                          # zero rows up to a width the tensor-core products take
            router.append(torch.zeros((16 - rows % 16, self.hidden_size), dtype=router[0].dtype,
                                      device=router[0].device))
        self.w_router = ops.pack_linear(torch.cat(router, dim=0))
        self.correction = as_float32(tensors["correction"]).contiguous() if self.has_correction else None
        self.w_experts = ops.pack_experts(stacked("gate"), stacked("up"), stacked("down"))

    def forward(self, ops, h, residual, step):
        t = h.shape[0]
        logits = torch.empty((t, self.w_router.shape[0]), dtype=torch.float32, device=h.device)
        ops.linear(h, self.w_router, logits)
        ids = torch.empty((t, self.top), dtype=torch.int32, device=h.device)
        weights = torch.empty((t, self.top), dtype=torch.float32, device=h.device)
        shared_gate = None
        if self.shared_size is not None and self.shared_gated:
            shared_gate = torch.empty((t,), dtype=torch.float32, device=h.device)
        general = bool(self.identity or self.has_correction or self.groups)
        if general:
            count, keep = self.groups or (1, 1)
            ops.router_choose(logits, self.routed, self.top, ids, weights, self.correction, count, keep)
        else:
            ops.router_topk(logits, self.experts, self.top, ids, weights, shared_gate, softmax=self.router == "softmax")
        shared = None
        plain = self.activation is None and self.shared_activation is None and self.shared_gated
        if self.shared_size is not None and plain:
            shared = (self.w_shared_gate_up, self.w_shared_down, shared_gate)
        if self.identity:
            ops.routed_experts(h, self.w_experts, ids, weights, residual, shared, act=self.activation, identity=True)
        else:
            ops.routed_experts(h, self.w_experts, ids, weights, residual, shared, act=self.activation)
        if self.shared_size is not None and not plain:
            # a shared expert with an activation of its own, or without a gate: a feed-forward beside the routed ones
            kind, limit, alpha = self.shared_activation or ("silu", 0.0, 0.0)
            if shared_gate is None:
                ops.glu_ffn(h, self.w_shared_gate_up, self.w_shared_down, residual, kind, limit, alpha)
            else:
                ops.glu_ffn(h, self.w_shared_gate_up, self.w_shared_down, residual, kind, limit, alpha,
                            row_scale=shared_gate)


register_part("ffn", "routed_experts", RoutedExperts)
