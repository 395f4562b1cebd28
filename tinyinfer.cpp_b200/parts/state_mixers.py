"""Recurrent mixers whose state per head is a float32 matrix ``S [key size, value size]``.

``gated_delta``: the gated delta rule.  ``q, k = Wq h, Wk h`` (``kv_heads x dim``), ``v = Wv h``
(``heads x vdim``); head ``a`` uses q/k head ``a // (heads / kv_heads)``.  Each of q, k, v passes
a short causal convolution over time per channel (``<name>.conv`` ``[channels, taps]``, the last
column is the token's own, zeros before a sequence's start) and silu; q and k become unit
vectors per head (``x / sqrt(sum x^2 + 1e-6)``), q also times ``dim^-1/2``.  With
``beta = sigmoid(Wb h)`` and the decay ``g = exp(-exp(A_log) softplus(Wa h + dt_bias))`` per head:

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

(the read-out sees the token's own write).  ``o`` is brought to unit root mean square over
``vdim``, multiplied by a weight of ``vdim`` elements that the heads share and by ``silu(Wg h)``;
then ``Wo``.

``matrix_memory``: a matrix memory with exponential input and forget gates under a running
maximum (the mLSTM cell of xLSTM).  ``q = Wq h * dim^-1/2``, ``k = Wk h`` (``heads x dim``),
``v = Wv h`` (``heads x vdim``); per head the log gates ``i = cap tanh((Wi h + bi) / cap)`` and
``f = logsigmoid(cap tanh((Wf h + bf) / cap))``.  With ``m`` the running maximum (0 at the start):

    m' = max(f + m, i);   S <- e^(f + m - m') S + e^(i - m') k v^T;   n likewise with k alone;
    o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)

``o`` is brought to unit root mean square per head, the heads side by side are multiplied by a
weight per element and by ``sigmoid(Wg h)``; then ``Wo``.

All projections of a mixer run as one product.  State, gates, decays, unit norms and the
recurrence are float32 whatever the activation dtype; the state of a request (and the
convolution's last ``taps - 1`` inputs) lives in its state slot and starts at zero, so a prompt
cut anywhere continues exactly.
"""
from __future__ import annotations

import torch

from .base import MATRIX, NORM_WEIGHT, NORM_ZERO, FixedStateSpec, Part, WeightSpec, as_float32, register_part


def _stack_rows(mats, width):
    """The matrices one below the other (widened if their storage differs), with zero rows up to
    a multiple of 16 that the tensor-core products take."""
    if len({m.dtype for m in mats}) > 1:
        mats = [m.to(torch.float32) for m in mats]
    rows = sum(m.shape[0] for m in mats)
    if rows % 16:
        mats = list(mats) + [torch.zeros((16 - rows % 16, width), dtype=mats[0].dtype, device=mats[0].device)]
    return torch.cat(mats, dim=0)


class GatedDeltaMixer(Part):
    category = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 conv_taps: int, norm_eps: float):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} key heads evenly")
        self.hidden_size = int(hidden_size)
        self.num_heads, self.num_kv_heads = int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.conv_taps, self.eps = int(conv_taps), float(norm_eps)
        if self.conv_taps < 1:
            raise ValueError(f"the short convolution needs at least one tap, got {conv_taps}")
        self.nk, self.nv = self.num_kv_heads * self.head_dim, self.num_heads * self.v_head_dim
        self.conv_channels = 2 * self.nk + self.nv
        self.state_floats = self.num_heads * self.head_dim * self.v_head_dim
        self.w_in = self.w_o = self.conv_w = self.a_log = self.dt_bias = self.norm = None

    def weight_specs(self):
        h, taps = self.hidden_size, self.conv_taps
        return {"q": WeightSpec((self.nk, h), MATRIX), "q.conv": WeightSpec((self.nk, taps), MATRIX),
                "k": WeightSpec((self.nk, h), MATRIX), "k.conv": WeightSpec((self.nk, taps), MATRIX),
                "v": WeightSpec((self.nv, h), MATRIX), "v.conv": WeightSpec((self.nv, taps), MATRIX),
                "b": WeightSpec((self.num_heads, h), MATRIX), "a": WeightSpec((self.num_heads, h), MATRIX),
                "A_log": WeightSpec((self.num_heads,), NORM_ZERO), "dt_bias": WeightSpec((self.num_heads,), NORM_ZERO),
                "norm": WeightSpec((self.v_head_dim,), NORM_WEIGHT), "g": WeightSpec((self.nv, h), MATRIX),
                "o": WeightSpec((h, self.nv), MATRIX)}

    def load_weights(self, tensors, ops):
        # columns of the product: q, k, v (what the convolution reads), the gate, beta's logit, the decay's argument
        self.w_in = ops.pack_linear(_stack_rows([tensors[n] for n in ("q", "k", "v", "g", "b", "a")], self.hidden_size))
        self.conv_w = torch.cat([as_float32(tensors[n + ".conv"]) for n in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = as_float32(tensors["A_log"]).contiguous()
        self.dt_bias = as_float32(tensors["dt_bias"]).contiguous()
        self.norm = as_float32(tensors["norm"]).contiguous()
        self.w_o = ops.pack_linear(tensors["o"])

    def cache_spec(self):
        return FixedStateSpec((self.state_floats + (self.conv_taps - 1) * self.conv_channels,), torch.float32)

    def forward(self, ops, h, residual, step, cache):
        t, dev = h.shape[0], h.device
        c, nk, nv, nh = self.conv_channels, self.nk, self.nv, self.num_heads
        proj = torch.empty((t, self.w_in.shape[0]), dtype=torch.float32, device=dev)
        ops.linear(h, self.w_in, proj)
        qkv = torch.empty((t, c), dtype=torch.float32, device=dev)
        ops.causal_conv(proj[:, :c], self.conv_w, step, cache, self.state_floats, qkv, silu=True, renew=True)
        out = torch.empty((t, nv), dtype=h.dtype, device=dev)
        ops.matrix_state("delta", qkv[:, :nk], qkv[:, nk:2 * nk], qkv[:, 2 * nk:], proj[:, c + nv:c + nv + nh],
                         proj[:, c + nv + nh:c + nv + 2 * nh], self.a_log, self.dt_bias, step, cache, out,
                         heads=nh, kv_heads=self.num_kv_heads, dk=self.head_dim, dv=self.v_head_dim, eps=self.eps,
                         norm_weight=self.norm, gate=proj[:, c:c + nv], gate_act="silu")
        ops.linear(out, self.w_o, residual, accumulate=True)


class MatrixMemoryMixer(Part):
    category = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, gate_cap: float,
                 norm_eps: float):
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.cap, self.eps = float(gate_cap), float(norm_eps)
        if not self.cap > 0:
            raise ValueError(f"the gates' cap must be positive, got {gate_cap}")
        self.nk, self.nv = self.num_heads * self.head_dim, self.num_heads * self.v_head_dim
        self.w_in = self.w_o = self.bias_i = self.bias_f = self.norm = None

    def weight_specs(self):
        h, nh = self.hidden_size, self.num_heads
        return {"q": WeightSpec((self.nk, h), MATRIX), "k": WeightSpec((self.nk, h), MATRIX),
                "v": WeightSpec((self.nv, h), MATRIX), "g": WeightSpec((self.nv, h), MATRIX),
                "i": WeightSpec((nh, h), MATRIX), "i.b": WeightSpec((nh,), NORM_ZERO),
                "f": WeightSpec((nh, h), MATRIX), "f.b": WeightSpec((nh,), NORM_WEIGHT),
                "norm": WeightSpec((self.nv,), NORM_WEIGHT), "o": WeightSpec((h, self.nv), MATRIX)}

    def load_weights(self, tensors, ops):
        self.w_in = ops.pack_linear(_stack_rows([tensors[n] for n in ("q", "k", "v", "g", "i", "f")], self.hidden_size))
        self.bias_i = as_float32(tensors["i.b"]).contiguous()
        self.bias_f = as_float32(tensors["f.b"]).contiguous()
        self.norm = as_float32(tensors["norm"]).contiguous()
        self.w_o = ops.pack_linear(tensors["o"])

    def cache_spec(self):
        # every head's S with the normaliser n as one more column, and the running maximum per head
        nh = self.num_heads
        return FixedStateSpec((nh * self.head_dim * (self.v_head_dim + 1) + nh,), torch.float32)

    def forward(self, ops, h, residual, step, cache):
        t, dev = h.shape[0], h.device
        nk, nv, nh = self.nk, self.nv, self.num_heads
        proj = torch.empty((t, self.w_in.shape[0]), dtype=torch.float32, device=dev)
        ops.linear(h, self.w_in, proj)
        out = torch.empty((t, nv), dtype=h.dtype, device=dev)
        at_g, at_i = 2 * nk + nv, 2 * nk + 2 * nv
        ops.matrix_state("gated_sum", proj[:, :nk], proj[:, nk:2 * nk], proj[:, 2 * nk:at_g], proj[:, at_i:at_i + nh],
                         proj[:, at_i + nh:at_i + 2 * nh], self.bias_i, self.bias_f, step, cache, out,
                         heads=nh, kv_heads=nh, dk=self.head_dim, dv=self.v_head_dim, eps=self.eps,
                         norm_weight=self.norm, norm_per_row=True, gate=proj[:, at_g:at_i], gate_act="sigmoid",
                         cap=self.cap)
        ops.linear(out, self.w_o, residual, accumulate=True)


register_part("mixer", "gated_delta", GatedDeltaMixer)
register_part("mixer", "matrix_memory", MatrixMemoryMixer)
