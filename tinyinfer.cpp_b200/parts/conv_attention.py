"""Grouped-query attention whose projections pass a short convolution over time and whose values
carry their position.

For token ``i`` and query head ``a`` (kv head ``a // (heads / kv_heads)``):

* ``q, k, v = Wq h, Wk h, Wv h`` (no biases); with ``conv_taps`` each channel of the three then
  passes a causal convolution over time, ``y_t = sum_j w[:, j] u_(t - taps + 1 + j)`` (tensors
  ``q.conv``, ``k.conv``, ``v.conv`` ``[channels, taps]``, zeros before the sequence's start); the
  request keeps its last ``taps - 1`` projected rows.
* the first ``rotary_dim`` elements of every query and key head are turned by the position part's
  rule; no norm.
* ``value_rotation`` (a position part over ``v_head_dim``): the value of position ``j`` is turned by
  ``j`` before it is cached, and head ``a``'s output at position ``i``, the weighted sum of such
  values, is turned back by ``-i``.  A sum of values that were turned by their own positions,
  turned back by the reader's, depends on the distances ``i - j`` alone.
* key ``j <= i`` is visible (and ``i - j < window`` if a window is given); ``score = (q . k) * scale``;
  float32 softmax; ``sink_one`` counts one more unit in the denominator, ``p_j = exp(s_j) / (1 +
  sum exp(s))``: a key whose score is 0 and which has no value.
* ``gate``: the heads side by side times ``sigmoid(Wg h)``, element by element; then
  ``residual += Wo (.)``.

``Wq, Wk, Wv, Wg`` run as one product.  Every option can be left out.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.plan import PartSpec
from .base import (MATRIX, CompositeSpec, FixedStateSpec, PagedKVSpec, Part, WeightSpec, as_float32, build_part,
                   register_part)


class ConvAttention(Part):
    category = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 scale: float, position: PartSpec, value_rotation: Optional[PartSpec] = None, conv_taps: int = 0,
                 window: Optional[int] = None, sink_one: bool = False, gate: bool = True):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} kv heads evenly")
        if window is not None and window < 1:
            raise ValueError(f"window must be positive, got {window}")
        self.hidden_size = int(hidden_size)
        self.num_heads, self.num_kv_heads = int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale, self.conv_taps = float(scale), int(conv_taps)
        self.window = None if window is None else int(window)
        self.sink_one, self.has_gate = bool(sink_one), bool(gate)
        self.position = build_part("position", position)
        self.value_position = None if value_rotation is None else build_part("position", value_rotation)
        self.nq, self.nk = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        self.nv, self.no = self.num_kv_heads * self.v_head_dim, self.num_heads * self.v_head_dim
        self.conv_channels = self.nq + self.nk + self.nv
        self.w_in = self.w_o = self.conv_w = self.sink = None

    def weight_specs(self):
        h, taps = self.hidden_size, self.conv_taps
        specs = {"q": WeightSpec((self.nq, h), MATRIX), "k": WeightSpec((self.nk, h), MATRIX),
                 "v": WeightSpec((self.nv, h), MATRIX), "o": WeightSpec((h, self.no), MATRIX)}
        if taps:
            specs.update({"q.conv": WeightSpec((self.nq, taps), MATRIX), "k.conv": WeightSpec((self.nk, taps), MATRIX),
                          "v.conv": WeightSpec((self.nv, taps), MATRIX)})
        if self.has_gate:
            specs["g"] = WeightSpec((self.no, h), MATRIX)
        return specs

    def load_weights(self, tensors, ops):
        mats = [tensors[n] for n in (("q", "k", "v", "g") if self.has_gate else ("q", "k", "v"))]
        if len({m.dtype for m in mats}) > 1:          # mixed storage: widen, never narrow
            mats = [m.to(torch.float32) for m in mats]
        self.w_in = ops.pack_linear(torch.cat(mats, dim=0))
        self.w_o = ops.pack_linear(tensors["o"])
        if self.conv_taps:
            self.conv_w = torch.cat([as_float32(tensors[n + ".conv"]) for n in ("q", "k", "v")], dim=0).contiguous()
        if self.sink_one:                             # one more logit of 0 in every head's softmax
            self.sink = torch.zeros((self.num_heads,), dtype=torch.float32, device=self.w_o.device)
        if hasattr(ops, "want_row_tiles"):
            ops.want_row_tiles(self.num_heads, self.num_kv_heads)

    def _paged_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window,
                           None if self.v_head_dim == self.head_dim else self.v_head_dim)

    def cache_spec(self):
        if self.conv_taps <= 1:
            return self._paged_spec()
        return CompositeSpec((("conv", FixedStateSpec(((self.conv_taps - 1) * self.conv_channels,), torch.float32)),
                              ("kv", self._paged_spec())))

    def forward(self, ops, h, residual, step, cache):
        t, dev, c = h.shape[0], h.device, self.conv_channels
        kept, pages = (cache["conv"], cache["kv"]) if self.conv_taps > 1 else (None, cache)
        proj = torch.empty((t, self.w_in.shape[0]), dtype=torch.float32, device=dev)
        ops.linear(h, self.w_in, proj)
        qkv = proj
        if self.conv_taps:
            qkv = torch.empty((t, c), dtype=torch.float32, device=dev)
            ops.causal_conv(proj[:, :c], self.conv_w, step, kept, 0, qkv, renew=True)
        q = torch.empty((t, self.nq), dtype=h.dtype, device=dev)
        v_rot = None if self.value_position is None else self.value_position.rotation(dev)
        ops.qkv_turn_store(qkv, self.position.rotation(dev), v_rot, step, pages, q, self.num_heads,
                           self.num_kv_heads, self.head_dim, self.v_head_dim)
        gate = proj[:, c:] if self.has_gate else None
        out = torch.empty((t, self.no), dtype=h.dtype, device=dev)
        if v_rot is None:
            ops.attention_options(q, step, pages, out, self.num_heads, self.num_kv_heads, self.head_dim,
                                  self.v_head_dim, self.scale, window=self.window, sink=self.sink, gate=gate)
        else:
            ops.attention_options(q, step, pages, out, self.num_heads, self.num_kv_heads, self.head_dim,
                                  self.v_head_dim, self.scale, window=self.window, sink=self.sink)
            ops.turn_rows(out, step, v_rot, self.num_heads, self.v_head_dim, back=True, gate=gate)
        ops.linear(out, self.w_o, residual, accumulate=True, may_defer=True)


register_part("mixer", "conv_attention", ConvAttention)
