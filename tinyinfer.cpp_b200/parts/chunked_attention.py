"""Grouped-query attention inside chunks of positions, with a norm over the whole query and key
rows, a score factor per head, a cap on the score and an output gate per head.

For token ``i`` and query head ``a`` (kv head ``a // (heads / kv_heads)``):

* ``q, k, v = Wq h, Wk h, Wv h`` (no biases); ``q`` (all heads as one row) and ``k`` likewise are
  RMS-normed with a weight per column, then the first ``rotary_dim`` elements of every head are
  turned by the position part's rule.
* key ``j <= i`` is visible when ``j // chunk == i // chunk`` (chunks are counted from the
  sequence's position 0) and, if a window is given, ``i - j < window``.
* ``score = (q . k) * scale * temp[a]``, then ``softcap * tanh(score / softcap)``; float32 softmax
  over the visible keys; weighted sum of the values (head size ``v_head_dim``).
* head ``a``'s output times ``sigmoid((Wg h)[a])``, then ``residual += Wo (.)``.

``Wq, Wk, Wv, Wg`` run as one product.  Every option can be left out (``chunk``, ``window``,
``softcap`` None; ``head_temperature``, ``head_gate`` False), and ``norm_per_head`` norms every
query and key head by itself with one weight of ``head_dim`` elements, so other designs can use the
part: with everything off it is plain causal grouped-query attention with a query/key norm.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.plan import PartSpec
from .base import MATRIX, NORM_WEIGHT, PagedKVSpec, Part, WeightSpec, as_float32, build_part, register_part


class ChunkedAttention(Part):
    category = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 scale: float, qk_norm_eps: float, position: PartSpec, chunk: Optional[int] = None,
                 window: Optional[int] = None, softcap: Optional[float] = None,
                 head_temperature: bool = True, head_gate: bool = True, norm_per_head: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} kv heads evenly")
        for name, v in (("chunk", chunk), ("window", window)):
            if v is not None and v < 1:
                raise ValueError(f"{name} must be positive, got {v}")
        self.hidden_size = int(hidden_size)
        self.num_heads, self.num_kv_heads = int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale, self.eps = float(scale), float(qk_norm_eps)
        self.chunk = None if chunk is None else int(chunk)
        self.window = None if window is None else int(window)
        self.softcap = None if softcap is None else float(softcap)
        self.head_temperature, self.head_gate = bool(head_temperature), bool(head_gate)
        # the norm of queries and keys: over the whole row with a weight per column, or over each
        # head by itself with a weight of head_dim elements that all heads share
        self.norm_per_head = bool(norm_per_head)
        self.position = build_part("position", position)
        self.nq, self.nk = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        self.nv, self.no = self.num_kv_heads * self.v_head_dim, self.num_heads * self.v_head_dim
        self.w_in = self.w_o = self.q_norm = self.k_norm = self.temp = None

    def weight_specs(self):
        h = self.hidden_size
        specs = {"q": WeightSpec((self.nq, h), MATRIX), "k": WeightSpec((self.nk, h), MATRIX),
                 "v": WeightSpec((self.nv, h), MATRIX), "o": WeightSpec((h, self.no), MATRIX),
                 "q.norm": WeightSpec((self.head_dim if self.norm_per_head else self.nq,), NORM_WEIGHT),
                 "k.norm": WeightSpec((self.head_dim if self.norm_per_head else self.nk,), NORM_WEIGHT)}
        if self.head_temperature:
            specs["temp"] = WeightSpec((self.num_heads,), NORM_WEIGHT)
        if self.head_gate:
            specs["g"] = WeightSpec((self.num_heads, h), MATRIX)
        return specs

    def load_weights(self, tensors, ops):
        mats = [tensors[n] for n in (("q", "k", "v", "g") if self.head_gate else ("q", "k", "v"))]
        if len({m.dtype for m in mats}) > 1:          # mixed storage: widen, never narrow
            mats = [m.to(torch.float32) for m in mats]
        self.w_in = ops.pack_linear(torch.cat(mats, dim=0))
        self.w_o = ops.pack_linear(tensors["o"])
        self.q_norm = as_float32(tensors["q.norm"]).contiguous()
        self.k_norm = as_float32(tensors["k.norm"]).contiguous()
        self.temp = as_float32(tensors["temp"]).contiguous() if self.head_temperature else None
        if hasattr(ops, "want_row_tiles"):
            ops.want_row_tiles(self.num_heads, self.num_kv_heads)

    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window,
                           None if self.v_head_dim == self.head_dim else self.v_head_dim, 0, self.chunk)

    def forward(self, ops, h, residual, step, cache):
        t = h.shape[0]
        proj = torch.empty((t, self.w_in.shape[0]), dtype=torch.float32, device=h.device)
        ops.linear(h, self.w_in, proj)
        q = torch.empty((t, self.nq), dtype=h.dtype, device=h.device)
        ops.qk_rownorm_rope_store(proj, self.q_norm, self.k_norm, self.eps, self.position.rotation(h.device),
                                  step, cache, q, self.num_heads, self.num_kv_heads, self.head_dim,
                                  self.v_head_dim, per_head=self.norm_per_head)
        gate = proj[:, self.nq + self.nk + self.nv:] if self.head_gate else None
        out = torch.empty((t, self.no), dtype=h.dtype, device=h.device)
        ops.attention_options(q, step, cache, out, self.num_heads, self.num_kv_heads, self.head_dim,
                              self.v_head_dim, self.scale, window=self.window, chunk=self.chunk,
                              softcap=self.softcap, head_scale=self.temp, gate=gate, gate_per_head=True)
        ops.linear(out, self.w_o, residual, accumulate=True, may_defer=True)


register_part("mixer", "chunked_attention", ChunkedAttention)
