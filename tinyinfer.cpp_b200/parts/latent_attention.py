"""Attention whose keys and values are made from one cached latent row per token.

For token ``i`` with input ``h``: ``q = Wq h``, per head ``[dk plain | dr rotated]``;
``Wdkv h`` gives ``rank + dr`` numbers: the first ``rank``, RMS-normed with a weight, are the
latent ``c``; the last ``dr`` are one rotated key part shared by all heads.  Head ``a``'s plain
key is ``Wuk_a c`` and its value ``Wuv_a c``; ``score = (q_plain . k_plain + q_rot . k_rot) *
scale``; causal softmax whose denominator also counts ``exp(sink[a])`` (a logit without a value);
``residual += Wo (heads)``.

With ``q_rank`` the queries pass a latent of their own: ``c_q = RMSnorm(Wdq h)`` with a weight
(``dq``, ``dq.norm``), ``q = Wuq c_q`` (``uq``), instead of ``q = Wq h``.  A window limits the keys
to ``i - j < window``.

Only ``[c | k_rot]`` is cached, one row per token.  The heads' keys and values are never built:
since ``q_plain . (Wuk_a c) = (Wuk_a^T q_plain) . c``, the query is carried into the latent's space
(``head_project`` with ``Wuk_a^T``), attention runs with one shared row as key (``rank + dr``
elements) and value (its first ``rank``), and the result is carried back by ``Wuv_a`` before the
output projection.  A prompt portion and a single decoded token take the same path.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.plan import PartSpec
from .base import MATRIX, NORM_WEIGHT, NORM_ZERO, PagedKVSpec, Part, WeightSpec, as_float32, build_part, register_part


class LatentAttention(Part):
    category = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int,
                 kv_rank: int, scale: float, norm_eps: float, position: PartSpec, sink: bool = True,
                 window: Optional[int] = None, q_rank: Optional[int] = None):
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.rot_dim, self.v_head_dim = int(head_dim), int(rot_dim), int(v_head_dim)
        self.rank, self.scale, self.eps = int(kv_rank), float(scale), float(norm_eps)
        self.has_sink = bool(sink)
        self.window = None if window is None else int(window)
        self.q_rank = None if q_rank is None else int(q_rank)
        self.position = build_part("position", position)
        self.nq = self.num_heads * (self.head_dim + self.rot_dim)
        self.row = self.rank + self.rot_dim
        self.w_in = self.w_o = self.latent_norm = self.sink = self.w_uk = self.w_uv = None
        self.w_uq = self.q_norm = None

    def weight_specs(self):
        h, nh = self.hidden_size, self.num_heads
        q = {"q": WeightSpec((self.nq, h), MATRIX)} if self.q_rank is None else {
            "dq": WeightSpec((self.q_rank, h), MATRIX), "dq.norm": WeightSpec((self.q_rank,), NORM_WEIGHT),
            "uq": WeightSpec((self.nq, self.q_rank), MATRIX)}
        specs = {**q, "dkv": WeightSpec((self.row, h), MATRIX),
                 "dkv.norm": WeightSpec((self.rank,), NORM_WEIGHT),
                 "uk": WeightSpec((nh * self.head_dim, self.rank), MATRIX),
                 "uv": WeightSpec((nh * self.v_head_dim, self.rank), MATRIX),
                 "o": WeightSpec((h, nh * self.v_head_dim), MATRIX)}
        if self.has_sink:
            specs["sink"] = WeightSpec((nh,), NORM_ZERO)
        return specs

    def load_weights(self, tensors, ops):
        if self.q_rank is None:
            q, dkv = tensors["q"], tensors["dkv"]
            if q.dtype != dkv.dtype:
                q, dkv = q.to(torch.float32), dkv.to(torch.float32)
            self.w_in = ops.pack_linear(torch.cat([q, dkv], dim=0))
        else:                                         # the two latents as one product: [query latent | latent | key part]
            dq, dkv = tensors["dq"], tensors["dkv"]
            if dq.dtype != dkv.dtype:
                dq, dkv = dq.to(torch.float32), dkv.to(torch.float32)
            mats = [dq, dkv]
            rows = dq.shape[0] + dkv.shape[0]
            if rows % 16:                             # zero rows up to a width the tensor-core products take
                mats.append(torch.zeros((16 - rows % 16, self.hidden_size), dtype=dq.dtype, device=dq.device))
            self.w_in = ops.pack_linear(torch.cat(mats, dim=0))
            self.w_uq = ops.pack_linear(tensors["uq"])
            self.q_norm = as_float32(tensors["dq.norm"]).contiguous()
        self.w_o = ops.pack_linear(tensors["o"])
        self.latent_norm = as_float32(tensors["dkv.norm"]).contiguous()
        self.sink = as_float32(tensors["sink"]).contiguous() if self.has_sink else None
        nh = self.num_heads
        # [heads, dk, rank]: a head's plain query times this lands in the latent's space
        self.w_uk = tensors["uk"].view(nh, self.head_dim, self.rank).contiguous()
        # [heads, rank, dv]: a head's weighted sum of latents times this is its value
        self.w_uv = tensors["uv"].view(nh, self.v_head_dim, self.rank).transpose(1, 2).contiguous()
        if hasattr(ops, "want_row_tiles"):
            ops.want_row_tiles(nh, 1)

    def cache_spec(self):
        return PagedKVSpec(1, self.row, self.window, 0)

    def forward(self, ops, h, residual, step, cache):
        t, nh = h.shape[0], self.num_heads
        proj = torch.empty((t, self.w_in.shape[0]), dtype=torch.float32, device=h.device)
        ops.linear(h, self.w_in, proj)
        q_proj = None
        if self.q_rank is not None:                   # the queries through their own normed latent
            q_lat = torch.empty((t, self.q_rank), dtype=h.dtype, device=h.device)
            ops.slice_rmsnorm(proj[:, :self.q_rank], self.q_norm, self.eps, q_lat)
            q_proj = torch.empty((t, self.nq), dtype=torch.float32, device=h.device)
            ops.linear(q_lat, self.w_uq, q_proj)
            proj = proj[:, self.q_rank:]
        q_plain = torch.empty((t, nh * self.head_dim), dtype=h.dtype, device=h.device)
        q_full = torch.empty((t, nh, self.row), dtype=h.dtype, device=h.device)
        ops.latent_prepare(proj, self.latent_norm, self.eps, self.position.rotation(h.device), step, cache,
                           q_plain, q_full, nh, self.head_dim, self.rot_dim, self.rank, q_proj=q_proj)
        ops.head_project(q_plain.view(t, nh, self.head_dim), self.w_uk, q_full[:, :, :self.rank])
        mixed = torch.empty((t, nh, self.rank), dtype=h.dtype, device=h.device)
        ops.attention_options(q_full.view(t, nh * self.row), step, cache, mixed.view(t, nh * self.rank), nh, 1,
                              self.row, self.rank, self.scale, window=self.window, sink=self.sink,
                              shared_rows=True)
        out = torch.empty((t, nh, self.v_head_dim), dtype=h.dtype, device=h.device)
        ops.head_project(mixed, self.w_uv, out)
        ops.linear(out.view(t, nh * self.v_head_dim), self.w_o, residual, accumulate=True, may_defer=True)


register_part("mixer", "latent_attention", LatentAttention)
