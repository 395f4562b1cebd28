"""Token embedding and the output head.

Embedding: ``x[t] = float32(E[token[t]])`` without scaling (reference:
src/inference.cu:14-24); ``scaled_sinusoid``: the row times a constant plus a sine/cosine
wave of the token's position (``scaled``: the constant alone); ``normed``: the row under an RMSNorm with a weight of its own.  Head: ``logits = h E_out^T`` in float32, where ``E_out``
is the embedding table when the head is tied (reference: always tied,
src/inference.cu:70-71) or a table of its own.
"""
from __future__ import annotations

import torch

from .base import MATRIX, NORM_WEIGHT, NORM_ZERO, Part, WeightSpec, as_float32, register_part


class Embedding(Part):
    category = "embedding"

    def __init__(self, vocab_size: int, hidden_size: int, tensor: str = "weight"):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.tensor = str(tensor)            # the table's name behind the part's prefix
        self.table = None

    def weight_specs(self):
        return {self.tensor: WeightSpec((self.vocab_size, self.hidden_size), MATRIX)}

    def load_weights(self, tensors, ops):
        self.table = ops.pack_linear(tensors[self.tensor])

    def shared_weights(self):
        return {"weight": self.table}

    def forward(self, ops, token_ids, out):
        ops.embed(self.table, token_ids, out)


class SinusoidEmbedding(Embedding):
    """``x[t] = E[token[t]] * scale + s(p_t)``: the table's row times a constant, plus a fixed
    wave of the token's position ``p``: ``s(p)[2i] = sin(p f_i)``, ``s(p)[2i+1] = cos(p f_i)``
    with ``f_i = base ** (-2i / hidden_size)``.  ``f`` is made once on the host in double
    precision and rounded to float32; angle, sine and cosine are float32 on the device.  A tied
    head reads the table itself, without the constant."""
    wants_positions = True

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, base: float = 10000.0,
                 tensor: str = "weight"):
        super().__init__(vocab_size, hidden_size)
        self.scale, self.base, self.tensor = float(scale), float(base), str(tensor)
        self.freq = None

    def weight_specs(self):
        return {self.tensor: WeightSpec((self.vocab_size, self.hidden_size), MATRIX)}

    def load_weights(self, tensors, ops):
        self.table = ops.pack_linear(tensors[self.tensor])
        i = torch.arange((self.hidden_size + 1) // 2, dtype=torch.float64)
        freq = torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * i / self.hidden_size)
        self.freq = freq.to(torch.float32).to(self.table.device)

    def forward(self, ops, token_ids, out, positions):
        ops.embed_sinusoid(self.table, token_ids, positions, self.freq, self.scale, out)


class ScaledEmbedding(SinusoidEmbedding):
    """``x[t] = E[token[t]] * scale``: the table's row times a constant, no wave."""

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, tensor: str = "weight"):
        super().__init__(vocab_size, hidden_size, scale=scale, tensor=tensor)

    def load_weights(self, tensors, ops):
        self.table = ops.pack_linear(tensors[self.tensor])


class NormedEmbedding(Embedding):
    """``x[t] = norm(E[token[t]])``: RMSNorm of the table's row (float32) with a weight of the
    model's width; ``one_plus``: the stored weight is the factor minus one."""

    def __init__(self, vocab_size: int, hidden_size: int, eps: float, tensor: str = "weight",
                 norm_tensor: str = "norm.weight", one_plus: bool = False):
        super().__init__(vocab_size, hidden_size)
        self.eps, self.tensor, self.norm_tensor = float(eps), str(tensor), str(norm_tensor)
        self.one_plus = bool(one_plus)
        self.norm_weight = None

    def weight_specs(self):
        return {self.tensor: WeightSpec((self.vocab_size, self.hidden_size), MATRIX),
                self.norm_tensor: WeightSpec((self.hidden_size,), NORM_ZERO if self.one_plus else NORM_WEIGHT)}

    def load_weights(self, tensors, ops):
        self.table = ops.pack_linear(tensors[self.tensor])
        w = as_float32(tensors[self.norm_tensor]).contiguous()
        self.norm_weight = 1.0 + w if self.one_plus else w

    def forward(self, ops, token_ids, out):
        rows = torch.empty_like(out)
        ops.embed(self.table, token_ids, rows)
        ops.rmsnorm(rows, self.norm_weight, self.eps, out)


class LMHead(Part):
    category = "head"

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool, tensor: str = "weight", softcap=None):
        self.vocab_size, self.hidden_size, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.tensor = str(tensor)
        self.softcap = None if softcap is None else float(softcap)
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"the logits' cap must be positive, got {softcap}")
        self.table = None

    def weight_specs(self):
        if self.tied:
            return {}
        return {self.tensor: WeightSpec((self.vocab_size, self.hidden_size), MATRIX)}

    def load_weights(self, tensors, ops):
        if not self.tied:
            self.table = ops.pack_linear(tensors[self.tensor])

    def tie(self, embedding: Embedding):
        self.table = embedding.shared_weights()["weight"]

    def forward(self, ops, h):
        logits = torch.empty((h.shape[0], self.vocab_size), dtype=torch.float32, device=h.device)
        ops.linear(h, self.table, logits)
        if self.softcap is not None:
            ops.cap_rows(logits, self.softcap)
        return logits


register_part("embedding", "embedding", Embedding)
register_part("embedding", "scaled_sinusoid", SinusoidEmbedding)
register_part("embedding", "scaled", ScaledEmbedding)
register_part("embedding", "normed", NormedEmbedding)
register_part("head", "lm_head", LMHead)
