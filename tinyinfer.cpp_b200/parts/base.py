"""Interfaces of the parts a decoder is put together from, and their registry.

Categories: ``norm``, ``position``, ``mixer``, ``ffn``, ``block``, ``embedding``,
``head``, ``junction``.  A part is built from a ``PartSpec`` (kind + parameters); it declares
the tensors it needs under names local to itself (``weight_specs``), receives
them once (``load_weights``), and then runs on device tensors through the
kernel set ``ops`` that the step hands it.  A part never sees the model's
configuration, its layer index or its checkpoint names.

Interfaces
----------
norm      ``forward(ops, x, out_dtype) -> h``; ``forward_rows(ops, x, rows, out_dtype)``.
position  ``rotation(device) -> Rotation``: the pairing rule, rotated width and table that the
          mixer hands on to the kernel that norms, rotates and stores its heads.
mixer     ``cache_spec()``: what it keeps per request (``PagedKVSpec``, ``FixedStateSpec`` or
          None); ``forward(ops, h, residual, step, cache)``: adds its output to ``residual``.
ffn       ``forward(ops, h, residual, step)``: adds its output to ``residual``.
block     arrangement of the four parts of a layer: ``forward(ops, x, step, cache)``.
embedding ``forward(ops, token_ids, out)``;  head ``forward(ops, h) -> logits``.
junction  ``forward(ops, x, x0, index, step)``: renews the residual stream ``x`` in place from itself
          and the embedding output ``x0`` where the schedule enters pass ``index`` of a run of layers.

``h`` is the normed activation in the engine's activation dtype (bfloat16 or
float32); ``residual``/``x`` is the float32 residual stream ``[T, hidden]``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping, Optional

import torch

from ..config.plan import PartSpec

MATRIX = "matrix"        # random mode: N(0, 0.02), stored in bfloat16
NORM_WEIGHT = "norm"     # random mode: 1 + N(0, 0.02), stored in float32
NORM_ZERO = "norm0"      # random mode: N(0, 0.02), stored in float32 (a factor stored minus one, a vector)


@dataclass(frozen=True)
class WeightSpec:
    shape: tuple[int, ...]           # an entry may be None: the stored tensor decides that size
    init: str = MATRIX
    optional: bool = False           # a folder may lack the tensor: the part then gets None for it


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every past token (or of the last ``window`` tokens, and of the
    request's first ``keep_first`` tokens whatever the window; or of the tokens of the current
    ``chunk`` of positions) in pages."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: all keys are kept
    v_head_dim: Optional[int] = None # None: values have the keys' head size; 0: a page holds one row
                                     # per token and kv head only (a mixer that makes keys and
                                     # values from the same cached row)
    keep_first: int = 0              # a request's first tokens stay readable behind the window
    chunk: Optional[int] = None      # positions are cut into chunks of this size, counted from 0,
                                     # and a token reads only keys of its own chunk


@dataclass(frozen=True)
class FixedStateSpec:
    """Per-request state of fixed size, zero when a request starts."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CompositeSpec:
    """Several things kept per request by one layer, each under a name: for instance the pages of
    an attention beside the fixed-size state of a recurrent mixer that reads the same input, or a
    mixer's cache beside what the block around it keeps.  The layer's view of its cache slot is
    then a ``CompositeView`` with one view per name."""
    items: tuple[tuple[str, "PagedKVSpec | FixedStateSpec | CompositeSpec"], ...]

    def flat(self, prefix: str = "") -> list:
        """``(dotted name, leaf spec)`` of every leaf, in order."""
        out = []
        for name, spec in self.items:
            if isinstance(spec, CompositeSpec):
                out += spec.flat(prefix + name + ".")
            elif spec is not None:
                out.append((prefix + name, spec))
        return out


class Part:
    category = ""

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {}

    def load_weights(self, tensors: Mapping[str, torch.Tensor], ops: Any) -> None:
        """Take the tensors named in ``weight_specs`` (already on the device, dtype as stored)."""

    def step_lists(self) -> list:
        """Integer lists (``engine.batch.StepList``) that this part wants built on the host for
        every step and handed to it as ``step.lists[name]``."""
        return []

    def shared_weights(self) -> dict[str, torch.Tensor]:
        """Tensors another part may alias (for instance the embedding table for a tied head)."""
        return {}


_REGISTRY: dict[tuple[str, str], Callable[..., Part]] = {}
CATEGORIES = ("norm", "position", "mixer", "ffn", "block", "embedding", "head", "junction")


def register_part(category: str, kind: str, factory: Callable[..., Part]) -> None:
    """Make ``factory(**params)`` the builder of parts of ``kind`` in ``category``."""
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; known: {', '.join(CATEGORIES)}")
    _REGISTRY[(category, kind)] = factory


def build_part(category: str, spec: PartSpec, **extra: Any) -> Part:
    try:
        factory = _REGISTRY[(category, spec.kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise ValueError(
            f"no {category} of kind {spec.kind!r} is registered; known: {', '.join(known)}") from None
    return factory(**dict(spec.params), **extra)


def as_float32(t: torch.Tensor) -> torch.Tensor:
    """Norm weights and tables are used in float32; widening bfloat16 is exact."""
    return t if t.dtype == torch.float32 else t.to(torch.float32)
