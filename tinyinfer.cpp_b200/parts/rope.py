"""Position encodings of the attention heads, and what they tell the mixer's kernels.

A position part does not rotate anything itself: it answers ``rotation(device)`` with a
``Rotation``, the contract between it and the kernel that norms, rotates and stores the heads
(``ops.qkv_rope_store``).  ``kind`` names the pairing rule; the kernel set has kernels for some
kinds and refuses the others, unless a part has registered a handler for its own kind
(``ops.register_rotation``).  The mixer passes the ``Rotation`` on without looking inside.

Kinds built in:

``neox``   half-split pairs over the first ``rotary_dim`` elements of a head: for pair index
           ``k`` in ``[0, rotary_dim/2)``, ``inv_freq[k] = theta ** (-2k / rotary_dim)``, angle
           ``a = pos * inv_freq[k]``, and ``(x[k], x[k + rotary_dim/2])`` becomes
           ``(x0 cos a - x1 sin a, x0 sin a + x1 cos a)``; elements from ``rotary_dim`` on are
           left as they are.  With ``rotary_dim = head_dim`` this is the reference's rotation
           (src/cuda/attention.cu:64-74, src/cuda/rope.cu:19-28).
``interleaved``  neighbouring pairs over the first ``rotary_dim`` elements of a head: elements
           ``2k`` and ``2k + 1`` form pair ``k`` with the same frequencies and the same turn as
           above.  The kernels that take it say so (``ops.qk_rownorm_rope_store``,
           ``ops.latent_prepare``); the per-head norm kernel of ``neox`` does not.
``none``   no rotation (``rotary_dim = 0``).

``rope_stretched`` (YaRN) answers with either pairing: frequencies that turn fast stay, slow ones are
divided by ``factor``, a ramp lies between; and ``Rotation.scale`` multiplies both sine and cosine.

``inv_freq`` is computed once on the host in double precision and rounded to float32; the
angle, its sine and cosine are float32 on the device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch

from .base import Part, register_part


@dataclass(frozen=True)
class Rotation:
    """What the kernels need to encode a head's position.

    kind        the pairing rule (a key of the kernel set's table of rotations)
    rotary_dim  how many leading elements of a head take part (0: none)
    inv_freq    ``[rotary_dim / 2]`` float32 on the device, or None
    extra       anything else a kind's own handler wants
    scale       a factor on both the sine and the cosine (1: a pure turn); the kernels that take it
                say so (``ops.latent_prepare``, ``ops.qkv_turn_store``)
    """
    kind: str
    rotary_dim: int
    inv_freq: Optional[torch.Tensor] = None
    extra: Any = None
    scale: float = 1.0


_TABLES: dict[tuple, torch.Tensor] = {}      # layers with the same constants share one device tensor


class RopeNeox(Part):
    category = "position"

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None):
        rotary_dim = head_dim if rotary_dim is None else int(rotary_dim)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary width {rotary_dim} must be even and lie in (0, head_dim {head_dim}]")
        self.head_dim = int(head_dim)
        self.rotary_dim = rotary_dim
        self.theta = float(theta)

    def inv_freq(self) -> torch.Tensor:
        half = self.rotary_dim // 2
        k = torch.arange(half, dtype=torch.float64)
        return torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                         -2.0 * k / self.rotary_dim).to(torch.float32)

    def rotation(self, device) -> Rotation:
        key = (self.rotary_dim, self.theta, str(device))
        if key not in _TABLES:
            _TABLES[key] = self.inv_freq().to(device)
        return Rotation("neox", self.rotary_dim, _TABLES[key])


class RopeInterleaved(RopeNeox):
    """The same frequencies and turn as ``RopeNeox`` on neighbouring pairs ``(2k, 2k + 1)``."""

    def rotation(self, device) -> Rotation:
        return Rotation("interleaved", self.rotary_dim, super().rotation(device).inv_freq)


class RopeStretched(RopeNeox):
    """Frequencies stretched for contexts longer than the ``original`` one (YaRN).  With
    ``d(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta)``, ``lo = max(floor(d(fast)), 0)``,
    ``hi = min(ceil(d(slow)), rotary_dim - 1)`` and ``ramp_k = clamp((k - lo) / max(hi - lo, 0.001),
    0, 1)``, pair ``k`` turns with ``f_k / factor * ramp_k + f_k * (1 - ramp_k)``, and sine and
    cosine are multiplied by ``0.1 ln(factor) + 1``.  ``layout``: ``interleaved`` or ``neox``."""

    def __init__(self, head_dim: int, theta: float, factor: float, original: float, fast: float, slow: float,
                 rotary_dim: Optional[int] = None, layout: str = "interleaved"):
        super().__init__(head_dim, theta, rotary_dim)
        if layout not in ("interleaved", "neox"):
            raise ValueError(f"pairing {layout!r}; known: interleaved, neox")
        self.factor, self.original = float(factor), float(original)
        self.fast, self.slow, self.layout = float(fast), float(slow), layout
        if not (self.factor > 0 and self.original > 0 and self.fast > 0 and self.slow > 0 and self.theta > 1):
            raise ValueError("stretched frequencies need positive constants and a base above 1")

    def inv_freq(self) -> torch.Tensor:
        import math
        n = self.rotary_dim

        def at(turns: float) -> float:
            return n * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo, hi = max(math.floor(at(self.fast)), 0), min(math.ceil(at(self.slow)), n - 1)
        k = torch.arange(n // 2, dtype=torch.float64)
        plain = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * k / n)
        ramp = torch.clamp((k - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return (plain / self.factor * ramp + plain * (1.0 - ramp)).to(torch.float32)

    def rotation(self, device) -> Rotation:
        import math
        key = ("stretched", self.rotary_dim, self.theta, self.factor, self.original, self.fast, self.slow, str(device))
        if key not in _TABLES:
            _TABLES[key] = self.inv_freq().to(device)
        return Rotation(self.layout, self.rotary_dim, _TABLES[key], scale=0.1 * math.log(self.factor) + 1.0)


class NoPosition(Part):
    """Heads are normed and stored without a rotation."""
    category = "position"

    def __init__(self, head_dim: int = 0):
        self.head_dim = int(head_dim)

    def rotation(self, device) -> Rotation:
        return Rotation("none", 0, None)


register_part("position", "rope_neox", RopeNeox)
register_part("position", "rope_interleaved", RopeInterleaved)
register_part("position", "rope_stretched", RopeStretched)
register_part("position", "none", NoPosition)
