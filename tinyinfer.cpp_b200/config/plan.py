"""Architecture-independent description of a decoder: which parts, in which order.

An architecture's typed configuration (for instance ``Qwen3Config``) is turned
into a ``ModelPlan`` by its builder.  Everything below the plan (parts, cache
manager, step function) reads only the plan, never the architecture's own
configuration, so no part knows which model it is in.

A plan is plain data:

* ``PartSpec``      : a part's kind (a registry key) and its parameters.
* ``LayerPlan``     : the parts of one layer and the checkpoint-name prefixes
                      under which their tensors are stored.
* ``ScheduleEntry`` : one execution of a layer.  The schedule is a list; it may
                      name a layer twice, and an entry may read the cache slot
                      that another entry writes.  An entry may first run the
                      plan's junction (a part that renews the residual stream
                      from itself and the embedding output).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence


@dataclass(frozen=True)
class PartSpec:
    """Kind of a part (key in the part registry) with the part's parameters."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def with_params(self, **more: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(more)
        return PartSpec(self.kind, merged)


@dataclass(frozen=True)
class LayerPlan:
    """One layer: a block arrangement over a mixer, a feed-forward and norms.

    ``names`` maps each part role to the checkpoint prefix of its tensors, e.g.
    ``{"mixer": "model.layers.3.self_attn.", "mixer_norm":
    "model.layers.3.input_layernorm."}``.
    """
    block: PartSpec
    mixer: PartSpec
    ffn: Optional[PartSpec]              # None: the layer has no feed-forward
    mixer_norm: PartSpec
    ffn_norm: Optional[PartSpec]         # None: the block has one norm (both sublayers read it)
    names: Mapping[str, str]
    mixer_post_norm: Optional[PartSpec] = None   # blocks that also norm a sublayer's output (``sandwich``)
    ffn_post_norm: Optional[PartSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """Run layer ``layer`` using cache slot ``cache_slot``.

    ``writes_cache`` is False for an entry that only reads what an earlier
    entry of the same step wrote into that slot.  ``enter`` (a number) runs the
    plan's junction with that number on the residual stream right before the layer:
    the first layer of a pass over a run of layers that is walked several times.
    """
    layer: int
    cache_slot: int
    writes_cache: bool = True
    enter: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    layers: Sequence[LayerPlan]
    schedule: Sequence[ScheduleEntry]
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    names: Mapping[str, str]
    junction: Optional[PartSpec] = None      # what schedule entries with ``enter`` run; tensors under names["junction"]

    def __post_init__(self) -> None:
        n = len(self.layers)
        if self.junction is None and any(e.enter is not None for e in self.schedule):
            raise ValueError("a schedule entry enters a pass, but the plan has no junction")
        writers: dict[int, int] = {}
        for pos, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < n:
                raise ValueError(f"schedule entry {pos} names layer {entry.layer}, model has {n}")
            if entry.writes_cache:
                if entry.cache_slot in writers:
                    raise ValueError(
                        f"cache slot {entry.cache_slot} is written by schedule entries "
                        f"{writers[entry.cache_slot]} and {pos}")
                writers[entry.cache_slot] = pos
        for pos, entry in enumerate(self.schedule):
            if not entry.writes_cache:
                w = writers.get(entry.cache_slot)
                if w is None or w > pos:
                    raise ValueError(
                        f"schedule entry {pos} reads cache slot {entry.cache_slot} "
                        f"before any entry has written it")

    @property
    def num_cache_slots(self) -> int:
        return 1 + max((e.cache_slot for e in self.schedule), default=-1)


def default_schedule(num_layers: int) -> list[ScheduleEntry]:
    """Every layer once, in order, each with a cache slot of its own."""
    return [ScheduleEntry(layer=i, cache_slot=i) for i in range(num_layers)]
