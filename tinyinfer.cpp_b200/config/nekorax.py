"""Typed configuration of the Nekorax decoder and its plan.

``config.json`` of this design is nested: ``architecture`` (the string ``Nekorax``), ``vocab``,
``width``, ``embedding.scale``, ``norm.eps``, ``logit_softcap``, ``loop`` and ``layers``, a list with
one object per layer: ``type`` (the mixer's kind), ``mixer`` (its sizes and constants) and ``mlp``
(the feed-forward, or null).  Sizes and constants have no defaults; an option that is not named
(the loop, the cap on the logits, a window, stretched frequencies, a convolution, identity experts,
groups of experts) does not exist.

The layer (``parts/block.py``, ``sandwich``): ``x += norm1b(mixer(norm1(x)))`` then ``x +=
norm2b(ff(norm2(x)))``; every norm is ``tanh(alpha x) w + b`` (``parts/norm.py``, ``dynamic_tanh``).
Mixers:

``attention``         grouped-query attention with a short convolution over time on q, k and v,
                      a half-split turn of the first ``rot.dims`` elements of a head, values turned
                      by their own position over the whole value head and outputs turned back, one
                      more unit in the softmax's denominator, a sigmoid gate per element
                      (``parts/conv_attention.py``)
``latent_attention``  queries through a normed latent of ``q_rank``; keys and values from a normed
                      latent of ``kv_rank`` and one turned key part of ``rot_dim`` that all heads
                      share (neighbouring pairs, frequencies stretched by ``rot.scaling``); a
                      sliding window ``mask.size`` (``parts/latent_attention.py``)

The feed-forward is a mixture of clamped gated experts (``g = min(g, limit)``, ``u = clamp(u,
-limit, limit)``, ``g sigmoid(1.702 g) (u + 1)``) chosen by a softmax router with a correction for
the choice, groups of experts and identity experts (``parts/moe.py``).  ``loop``: the layers
``start .. stop - 1`` are walked ``times`` times with the same tensors, every pass on a cache of its
own; before each pass the residual stream passes the junction ``x <- Win [x ; x0] + step[pass]``
(``parts/junction.py``).  The head has a table of its own behind ``final.norm``; the logits are
capped by ``logit_softcap tanh(. / logit_softcap)``.

Tensor names: ``embed``, ``head``, ``final.norm{,.alpha,.b}``, ``loop.in``, ``loop.step``,
``l<i>.norm{1,1b,2,2b}{,.alpha,.b}``, ``l<i>.mix.*`` (attention: ``q k v q.conv k.conv v.conv g o``;
latent attention: ``dq dq.norm uq dkv dkv.norm uk uv o``), ``l<i>.mlp.{router, correction,
e<n>.gate, e<n>.up, e<n>.down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .kagorax import MAX_POSITION, _get, _int, _positive
from .plan import LayerPlan, ModelPlan, PartSpec, ScheduleEntry
from .registry import Architecture, ConfigError, register_architecture

MIXER_TYPES = ("attention", "latent_attention")
GLU_ALPHA = 1.702            # the design's constant inside the activation's sigmoid


def _has(cfg, path: str) -> bool:
    node: Any = cfg
    for key in path.split("."):
        if not isinstance(node, Mapping) or node.get(key) is None:
            return False
        node = node[key]
    return True


def _even(entry, path: str, most: int, where: str, least: int = 0) -> int:
    v = _int(entry, path, least)
    if v % 2 or v > most:
        raise ConfigError(f"'{where}.{path}' must be even and at most {most}, got {v}")
    return v


def _mixer(entry, where: str, kind: str) -> dict:
    heads = _int(entry, "mixer.heads")
    out = {"heads": heads, "dim": _int(entry, "mixer.dim"), "vdim": _int(entry, "mixer.vdim"),
           "scale": _positive(entry, "mixer.scale"), "rot_base": _positive(entry, "mixer.rot.base"),
           "window": _int(entry, "mixer.mask.size") if _has(entry, "mixer.mask.size") else None}
    if kind == "attention":
        kv_heads = _int(entry, "mixer.kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"'{where}.mixer': {heads} heads cannot share {kv_heads} kv heads evenly")
        if out["vdim"] % 2:
            raise ConfigError(f"'{where}.mixer.vdim' must be even (values are turned in pairs), got {out['vdim']}")
        out.update(kv_heads=kv_heads, rot_dims=_even(entry, "mixer.rot.dims", out["dim"], where),
                   conv=_int(entry, "mixer.conv", 0) if _has(entry, "mixer.conv") else 0)
        return out
    rot_dim = _even(entry, "mixer.rot_dim", 1 << 20, where, 2)
    if _has(entry, "mixer.rot.dims") and _int(entry, "mixer.rot.dims") != rot_dim:
        raise ConfigError(f"'{where}.mixer.rot.dims' must equal 'rot_dim' ({rot_dim})")
    out.update(rot_dim=rot_dim, kv_rank=_int(entry, "mixer.kv_rank"), q_rank=_int(entry, "mixer.q_rank"), scaling=None)
    if _has(entry, "mixer.rot.scaling"):
        out["scaling"] = {k: _positive(entry, "mixer.rot.scaling." + k) for k in ("factor", "original", "fast", "slow")}
        if not out["rot_base"] > 1:
            raise ConfigError(f"'{where}.mixer.rot.base' must exceed 1 where frequencies are stretched")
    return out


def _mlp(entry, where: str) -> Optional[dict]:
    mlp = entry.get("mlp")
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, Mapping) else mlp
    if kind != "moe":
        raise ConfigError(f"'{where}.mlp.kind' is {kind!r}; known: 'moe'")
    experts, top = _int(mlp, "router.experts"), _int(mlp, "router.top")
    identity = _int(mlp, "router.identity", 0) if _has(mlp, "router.identity") else 0
    groups = None
    if _has(mlp, "router.groups"):
        groups = (_int(mlp, "router.groups.count"), _int(mlp, "router.groups.keep"))
    count, keep = groups or (1, 1)
    if keep > count or (experts + identity) % count:
        raise ConfigError(f"'{where}.mlp.router': {experts + identity} outputs in {count} groups of which {keep} are kept")
    if top > (experts + identity) // count * keep:
        raise ConfigError(f"'{where}.mlp.router': top {top} of {(experts + identity) // count * keep} experts that can be chosen")
    return {"experts": experts, "top": top, "identity": identity, "groups": groups, "ff": _int(mlp, "expert.ff"),
            "limit": _positive(mlp, "expert.limit")}


@dataclass(frozen=True)
class NekoraxLayer:
    type: str
    mixer: Mapping[str, Any]            # the validated sizes and constants of the mixer
    mlp: Optional[Mapping[str, Any]]    # None: no feed-forward


@dataclass(frozen=True)
class NekoraxConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_softcap: Optional[float]
    loop: Optional[tuple[int, int, int]]          # (start, stop, times)
    layers: tuple[NekoraxLayer, ...]
    source: Mapping[str, Any]

    ARCHITECTURE = "Nekorax"

    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "NekoraxConfig":
        vocab, width = _int(cfg, "vocab"), _int(cfg, "width")
        raw = _get(cfg, "layers")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping):
                raise ConfigError(f"'{where}' must be an object")
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"'{where}.type' is {kind!r}; known: {', '.join(MIXER_TYPES)}")
            layers.append(NekoraxLayer(kind, _mixer(entry, where, kind), _mlp(entry, where)))
        loop = None
        if _has(cfg, "loop"):
            loop = (_int(cfg, "loop.start", 0), _int(cfg, "loop.stop", 0), _int(cfg, "loop.times"))
            if not loop[0] < loop[1] <= len(layers):
                raise ConfigError(f"'loop': layers {loop[0]} .. {loop[1] - 1} of {len(layers)}")
        return NekoraxConfig(
            vocab=vocab, width=width, embedding_scale=_positive(cfg, "embedding.scale"),
            norm_eps=_positive(cfg, "norm.eps"),
            logit_softcap=_positive(cfg, "logit_softcap") if _has(cfg, "logit_softcap") else None,
            loop=loop, layers=tuple(layers), source=dict(cfg))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.source)


def _mixer_spec(cfg: NekoraxConfig, layer: NekoraxLayer) -> PartSpec:
    m = layer.mixer
    if layer.type == "attention":
        return PartSpec("conv_attention", {
            "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_head_dim": m["vdim"], "scale": m["scale"], "conv_taps": m["conv"], "window": m["window"],
            "sink_one": True, "gate": True,
            "position": PartSpec("rope_neox", {"head_dim": m["dim"], "theta": m["rot_base"], "rotary_dim": m["rot_dims"]})
            if m["rot_dims"] else PartSpec("none", {"head_dim": m["dim"]}),
            # the values turn over their whole head, in the pairing of the heads, never stretched
            "value_rotation": PartSpec("rope_neox", {"head_dim": m["vdim"], "theta": m["rot_base"]})})
    rot = {"head_dim": m["rot_dim"], "theta": m["rot_base"]}
    position = (PartSpec("rope_interleaved", rot) if m["scaling"] is None
                else PartSpec("rope_stretched", {**rot, **m["scaling"], "layout": "interleaved"}))
    return PartSpec("latent_attention", {
        "hidden_size": cfg.width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
        "v_head_dim": m["vdim"], "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"],
        "norm_eps": cfg.norm_eps, "sink": False, "window": m["window"], "position": position})


def _ffn_spec(cfg: NekoraxConfig, mlp: Mapping[str, Any]) -> PartSpec:
    return PartSpec("routed_experts", {
        "hidden_size": cfg.width, "experts": mlp["experts"], "top": mlp["top"], "expert_size": mlp["ff"],
        "router": "softmax", "activation": ("clamped", mlp["limit"], GLU_ALPHA), "identity": mlp["identity"],
        "correction": True, "groups": mlp["groups"]})


def schedule_of(num_layers: int, loop: Optional[tuple[int, int, int]]) -> list[ScheduleEntry]:
    """Every layer run in order, each on a cache slot of its own; the first layer of a pass enters it."""
    if loop is None:
        return [ScheduleEntry(layer=i, cache_slot=i) for i in range(num_layers)]
    start, stop, times = loop
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    runs += [(i, None) for i in range(stop, num_layers)]
    return [ScheduleEntry(layer=i, cache_slot=slot, enter=enter) for slot, (i, enter) in enumerate(runs)]


def build_plan(cfg: NekoraxConfig) -> ModelPlan:
    def norm(tensor: str) -> PartSpec:
        return PartSpec("dynamic_tanh", {"size": cfg.width, "tensor": tensor})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        has_ff = layer.mlp is not None
        layers.append(LayerPlan(
            block=PartSpec("sandwich"), mixer=_mixer_spec(cfg, layer),
            ffn=_ffn_spec(cfg, layer.mlp) if has_ff else None,
            mixer_norm=norm("norm1"), ffn_norm=norm("norm2") if has_ff else None,
            mixer_post_norm=norm("norm1b"), ffn_post_norm=norm("norm2b") if has_ff else None,
            names={"mixer": p + "mix.", "ffn": p + "mlp.", "mixer_norm": p, "ffn_norm": p, "mixer_post_norm": p,
                   "ffn_post_norm": p}))
    return ModelPlan(
        architecture=cfg.ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        layers=layers, schedule=schedule_of(len(layers), cfg.loop),
        embedding=PartSpec("scaled", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                      "scale": cfg.embedding_scale, "tensor": "embed"}),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": False,
                                  "tensor": "head", "softcap": cfg.logit_softcap}),
        junction=None if cfg.loop is None else PartSpec("loop_input", {"hidden_size": cfg.width, "passes": cfg.loop[2]}),
        names={"embedding": "", "final_norm": "", "head": "", "junction": "loop."})


register_architecture(Architecture(
    name=NekoraxConfig.ARCHITECTURE, from_dict=NekoraxConfig.from_dict, build_plan=build_plan,
    aliases=("nekorax",)))
