"""Typed configuration of the Feruzen decoder and its plan.

``config.json`` of this design is nested: ``architecture`` (the string ``Feruzen``), ``vocab``,
``width``, ``norm.eps``, ``norm.groups``, ``canon.taps`` and ``layers``, a list with one object per
layer: ``type`` (the mixer's kind), ``mixer`` (its sizes and constants) and ``mlp`` (the
feed-forward, or null).  Nothing has a default: a missing size or constant is an error.

The layer (``parts/block.py``, ``output_norm``): the norm sits on the sublayer's output,
``x += norm1(mixer(x + conv(x)))`` then ``x += norm2(ff(x))``; the norms are RMS norms in
``norm.groups`` groups, ``conv`` is a causal convolution of ``canon.taps`` taps over time on every
channel, and behind every layer stands a weighted sum over the results of all layers so far
(``dwa``).  Mixers:

``delta``     the gated delta rule with short convolutions on q, k, v (``parts/state_mixers.py``)
``parallel``  two mixers side by side whose outputs are added with ``left_scale`` and
              ``right_scale`` (``parts/parallel_mixers.py``): on the left causal grouped-query
              attention with a norm per query and key head and a neighbouring-pair rotation of the
              first ``rot.dims`` elements (``parts/chunked_attention.py`` with its options off), on
              the right a matrix memory with exponential gates (``parts/state_mixers.py``)

The feed-forward is gated with clamps, ``g = min(g, limit)``, ``u = clamp(u, -limit, limit)``,
``g sigmoid(1.702 g) (u + 1)`` (``parts/mlp.py``), either dense or as routed experts chosen by a
softmax router whose scores are the weights as they are, with an ungated shared expert
(``parts/moe.py``).  The head is the embedding table behind ``final.norm``.

Tensor names: ``embed``, ``final.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.canon1``,
``l<i>.dwa``, ``l<i>.mix.*`` (delta: ``q q.conv k k.conv v v.conv b a A_log dt_bias norm g o``;
parallel: ``left.{q,k,v,q.norm,k.norm,o}`` and ``right.{q,k,v,g,i,i.b,f,f.b,norm,o}``),
``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.{router, e<n>.gate, e<n>.up, e<n>.down, shared.gate,
shared.up, shared.down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .kagorax import MAX_POSITION, _get, _int, _positive
from .plan import LayerPlan, ModelPlan, PartSpec, default_schedule
from .registry import Architecture, ConfigError, register_architecture

MIXER_TYPES = ("delta", "parallel")
GLU_ALPHA = 1.702            # the design's constant inside the activation's sigmoid


@dataclass(frozen=True)
class FeruzenLayer:
    type: str
    mixer: Mapping[str, Any]            # the validated sizes and constants of the mixer
    mlp: Optional[Mapping[str, Any]]    # None: no feed-forward


def _heads(entry, where: str, path: str) -> tuple[int, int]:
    heads, kv_heads = _int(entry, path + ".heads"), _int(entry, path + ".kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"'{where}.{path}': {heads} heads cannot share {kv_heads} kv heads evenly")
    return heads, kv_heads


def _mixer(entry, where: str, kind: str) -> dict:
    if kind == "delta":
        heads, kv_heads = _heads(entry, where, "mixer")
        return {"heads": heads, "kv_heads": kv_heads, "dim": _int(entry, "mixer.dim"),
                "vdim": _int(entry, "mixer.vdim"), "conv": _int(entry, "mixer.conv")}
    heads, kv_heads = _heads(entry, where, "mixer.left")
    dim = _int(entry, "mixer.left.dim")
    dims = _int(entry, "mixer.left.rot.dims", 0)
    if dims % 2 or dims > dim:
        raise ConfigError(f"'{where}.mixer.left.rot.dims' must be even and at most {dim}, got {dims}")
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": _int(entry, "mixer.left.vdim"),
            "scale": _positive(entry, "mixer.left.scale"), "rot_dims": dims,
            "rot_base": _positive(entry, "mixer.left.rot.base")}
    right = {"heads": _int(entry, "mixer.right.heads"), "dim": _int(entry, "mixer.right.dim"),
             "vdim": _int(entry, "mixer.right.vdim"), "gate_cap": _positive(entry, "mixer.right.gate_cap")}
    return {"left": left, "right": right, "left_scale": _number(entry, "mixer.left_scale"),
            "right_scale": _number(entry, "mixer.right_scale")}


def _number(cfg, path: str) -> float:
    v = _get(cfg, path)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or v != v or v in (float("inf"), float("-inf")):
        raise ConfigError(f"'{path}' must be a number, got {v!r}")
    return float(v)


def _mlp(entry, where: str) -> Optional[dict]:
    mlp = entry.get("mlp")
    if mlp is None:
        return None
    kind = mlp.get("kind") if isinstance(mlp, Mapping) else mlp
    if kind == "dense":
        return {"kind": "dense", "ff": _int(mlp, "ff"), "limit": _positive(mlp, "limit")}
    if kind == "moe":
        experts, top = _int(mlp, "router.experts"), _int(mlp, "router.top")
        if top > experts:
            raise ConfigError(f"'{where}.mlp.router': top {top} of {experts} experts")
        out = {"kind": "moe", "experts": experts, "top": top, "ff": _int(mlp, "expert.ff"),
               "limit": _positive(mlp, "expert.limit"), "shared": None}
        if mlp.get("shared") is not None:
            out["shared"] = {"ff": _int(mlp, "shared.ff"), "limit": _positive(mlp, "shared.limit")}
        return out
    raise ConfigError(f"'{where}.mlp.kind' is {kind!r}; known: 'dense', 'moe'")


@dataclass(frozen=True)
class FeruzenConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    conv_taps: int
    layers: tuple[FeruzenLayer, ...]
    source: Mapping[str, Any]

    ARCHITECTURE = "Feruzen"

    @staticmethod
    def from_dict(cfg: Mapping[str, Any]) -> "FeruzenConfig":
        vocab, width = _int(cfg, "vocab"), _int(cfg, "width")
        groups = _int(cfg, "norm.groups")
        if width % groups:
            raise ConfigError(f"'norm.groups': {width} channels do not fall into {groups} equal groups")
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
            layers.append(FeruzenLayer(kind, _mixer(entry, where, kind), _mlp(entry, where)))
        return FeruzenConfig(vocab=vocab, width=width, norm_eps=_positive(cfg, "norm.eps"), norm_groups=groups,
                             conv_taps=_int(cfg, "canon.taps"), layers=tuple(layers), source=dict(cfg))

    def to_dict(self) -> dict[str, Any]:
        return dict(self.source)


def _mixer_spec(cfg: FeruzenConfig, layer: FeruzenLayer) -> PartSpec:
    m = layer.mixer
    if layer.type == "delta":
        return PartSpec("gated_delta", {
            "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_head_dim": m["vdim"], "conv_taps": m["conv"], "norm_eps": cfg.norm_eps})
    a, b = m["left"], m["right"]
    left = PartSpec("chunked_attention", {
        "hidden_size": cfg.width, "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "head_dim": a["dim"],
        "v_head_dim": a["vdim"], "scale": a["scale"], "qk_norm_eps": cfg.norm_eps, "norm_per_head": True,
        "head_temperature": False, "head_gate": False,
        "position": PartSpec("rope_interleaved", {"head_dim": a["dim"], "theta": a["rot_base"],
                                                  "rotary_dim": a["rot_dims"]})
        if a["rot_dims"] else PartSpec("none", {"head_dim": a["dim"]})})
    right = PartSpec("matrix_memory", {
        "hidden_size": cfg.width, "num_heads": b["heads"], "head_dim": b["dim"], "v_head_dim": b["vdim"],
        "gate_cap": b["gate_cap"], "norm_eps": cfg.norm_eps})
    return PartSpec("parallel_mixers", {"hidden_size": cfg.width, "left": left, "right": right,
                                        "left_scale": m["left_scale"], "right_scale": m["right_scale"]})


def _ffn_spec(cfg: FeruzenConfig, mlp: Mapping[str, Any]) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("glu_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp["ff"],
                                    "activation": "clamped", "limit": mlp["limit"], "alpha": GLU_ALPHA})
    shared = mlp["shared"]
    return PartSpec("routed_experts", {
        "hidden_size": cfg.width, "experts": mlp["experts"], "top": mlp["top"], "expert_size": mlp["ff"],
        "router": "softmax", "activation": ("clamped", mlp["limit"], GLU_ALPHA),
        "shared_size": None if shared is None else shared["ff"], "shared_gated": False,
        "shared_activation": None if shared is None else ("clamped", shared["limit"], GLU_ALPHA)})


def build_plan(cfg: FeruzenConfig) -> ModelPlan:
    def norm(tensor: str) -> PartSpec:
        return PartSpec("group_rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "groups": cfg.norm_groups,
                                          "tensor": tensor})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        has_ff = layer.mlp is not None
        layers.append(LayerPlan(
            block=PartSpec("output_norm", {"hidden_size": cfg.width, "conv_taps": cfg.conv_taps, "depth_index": i,
                                           "depth_total": len(cfg.layers)}),
            mixer=_mixer_spec(cfg, layer), ffn=_ffn_spec(cfg, layer.mlp) if has_ff else None,
            mixer_norm=norm("norm1"), ffn_norm=norm("norm2") if has_ff else None,
            names={"block": p, "mixer": p + "mix.", "ffn": p + "mlp.", "mixer_norm": p, "ffn_norm": p}))
    return ModelPlan(
        architecture=cfg.ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        layers=layers, schedule=default_schedule(len(layers)),
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tensor": "embed"}),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": True}),
        names={"embedding": "", "final_norm": "", "head": "head."})


register_architecture(Architecture(
    name=FeruzenConfig.ARCHITECTURE, from_dict=FeruzenConfig.from_dict, build_plan=build_plan,
    aliases=("feruzen",)))
