"""Small Nekorax configurations with random weights, written as model folders by the tests.

The weights are drawn here with torch's generator (not with the package's), large enough that
every mechanism moves the logits: norms whose tanh bends, convolutions whose earlier taps count,
routers with clear winners and corrections that change the choice, junctions that mix the stream
with the embedding output.  Everything is stored in bfloat16, so the plain implementation and the
engine read the same values.
"""
from __future__ import annotations

import json
import os

import torch

from tinyinfer_b200.weights.safetensors_io import write_safetensors


def attention(heads, kv_heads, dim, vdim, rot_dims, base, scale, conv=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot_dims},
         "scale": scale}
    if conv is not None:
        m["conv"] = conv
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base, scale, window=None, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "rot": rot, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def moe(experts, top, ff, limit, identity=None, groups=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": router, "expert": {"ff": ff, "limit": limit}}


def layer(entry, mlp=None):
    return dict(entry, mlp=mlp)


# every size differs between the parts: fewer kv heads than heads, value heads of another size, a turn
# over part of a head, three taps, a window shorter than two pages, identity experts, three groups of
# which two are kept, a layer without a feed-forward, a loop over the two middle layers
SMALL_A = {"architecture": "Nekorax", "vocab": 131, "width": 48, "embedding": {"scale": 1.7}, "norm": {"eps": 1e-6},
           "logit_softcap": 9.0, "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
    layer(attention(4, 2, 12, 8, 6, 1000.0, 0.29, conv=3), moe(4, 2, 24, 1.5, identity=2, groups=(3, 2))),
    layer(latent(3, 8, 4, 10, 12, 20, 100.0, 0.3, window=20, scaling=(4.0, 16, 8.0, 1.0)), moe(6, 3, 16, 2.5, identity=3, groups=(3, 1))),
    layer(attention(2, 1, 16, 20, 16, 50.0, 0.2, conv=2)),
    layer(latent(2, 6, 8, 6, 10, 8, 3000.0, 0.35, window=7), moe(5, 1, 8, 0.8, identity=1))]}
# values that make branches coincide or vanish: one pass of a loop over all layers, one tap (a
# convolution that is a plain factor and keeps nothing) and none at all, one head, as many kv heads as
# heads, no turn of the heads, a window longer than any prompt and none, plain frequencies, no identity
# experts, no groups, every expert chosen, one expert, no cap on the logits
SMALL_B = {"architecture": "Nekorax", "vocab": 97, "width": 36, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
           "loop": {"start": 0, "stop": 4, "times": 1}, "layers": [
    layer(attention(1, 1, 16, 16, 0, 7.0, 0.25, conv=1), moe(4, 4, 8, 1.0)),
    layer(latent(1, 16, 2, 16, 8, 8, 30.0, 0.25, window=100000), moe(1, 1, 24, 3.0, identity=0)),
    layer(attention(3, 3, 8, 8, 2, 30.0, 0.35), moe(3, 2, 8, 1.0, groups=(1, 1))),
    layer(latent(2, 4, 4, 8, 6, 4, 10.0, 0.4))]}
# sizes that the tensor-core kernels take (head sizes 64 and 128, widths that are multiples of 64),
# four taps, three passes over the first three layers, experts whose sizes the grouped products take
SMALL_C = {"architecture": "Nekorax", "vocab": 1009, "width": 128, "embedding": {"scale": 0.8}, "norm": {"eps": 2e-6},
           "logit_softcap": 30.0, "loop": {"start": 0, "stop": 3, "times": 3}, "layers": [
    layer(latent(4, 64, 32, 64, 128, 96, 20000.0, 0.1, window=70, scaling=(16.0, 64, 32.0, 1.0)), moe(8, 2, 64, 2.0, identity=4, groups=(4, 2))),
    layer(attention(4, 2, 64, 64, 32, 20000.0, 0.125, conv=4), moe(12, 3, 32, 1.5, identity=4, groups=(2, 1))),
    layer(attention(2, 1, 128, 128, 128, 300000.0, 0.09, conv=2), moe(16, 4, 64, 2.5)),
    layer(latent(2, 128, 64, 128, 64, 64, 1000.0, 0.07), moe(6, 2, 32, 1.0, identity=2))]}
# no loop at all
SMALL_D = {"architecture": "Nekorax", "vocab": 61, "width": 24, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
           "logit_softcap": 4.0, "layers": [
    layer(latent(2, 4, 2, 6, 8, 6, 10.0, 0.4, window=3), moe(2, 1, 8, 1.0, identity=2, groups=(2, 1))),
    layer(attention(2, 2, 6, 4, 4, 20.0, 0.4, conv=5), moe(3, 2, 8, 1.0, identity=1, groups=(2, 2)))]}

SMALL = {"A": SMALL_A, "B": SMALL_B, "C": SMALL_C, "D": SMALL_D}


def _mat(g, rows, cols, gain=1.0):
    return (torch.randn((rows, cols), generator=g) * gain / cols ** 0.5).to(torch.bfloat16)


def _vec(g, n, std, mean=0.0):
    return (mean + torch.randn((n,), generator=g) * std).to(torch.bfloat16)


def norm_weights(name: str, width: int, g: torch.Generator) -> dict:
    return {name: _vec(g, width, 0.2, 0.9), name + ".b": _vec(g, width, 0.1),
            name + ".alpha": (0.4 + 0.6 * torch.rand((), generator=g)).to(torch.bfloat16)}


def mixer_weights(kind: str, m: dict, width: int, g: torch.Generator) -> dict:
    """Tensors of one mixer under their local names."""
    if kind == "attention":
        nq, nk, nv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
        no = m["heads"] * m["vdim"]
        w = {"q": _mat(g, nq, width, 2.0), "k": _mat(g, nk, width, 2.0), "v": _mat(g, nv, width, 1.5),
             "g": _mat(g, no, width, 2.0), "o": _mat(g, width, no)}
        taps = m.get("conv")
        if taps:
            for name, n in (("q", nq), ("k", nk), ("v", nv)):
                w[name + ".conv"] = (torch.randn((n, taps), generator=g) * 0.5
                                     + (torch.arange(taps) == taps - 1) * 0.8).to(torch.bfloat16)
        return w
    nh, d, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    return {"dq": _mat(g, m["q_rank"], width, 2.0), "dq.norm": _vec(g, m["q_rank"], 0.2, 1.0),
            "uq": _mat(g, nh * (d + dr), m["q_rank"], 2.0), "dkv": _mat(g, m["kv_rank"] + dr, width, 2.0),
            "dkv.norm": _vec(g, m["kv_rank"], 0.2, 1.0), "uk": _mat(g, nh * d, m["kv_rank"], 1.5),
            "uv": _mat(g, nh * dv, m["kv_rank"], 1.5), "o": _mat(g, width, nh * dv)}


def mlp_weights(mlp: dict, width: int, g: torch.Generator) -> dict:
    r = mlp["router"]
    total = r["experts"] + r.get("identity", 0)
    # logits a few units apart, and corrections of the size of a typical score: the choice is not the
    # plain order of the scores
    w = {"router": _mat(g, total, width, 3.0), "correction": _vec(g, total, 0.5 / total)}
    for e in range(r["experts"]):
        ff = mlp["expert"]["ff"]
        w.update({f"e{e}.gate": _mat(g, ff, width, 2.0), f"e{e}.up": _mat(g, ff, width, 2.0), f"e{e}.down": _mat(g, width, ff)})
    return w


def random_weights(cfg: dict, seed: int) -> dict:
    g = torch.Generator().manual_seed(seed)
    width = cfg["width"]
    w = {"embed": (torch.randn((cfg["vocab"], width), generator=g) * 0.5).to(torch.bfloat16),
         "head": _mat(g, cfg["vocab"], width, 3.0), **norm_weights("final.norm", width, g)}
    if cfg.get("loop"):
        eye = torch.eye(width)
        w["loop.in"] = (torch.cat([0.8 * eye, 0.5 * eye], dim=1)
                        + torch.randn((width, 2 * width), generator=g) * 0.3 / width ** 0.5).to(torch.bfloat16)
        w["loop.step"] = (torch.randn((cfg["loop"]["times"], width), generator=g) * 0.3).to(torch.bfloat16)
    for i, entry in enumerate(cfg["layers"]):
        p = f"l{i}."
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if entry["mlp"] is not None else ()):
            w.update(norm_weights(p + n, width, g))
        for name, t in mixer_weights(entry["type"], entry["mixer"], width, g).items():
            w[p + "mix." + name] = t
        if entry["mlp"] is not None:
            for name, t in mlp_weights(entry["mlp"], width, g).items():
                w[p + "mlp." + name] = t
    return w


def make_model(tmp_path, name: str, seed: int = 11) -> str:
    d = os.path.join(str(tmp_path), f"nekorax_{name}_{seed}")
    if not os.path.isdir(d):
        os.makedirs(d)
        with open(os.path.join(d, "config.json"), "w") as fh:
            json.dump(SMALL[name], fh)
        write_safetensors(os.path.join(d, "model.safetensors"), random_weights(SMALL[name], seed))
    return d


def drawn_configuration(seed: int) -> dict:
    """A configuration whose every size, constant, option and order of layers is drawn from ``seed``."""
    import random
    r = random.Random(seed)
    pick = r.choice
    width = pick([16, 24, 40, 64, 72])

    def drawn_moe():
        if r.random() < 0.15:
            return None
        experts, identity = pick([1, 2, 3, 5, 8]), pick([0, 0, 1, 2, 3])
        total = experts + identity
        counts = [c for c in (1, 2, 3, 4) if total % c == 0]
        count = pick(counts)
        keep = r.randint(1, count)
        top = r.randint(1, min(total // count * keep, 4))
        groups = (count, keep) if (count > 1 or r.random() < 0.3) else None
        return moe(experts, top, pick([8, 16, 24, 32]), pick([0.5, 1.0, 3.0]), identity=identity if identity or r.random() < 0.5 else None,
                   groups=groups)

    layers = []
    for _ in range(r.randint(1, 5)):
        if r.random() < 0.5:
            kv = pick([1, 2, 3])
            heads = kv * pick([1, 2, 3])
            dim, vdim = pick([4, 6, 10, 16, 32, 48]), pick([2, 6, 8, 16, 32, 40])
            rot = pick([0, 2, dim // 2 // 2 * 2, dim])
            entry = attention(heads, kv, dim, vdim, rot, pick([10.0, 500.0, 250000.0]), r.uniform(0.05, 0.4),
                              conv=pick([None, 1, 2, 3, 4, 6]))
        else:
            rot_dim = pick([2, 4, 8, 16])
            scaling = None if r.random() < 0.4 else (pick([2.0, 8.0, 40.0]), pick([8, 32, 256]), pick([32.0, 4.0]), pick([1.0, 2.0]))
            entry = latent(pick([1, 2, 3, 4, 5]), pick([4, 8, 16, 24]), rot_dim, pick([4, 8, 12, 16]), pick([6, 16, 32, 48]),
                           pick([4, 16, 40]), pick([50.0, 10000.0]), r.uniform(0.05, 0.4),
                           window=pick([None, 1, 2, 5, 16, 17, 33, 64, 200]), scaling=scaling)
        layers.append(layer(entry, drawn_moe()))
    cfg = {"architecture": "Nekorax", "vocab": pick([33, 100, 257]), "width": width, "embedding": {"scale": r.uniform(0.3, 2.0)},
           "norm": {"eps": pick([1e-6, 1e-5])}, "layers": layers}
    if r.random() < 0.8:
        cfg["logit_softcap"] = pick([5.0, 15.0, 50.0])
    if r.random() < 0.8:
        start = r.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": start, "stop": r.randint(start + 1, len(layers)), "times": pick([1, 2, 2, 3])}
    return cfg


def make_drawn_model(tmp_path, seed: int) -> str:
    d = os.path.join(str(tmp_path), f"nekorax_drawn_{seed}")
    if not os.path.isdir(d):
        os.makedirs(d)
        cfg = drawn_configuration(seed)
        with open(os.path.join(d, "config.json"), "w") as fh:
            json.dump(cfg, fh)
        write_safetensors(os.path.join(d, "model.safetensors"), random_weights(cfg, seed))
    return d
