"""Small Feruzen configurations with random weights, written as model folders by the tests.

The weights are drawn here with torch's generator (not with the package's), large enough that
every mechanism moves the logits: decays spread between fast and slow, gates on both sides of
their caps, feed-forward inputs on both sides of their clamps, routers with clear winners,
depth weights that give earlier layers a say.  Everything is stored in bfloat16, so the plain
implementation and the engine read the same values.
"""
from __future__ import annotations

import json
import os

import torch

from tinyinfer_b200.weights.safetensors_io import write_safetensors


def delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def parallel(left, right, left_scale, right_scale):
    heads, kv_heads, dim, vdim, rot_dims, base, scale = left
    r_heads, r_dim, r_vdim, cap = right
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                 "rot": {"dims": rot_dims, "base": base}, "scale": scale},
        "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "gate_cap": cap},
        "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(entry, mlp=None):
    return dict(entry, mlp=mlp)


# every size differs between the parts; three norm groups, two taps in front of the mixers, a
# rotation over half a head, experts with and without a shared one, a layer without a feed-forward
SMALL_A = {"architecture": "Feruzen", "vocab": 131, "width": 48, "norm": {"eps": 1e-6, "groups": 3},
           "canon": {"taps": 2}, "layers": [
    layer(parallel((4, 2, 12, 8, 6, 1000.0, 0.29), (3, 8, 12, 5.0), 0.7, 1.3), dense(40, 1.5)),
    layer(delta(4, 2, 8, 12, 3), moe(5, 2, 24, 2.5, shared=(16, 1.0))),
    layer(delta(2, 2, 12, 8, 2)),
    layer(parallel((2, 1, 16, 20, 16, 50.0, 0.2), (1, 12, 20, 3.0), -0.5, 0.9), moe(3, 1, 16, 0.8))]}
# values that make branches coincide or vanish: one norm group, one tap everywhere (a convolution
# that is a plain factor and keeps nothing), one head, as many kv heads as heads, no rotation,
# every expert chosen, one expert, a side with the scale 0
SMALL_B = {"architecture": "Feruzen", "vocab": 97, "width": 36, "norm": {"eps": 1e-5, "groups": 1},
           "canon": {"taps": 1}, "layers": [
    layer(delta(1, 1, 16, 16, 1), moe(4, 4, 8, 1.0)),
    layer(parallel((1, 1, 16, 16, 0, 7.0, 0.25), (1, 16, 16, 1.0), 1.0, 0.0), moe(1, 1, 24, 3.0, shared=(8, 2.0))),
    layer(parallel((3, 3, 8, 8, 2, 30.0, 0.35), (2, 4, 8, 20.0), 1.0, 1.0)),
    layer(delta(2, 1, 8, 4, 5), dense(32, 4.0))]}
# sizes that tensor-core kernels take (head sizes 64 and 128, widths that are multiples of 64),
# value heads wider than a block of state columns, four taps
SMALL_C = {"architecture": "Feruzen", "vocab": 1009, "width": 128, "norm": {"eps": 2e-6, "groups": 4},
           "canon": {"taps": 4}, "layers": [
    layer(delta(4, 2, 64, 64, 4), dense(192, 2.0)),
    layer(parallel((4, 2, 64, 64, 32, 20000.0, 0.125), (2, 64, 128, 8.0), 0.9, 1.1), moe(8, 2, 64, 2.0, shared=(128, 1.5))),
    layer(delta(2, 1, 128, 192, 3), moe(16, 3, 32, 1.5)),
    layer(parallel((2, 1, 128, 128, 128, 300000.0, 0.09), (1, 32, 160, 12.0), 1.2, 0.6), dense(256, 2.5))]}

SMALL = {"A": SMALL_A, "B": SMALL_B, "C": SMALL_C}


def mixer_weights(kind: str, m: dict, width: int, g: torch.Generator) -> dict:
    """Tensors of one mixer under their local names."""
    def mat(rows, cols, gain=1.0):
        return (torch.randn((rows, cols), generator=g) * gain / cols ** 0.5).to(torch.bfloat16)

    def vec(n, std, mean=0.0):
        return (mean + torch.randn((n,), generator=g) * std).to(torch.bfloat16)

    if kind == "delta":
        nk, nv, taps = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m["conv"]
        conv = lambda n: (torch.randn((n, taps), generator=g) * 0.6 + (torch.arange(taps) == taps - 1) * 0.8).to(torch.bfloat16)
        return {"q": mat(nk, width, 2.0), "q.conv": conv(nk), "k": mat(nk, width, 2.0), "k.conv": conv(nk),
                "v": mat(nv, width, 2.0), "v.conv": conv(nv), "b": mat(m["heads"], width, 2.0),
                "a": mat(m["heads"], width, 2.0), "A_log": vec(m["heads"], 1.0, -1.0), "dt_bias": vec(m["heads"], 1.0),
                "norm": vec(m["vdim"], 0.2, 1.0), "g": mat(nv, width, 2.0), "o": mat(width, nv)}
    w = {}
    a, b = m["left"], m["right"]
    nq, nk, nv = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], a["kv_heads"] * a["vdim"]
    w.update({"left.q": mat(nq, width, 2.0), "left.k": mat(nk, width, 2.0), "left.v": mat(nv, width),
              "left.q.norm": vec(a["dim"], 0.3, 1.5), "left.k.norm": vec(a["dim"], 0.3, 1.5),
              "left.o": mat(width, a["heads"] * a["vdim"])})
    rk, rv = b["heads"] * b["dim"], b["heads"] * b["vdim"]
    w.update({"right.q": mat(rk, width, 2.0), "right.k": mat(rk, width, 2.0), "right.v": mat(rv, width),
              "right.g": mat(rv, width, 2.0), "right.i": mat(b["heads"], width, 3.0), "right.i.b": vec(b["heads"], 1.0),
              "right.f": mat(b["heads"], width, 3.0), "right.f.b": vec(b["heads"], 1.0, 2.0),
              "right.norm": vec(rv, 0.2, 1.0), "right.o": mat(width, rv)})
    return w


def glu_weights(width: int, ff: int, g: torch.Generator) -> dict:
    mat = lambda rows, cols, gain: (torch.randn((rows, cols), generator=g) * gain / cols ** 0.5).to(torch.bfloat16)
    return {"gate": mat(ff, width, 2.0), "up": mat(ff, width, 2.0), "down": mat(width, ff, 1.0)}


def mlp_weights(mlp: dict, width: int, g: torch.Generator) -> dict:
    if mlp["kind"] == "dense":
        return glu_weights(width, mlp["ff"], g)
    w = {"router": (torch.randn((mlp["router"]["experts"], width), generator=g) * 3.0 / width ** 0.5).to(torch.bfloat16)}
    for e in range(mlp["router"]["experts"]):
        for name, t in glu_weights(width, mlp["expert"]["ff"], g).items():
            w[f"e{e}.{name}"] = t
    if mlp.get("shared") is not None:
        for name, t in glu_weights(width, mlp["shared"]["ff"], g).items():
            w["shared." + name] = t
    return w


def random_weights(cfg: dict, seed: int) -> dict:
    g = torch.Generator().manual_seed(seed)
    width = cfg["width"]
    norm = lambda: (0.6 + 0.2 * torch.randn((width,), generator=g)).to(torch.bfloat16)
    w = {"embed": (torch.randn((cfg["vocab"], width), generator=g) * 0.5).to(torch.bfloat16), "final.norm": norm()}
    for i, entry in enumerate(cfg["layers"]):
        p = f"l{i}."
        w[p + "norm1"] = norm()
        w[p + "canon1"] = (torch.randn((width, cfg["canon"]["taps"]), generator=g) * 0.4).to(torch.bfloat16)
        depth = 0.3 * torch.randn((i + 2,), generator=g)
        depth[-1] += 1.0
        w[p + "dwa"] = depth.to(torch.bfloat16)
        for name, t in mixer_weights(entry["type"], entry["mixer"], width, g).items():
            w[p + "mix." + name] = t
        if entry["mlp"] is not None:
            w[p + "norm2"] = norm()
            for name, t in mlp_weights(entry["mlp"], width, g).items():
                w[p + "mlp." + name] = t
    return w


def write_model(folder: str, cfg: dict, seed: int) -> str:
    os.makedirs(folder, exist_ok=True)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_weights(cfg, seed))
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    return folder


def make_model(tmp_path, name: str, seed: int = 5) -> str:
    d = os.path.join(str(tmp_path), f"feruzen_{name}_{seed}")
    if not os.path.isdir(d):
        write_model(d, SMALL[name], seed)
    return d
