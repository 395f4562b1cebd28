"""A plain, slow implementation of the Nekorax decoder in float64, one function per mechanism,
written from the design's equations.  It runs one whole sequence at a time on the CPU and shares
no code with the engine; the tests compare the engine with it.

Notation: ``x`` is ``[T, width]``, a linear weight is stored ``[out, in]`` and applied as ``x @ W.T``;
``cfg`` is the dictionary of ``config.json`` and ``w`` maps tensor names to float64 tensors.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

F = torch.float64
GLU_ALPHA = 1.702


def load_folder(folder: str):
    """Configuration and float64 tensors of a model folder, read with the standard library and torch alone."""
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    with open(os.path.join(folder, "model.safetensors"), "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n))
        data = fh.read()
    weights = {}
    for name, ent in header.items():
        if name != "__metadata__":
            lo, hi = ent["data_offsets"]
            weights[name] = torch.frombuffer(bytearray(data[lo:hi]), dtype=kinds[ent["dtype"]]).view(ent["shape"]).to(F)
    return cfg, weights


# ---- small pieces ---------------------------------------------------------------------------------
def dyt(x, w, name):
    """Dynamic tanh: no mean, no variance; ``tanh(alpha x) weight + bias``."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def time_conv(u, taps_w):
    """``y_t = sum_j w[:, j] u_(t - taps + 1 + j)`` with zeros before the start; ``taps_w`` is ``[channels, taps]``."""
    t, taps = u.shape[0], taps_w.shape[1]
    y = torch.zeros_like(u)
    for i in range(t):
        for j in range(taps):
            src = i - taps + 1 + j
            if src >= 0:
                y[i] += taps_w[:, j] * u[src]
    return y


def frequencies(base, dims):
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)


def yarn(freq, base, dims, scaling):
    """Frequencies stretched by ``factor`` where they turn slowly, left alone where they turn fast, a ramp
    between; and the factor that both sine and cosine are multiplied with."""
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    out = torch.empty_like(freq)
    for i in range(dims // 2):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = freq[i] / factor * ramp + freq[i] * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def turn(x, pos, freq, dims, layout, mag=1.0):
    """Turn the first ``dims`` elements of the last axis of ``x [T, ..., n]`` by ``pos[t] * freq``.
    ``layout`` "halves": element i with i + dims/2; "pairs": 2i with 2i + 1."""
    out = x.clone()
    half = dims // 2
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    ang = (pos.to(F).reshape(-1, 1) * freq.reshape(1, -1)).reshape(shape)
    c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
    if layout == "halves":
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    else:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    return out


# ---- mixers ---------------------------------------------------------------------------------------
def attention(w, p, h, m):
    """Grouped-query attention with short convolutions on q, k, v, partly turned heads (halves), values
    turned by their own position and the output turned back, one more unit in the softmax's
    denominator, and a sigmoid gate per element."""
    t = h.shape[0]
    nh, ng, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if m.get("conv"):
        q, k, v = (time_conv(u, w[p + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.reshape(t, nh, d), k.reshape(t, ng, d), v.reshape(t, ng, dv)
    pos = torch.arange(t)
    base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    if dims:
        fq = frequencies(base, dims)
        q, k = turn(q, pos, fq, dims, "halves"), turn(k, pos, fq, dims, "halves")
    fv = frequencies(base, dv)
    v = turn(v, pos, fv, dv, "halves")
    out = torch.zeros((t, nh, dv), dtype=F)
    for a in range(nh):
        g = a // (nh // ng)
        for i in range(t):
            s = (k[:i + 1, g] @ q[i, a]) * m["scale"]
            e = torch.exp(s)
            out[i, a] = (e / (1.0 + e.sum())) @ v[:i + 1, g]
    out = turn(out, -pos, fv, dv, "halves")
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(t, nh * dv) * gate) @ w[p + "o"].T


def latent_attention(w, p, h, m, eps):
    """Queries through a normed latent; keys and values from one normed latent per token plus one turned
    key part that all heads share (pairs, stretched frequencies); a window; ordinary softmax."""
    t = h.shape[0]
    nh, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(t, nh, d + dr)
    kv = h @ w[p + "dkv"].T
    c = unit_rms(kv[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = kv[:, rank:]
    pos = torch.arange(t)
    rot = m["rot"]
    freq, mag = frequencies(float(rot["base"]), dr), 1.0
    if rot.get("scaling"):
        freq, mag = yarn(freq, float(rot["base"]), dr, rot["scaling"])
    q_rot = turn(q[:, :, d:], pos, freq, dr, "pairs", mag)
    k_rot = turn(k_rot, pos, freq, dr, "pairs", mag)
    k_plain = (c @ w[p + "uk"].T).reshape(t, nh, d)
    v = (c @ w[p + "uv"].T).reshape(t, nh, dv)
    window = (m.get("mask") or {}).get("size")
    out = torch.zeros((t, nh, dv), dtype=F)
    for a in range(nh):
        for i in range(t):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k_plain[lo:i + 1, a] @ q[i, a, :d] + k_rot[lo:i + 1] @ q_rot[i, a]) * m["scale"]
            out[i, a] = torch.softmax(s, dim=0) @ v[lo:i + 1, a]
    return out.reshape(t, nh * dv) @ w[p + "o"].T


# ---- feed-forward -----------------------------------------------------------------------------------
def route(z, correction, r):
    """The chosen experts and their weights for one token's router logits ``z`` (all experts, identity ones
    last).  Returns a list of ``(index, weight)``."""
    s = torch.softmax(z, dim=0)
    choice = s + correction
    total = z.shape[0]
    groups = r.get("groups")
    if groups:
        per = total // groups["count"]
        best = sorted(range(groups["count"]), key=lambda g: (-float(choice[g * per:(g + 1) * per].max()), g))
        allowed = set(best[:groups["keep"]])
        choice = torch.tensor([float(choice[e]) if e // per in allowed else -math.inf for e in range(total)], dtype=F)
    order = sorted(range(total), key=lambda e: (-float(choice[e]), e))
    return [(e, s[e]) for e in order[:r["top"]]]


def expert(w, p, h, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(GLU_ALPHA * g) * (u + 1.0)) @ w[p + "down"].T


def moe(w, p, h, mlp):
    r = mlp["router"]
    real = r["experts"]
    z = h @ w[p + "router"].T
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e, weight in route(z[i], w[p + "correction"], r):
            out[i] += weight * (expert(w, f"{p}e{e}.", h[i], mlp["expert"]["limit"]) if e < real else h[i])
    return out


# ---- the model ----------------------------------------------------------------------------------------
def layer(cfg, w, i, x):
    entry = cfg["layers"][i]
    p = f"l{i}."
    h = dyt(x, w, p + "norm1")
    if entry["type"] == "attention":
        y = attention(w, p + "mix.", h, entry["mixer"])
    else:
        y = latent_attention(w, p + "mix.", h, entry["mixer"], cfg["norm"]["eps"])
    x = x + dyt(y, w, p + "norm1b")
    if entry.get("mlp") is not None:
        x = x + dyt(moe(w, p + "mlp.", dyt(x, w, p + "norm2"), entry["mlp"]), w, p + "norm2b")
    return x


def order_of_layers(cfg):
    """``(layer, pass)`` of every layer run; ``pass`` is None outside the loop, and a pass's first run is
    the one with the lowest layer index."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, layers_out=None):
    """Logits ``[T, vocab]`` of one sequence; ``layers_out`` (a list) receives the rows behind every layer run."""
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    x = x0
    loop = cfg.get("loop")
    for i, t in order_of_layers(cfg):
        if t is not None and i == loop["start"]:
            x = torch.cat([x, x0], dim=1) @ w["loop.in"].T + w["loop.step"][t]
        x = layer(cfg, w, i, x)
        if layers_out is not None:
            layers_out.append(x)
    logits = dyt(x, w, "final.norm") @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(cfg, w, prompt, n):
    """``n`` tokens by argmax, each from a whole pass over everything so far."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(torch.argmax(forward(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]
