"""A plain, slow implementation of the Feruzen decoder in float64, one function per mechanism,
written from the design's equations.  It runs one whole sequence at a time on the CPU and shares
no code with the engine; the tests compare the engine with it.

Notation: ``x`` is ``[T, width]``, a linear weight is stored ``[out, in]`` and applied as ``x @ W.T``.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

F = torch.float64


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
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, w, groups, eps):
    """Every row in ``groups`` equal consecutive parts, each divided by its own root mean square."""
    t, n = x.shape
    return unit_rms(x.reshape(t, groups, n // groups), eps).reshape(t, n) * w


def time_conv(x, w):
    """``y_t = sum_j w[:, j] x_(t - taps + 1 + j)`` with zeros before the start; ``w`` is ``[channels, taps]``."""
    t, taps = x.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, x.shape[1]), dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j:j + t] * w[:, j]
    return y


def silu(z):
    return z * torch.sigmoid(z)


def clamped_glu(h, w_gate, w_up, w_down, limit, alpha=1.702):
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)) @ w_down.T


# ---- mixers ---------------------------------------------------------------------------------------
def gated_delta(w, p, h, m, eps):
    t = h.shape[0]
    nh, ng, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(time_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(t, ng, d)
    k = silu(time_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(t, ng, d)
    v = silu(time_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(t, nh, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    out = torch.zeros((t, nh, dv), dtype=F)
    for a in range(nh):
        kv = a // (nh // ng)
        s = torch.zeros((d, dv), dtype=F)
        for i in range(t):
            s = decay[i, a] * s
            u = beta[i, a] * (v[i, a] - s.T @ k[i, kv])
            s = s + torch.outer(k[i, kv], u)
            out[i, a] = s.T @ q[i, kv]
    out = unit_rms(out, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).reshape(t, nh, dv)
    return out.reshape(t, nh * dv) @ w[p + "o"].T


def turn_pairs(x, positions, dims, base):
    """Neighbouring pairs (2i, 2i+1) of the first ``dims`` elements of every head turn by ``p * base^(-2i/dims)``."""
    if dims == 0:
        return x
    freq = base ** (-2.0 * torch.arange(dims // 2, dtype=F) / dims)
    ang = positions.to(F)[:, None] * freq[None]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def causal_attention(w, p, h, m, eps):
    t = h.shape[0]
    nh, ng, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ w[p + "q"].T).reshape(t, nh, d), eps) * w[p + "q.norm"]
    k = unit_rms((h @ w[p + "k"].T).reshape(t, ng, d), eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).reshape(t, ng, dv)
    pos = torch.arange(t)
    q = turn_pairs(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = turn_pairs(k, pos, m["rot"]["dims"], m["rot"]["base"])
    out = torch.zeros((t, nh, dv), dtype=F)
    for a in range(nh):
        kv = a // (nh // ng)
        for i in range(t):
            score = (k[:i + 1, kv] @ q[i, a]) * m["scale"]
            out[i, a] = torch.softmax(score, dim=0) @ v[:i + 1, kv]
    return out.reshape(t, nh * dv) @ w[p + "o"].T


def matrix_memory(w, p, h, m, eps):
    t = h.shape[0]
    nh, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).reshape(t, nh, d) * d ** -0.5
    k = (h @ w[p + "k"].T).reshape(t, nh, d)
    v = (h @ w[p + "v"].T).reshape(t, nh, dv)
    log_i = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = torch.zeros((t, nh, dv), dtype=F)
    for a in range(nh):
        s, n, top = torch.zeros((d, dv), dtype=F), torch.zeros((d,), dtype=F), 0.0
        for i in range(t):
            new_top = max(float(log_f[i, a]) + top, float(log_i[i, a]))
            keep, take = math.exp(float(log_f[i, a]) + top - new_top), math.exp(float(log_i[i, a]) - new_top)
            s = keep * s + take * torch.outer(k[i, a], v[i, a])
            n = keep * n + take * k[i, a]
            top = new_top
            out[i, a] = (s.T @ q[i, a]) / (max(abs(float(n @ q[i, a])), math.exp(-top)) + 1e-6)
    out = unit_rms(out, eps).reshape(t, nh * dv) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def side_by_side(w, p, h, m, eps):
    return (m["left_scale"] * causal_attention(w, p + "left.", h, m["left"], eps)
            + m["right_scale"] * matrix_memory(w, p + "right.", h, m["right"], eps))


# ---- feed-forwards --------------------------------------------------------------------------------
def feed_forward(w, p, h, mlp):
    if mlp["kind"] == "dense":
        return clamped_glu(h, w[p + "gate"], w[p + "up"], w[p + "down"], mlp["limit"])
    score = torch.softmax(h @ w[p + "router"].T, dim=-1)
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        chosen = sorted(range(mlp["router"]["experts"]), key=lambda e: (-float(score[i, e]), e))[:mlp["router"]["top"]]
        for e in chosen:
            q = f"{p}e{e}."
            out[i] += score[i, e] * clamped_glu(h[i:i + 1], w[q + "gate"], w[q + "up"], w[q + "down"],
                                               mlp["expert"]["limit"])[0]
    if mlp.get("shared") is not None:
        q = p + "shared."
        out = out + clamped_glu(h, w[q + "gate"], w[q + "up"], w[q + "down"], mlp["shared"]["limit"])
    return out


# ---- the model ------------------------------------------------------------------------------------
def forward(cfg, w, tokens, layer_rows=None):
    """Logits ``[T, vocab]`` of one sequence; ``layer_rows`` (a list) receives what every layer hands on."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    results = [x]                                     # X_0, X_1, ...: the embedding's rows and every layer's result
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = x + time_conv(x, w[p + "canon1"])
        mix = gated_delta if layer["type"] == "delta" else side_by_side
        x = x + group_norm(mix(w, p + "mix.", h, layer["mixer"], eps), w[p + "norm1"], groups, eps)
        if layer["mlp"] is not None:
            x = x + group_norm(feed_forward(w, p + "mlp.", x, layer["mlp"]), w[p + "norm2"], groups, eps)
        results.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(len(results)))
        if layer_rows is not None:
            layer_rows.append(x)
    return group_norm(x, w["final.norm"], groups, eps) @ w["embed"].T


def greedy(cfg, w, prompt, new_tokens):
    """Greedy continuation by running the whole sequence again for every token."""
    seq = list(prompt)
    for _ in range(new_tokens):
        seq.append(int(torch.argmax(forward(cfg, w, seq)[-1])))
    return seq[len(prompt):]
