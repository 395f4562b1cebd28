"""Arrangement of a layer's parts.

``prenorm`` (reference: src/inference.cu:35-66): ``x += mixer(norm1(x))`` then
``x += ffn(norm2(x))``; both sums happen in the float32 residual stream, inside the
mixer's and the feed-forward's last product.  A layer without a feed-forward stops after the mixer.

``parallel``: ``h = norm(x)``, then ``x += mixer(h)`` and ``x += ffn(h)``.

``sandwich``: a norm before and behind each sublayer, ``x += norm1b(mixer(norm1(x)))`` then
``x += norm2b(ffn(norm2(x)))``.

``output_norm``: the norm sits on the sublayer's output, ``x += norm1(mixer(x + conv(x)))`` then
``x += norm2(ffn(x))``, with an optional short causal convolution over time in front of the mixer
and an optional weighted sum over the results of all layers so far behind the layer.
"""
from __future__ import annotations

import torch

from .base import MATRIX, NORM_WEIGHT, CompositeSpec, FixedStateSpec, Part, WeightSpec, as_float32, register_part


class PreNormBlock(Part):
    category = "block"

    def __init__(self, mixer, mixer_norm, ffn=None, ffn_norm=None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer, self.ffn = mixer, ffn
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm

    def forward(self, ops, x, step, cache):
        self.mixer.forward(ops, self.mixer_norm.forward(ops, x, step.act_dtype), x, step, cache)
        if self.ffn is not None:
            self.ffn.forward(ops, self.ffn_norm.forward(ops, x, step.act_dtype), x, step)


class ParallelBlock(Part):
    """``x += mixer(h) + ffn(h)`` with ``h = norm(x)``: one norm, and both sublayers read its
    output.  Each adds its result to the float32 residual stream in its last product; the
    feed-forward may be absent."""
    category = "block"

    def __init__(self, mixer, mixer_norm, ffn=None, ffn_norm=None):
        if ffn_norm is not None:
            raise ValueError("a parallel block has one norm")
        self.mixer, self.ffn, self.mixer_norm = mixer, ffn, mixer_norm

    def forward(self, ops, x, step, cache):
        h = self.mixer_norm.forward(ops, x, step.act_dtype)
        self.mixer.forward(ops, h, x, step, cache)
        if self.ffn is not None:
            self.ffn.forward(ops, h, x, step)


class SandwichBlock(Part):
    """``x += post1(mixer(pre1(x)))`` then, where the layer has a feed-forward, ``x += post2(ffn(pre2(x)))``:
    every sublayer reads a normed input and its output passes a second norm before it joins the
    float32 residual stream.  The norms behind the sublayers must be able to add to a residual
    (``add_to``)."""
    category = "block"

    def __init__(self, mixer, mixer_norm, mixer_post_norm, ffn=None, ffn_norm=None, ffn_post_norm=None):
        if not ((ffn is None) == (ffn_norm is None) == (ffn_post_norm is None)):
            raise ValueError("a feed-forward and its two norms come together")
        self.mixer, self.ffn = mixer, ffn
        self.mixer_norm, self.mixer_post_norm = mixer_norm, mixer_post_norm
        self.ffn_norm, self.ffn_post_norm = ffn_norm, ffn_post_norm

    def forward(self, ops, x, step, cache):
        y = torch.zeros_like(x)
        self.mixer.forward(ops, self.mixer_norm.forward(ops, x, step.act_dtype), y, step, cache)
        if self.ffn is None:
            self.mixer_post_norm.add_to(ops, y, x)
            return
        if hasattr(self.mixer_post_norm, "add_then") and type(self.ffn_norm) is type(self.mixer_post_norm):
            h = self.mixer_post_norm.add_then(ops, y, x, self.ffn_norm, step.act_dtype)     # both norms in one launch
        else:
            self.mixer_post_norm.add_to(ops, y, x)
            h = self.ffn_norm.forward(ops, x, step.act_dtype)
        y.zero_()
        self.ffn.forward(ops, h, y, step)
        self.ffn_post_norm.add_to(ops, y, x)


class OutputNormBlock(Part):
    """A layer whose norms sit on the sublayers' outputs; the sublayers read the residual stream
    itself (rounded to the activation dtype):

        x += norm1(mixer(x + conv(x)))          x += norm2(ffn(x))

    ``conv`` (``conv_taps`` >= 1; tensor ``canon1`` ``[width, taps]``, no bias) is a causal
    convolution over time on every channel, ``conv(x)_t = sum_j w[:, j] x_(t - taps + 1 + j)``
    with zeros before a sequence's start; the request keeps its last ``taps - 1`` rows of ``x``.

    ``depth_index = i`` (of ``depth_total`` layers) turns on the weighted sum over depth: with
    ``X_0`` the rows that entered layer 0 and ``X_(i+1)`` what the lines above leave, the layer
    hands on ``sum_{j <= i+1} dwa[j] X_j`` (tensor ``dwa`` of ``i + 2`` weights).  The ``X_j`` of a
    step live in the step's scratch.

    The norms must be able to add to a residual (``add_to``).  What the request keeps is a
    composite: the convolution's rows under ``conv``, the mixer's own cache under ``mixer``."""
    category = "block"

    def __init__(self, mixer, mixer_norm, ffn=None, ffn_norm=None, hidden_size: int = 0, conv_taps: int = 0,
                 depth_index=None, depth_total: int = 0):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self.hidden_size, self.conv_taps = int(hidden_size), int(conv_taps)
        self.depth_index = None if depth_index is None else int(depth_index)
        self.depth_total = int(depth_total)
        if self.depth_index is not None and not 0 <= self.depth_index < self.depth_total:
            raise ValueError(f"layer {depth_index} of {depth_total} in the sum over depth")
        self.conv_w = self.dwa = None

    def weight_specs(self):
        specs = {}
        if self.conv_taps >= 1:
            specs["canon1"] = WeightSpec((self.hidden_size, self.conv_taps), MATRIX)
        if self.depth_index is not None:
            specs["dwa"] = WeightSpec((self.depth_index + 2,), NORM_WEIGHT)
        return specs

    def load_weights(self, tensors, ops):
        if self.conv_taps >= 1:
            self.conv_w = as_float32(tensors["canon1"]).contiguous()
        if self.depth_index is not None:
            self.dwa = as_float32(tensors["dwa"]).contiguous()

    def cache_spec(self):
        items = []
        if self.conv_taps > 1:
            items.append(("conv", FixedStateSpec(((self.conv_taps - 1) * self.hidden_size,), torch.float32)))
        items.append(("mixer", self.mixer.cache_spec()))
        return CompositeSpec(tuple(items))

    def forward(self, ops, x, step, cache):
        t, dev = x.shape[0], x.device
        hist = None
        if self.depth_index is not None:
            hist = step.scratch.get("depth_rows")
            if hist is None or hist.shape[0] != self.depth_total + 1 or hist.shape[1] != t:
                hist = torch.empty((self.depth_total + 1, t, self.hidden_size), dtype=torch.float32, device=dev)
                step.scratch["depth_rows"] = hist
            if self.depth_index == 0:
                ops.depth_mix(x, hist, 0)                      # X_0: what enters the first layer
        h = torch.empty((t, self.hidden_size), dtype=step.act_dtype, device=dev)
        kept = cache["conv"] if self.conv_taps > 1 else None
        ops.causal_conv(x, self.conv_w, step, kept, 0, h, add_input=True, renew=True)     # kept rows renewed before x moves on
        y = torch.zeros((t, self.hidden_size), dtype=torch.float32, device=dev)
        self.mixer.forward(ops, h, y, step, cache.child("mixer"))
        self.mixer_norm.add_to(ops, y, x)
        if self.ffn is not None:
            ops.causal_conv(x, None, step, None, 0, h)         # the rows themselves, in the activation dtype
            y.zero_()
            self.ffn.forward(ops, h, y, step)
            self.ffn_norm.add_to(ops, y, x)
        if hist is not None:
            ops.depth_mix(x, hist, self.depth_index + 1, self.dwa)


register_part("block", "prenorm", PreNormBlock)
register_part("block", "output_norm", OutputNormBlock)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "parallel", ParallelBlock)
