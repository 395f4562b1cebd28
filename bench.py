#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096]
    python bench.py --impl reference        # the reference arm (see below)

Default run: the Qwen3-0.6B layer sizes (28 layers, hidden 1024, 16 heads over 8 kv heads of
128, intermediate 3072, vocabulary 151936, tied head) with seeded random weights, 8 requests
decoding at a context of 4,096 tokens, pages of 64 tokens.  A step is one decode step of the
whole batch.  Prints one JSON line:

value      decoded tokens a second, timed on the device with CUDA events over K graph-replayed
           steps with the argmax on the device (nothing is read back inside the timed region);
e2e        the same through the Python entry point (LLM.start and Session.step, after the prompts
           have run): every step schedules, copies its host token ids and block tables to the
           device from pinned memory, decodes, samples and reads the chosen tokens back;
prefill    one request's 2,048-token prompt in one step: tokens a second and the step's
           flops / time / bf16 peak;
roofline   the bytes a decode step has to read (every weight once, and the keys and values of
           the live requests) / its time, against the copy bandwidth;
points     decode tokens a second at batch 1 and 64, the same steps without a CUDA graph, a mixed
           step (63 requests decoding beside a 512-token portion of a prompt that ends between
           3,072 and 4,096 tokens); then, as `page16_*`, `8b_*` and
           `32b_*`, the page size of 16 tokens and the Qwen3-8B and Qwen3-32B shapes (decode at
           batch 1, 8, 64, the 2,048-token prefill, the 8B mixed step);
points_frac  for each point its fraction of its roofline (decode: bytes / time / copy bandwidth;
           prefill: flops / time / the bf16 peak, the sustained one for steps over 5 ms).

``--design kagorax`` leaves all of the above alone and instead prints one JSON line that sets
the Kagorax decoder (attention with a distance bias, kept first tokens and an output gate; a
routed feed-forward) beside the Qwen3 decoder at equal sizes: the same width, heads and window
in every layer, and a dense feed-forward as wide as the rows a token uses of the routed one
(top x expert size + the shared expert).  Per size: the prefill of one prompt and graph-replayed
decode steps of both, in tokens a second, and, from one eager step of each with CUDA events
around the kernel set's calls while the device is kept busy, the time per layer of the kernels
that differ (prompt attention, single-token attention, feed-forward) with each one's fraction of
its roofline: flops / time / bf16 peak for prompt kernels, bytes / time / copy bandwidth for
the kernels of a decode step.

Peaks come from MEASURED_PEAKS.json beside this file when present, else from an earlier
measurement on this pool (6.65 TB/s, 1.59 PFLOP/s), and the fractions say which.  The working
set (1.2 GB of weights and gigabytes of cache) is far larger than the 126 MB L2, so no flush is
needed between steps.  Keys and values of the decoding requests are filled with random numbers
instead of being computed from prompts: a decode step's work does not depend on their values.

The reference arm (``--impl reference``): beyondHJM/tinyinfer.cpp is a CMake project of C++/CUDA
executables, not a Python package, so the offline `pip install` fails ("Neither 'setup.py' nor
'pyproject.toml' found").  Its command-line program is instead built from an untouched copy of
its tree under ``baseline/_ref/src`` with its own CMakeLists (sm_100) into
``baseline/_ref/build/tinyinfer`` and run through its own command line on a GGUF file of the same
shape with seeded random weights: ``--batch`` prompts of three tokens each, decoded greedily to
the context length with ``--cuda-graph``.  Its prompts stay this short because a pass of more than
32 tokens takes its tiled mma.sync product, which reads past its shared tile as the sources
stand (src/cuda/gemm.cu:156,201: found by reading and by running that code on the CPU under the
address sanitizer, tests/golden/make_golden.py --asan --long-pass 40; on a B200 such a pass ended
with an illegal memory access) and is therefore never run here.  The number it reports is its own
("main: decode: ... tok/s", src/main.cpp:306-308): tokens a second over the whole decode, from a
context of 3 to the full one, where this engine's `value` is taken at the full context.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_0_6B = dict(
    architectures=["Qwen3ForCausalLM"], num_hidden_layers=28, hidden_size=1024,
    num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
    max_position_embeddings=4096)
# the two larger shapes of the same architecture (untied heads)
QWEN3_8B = dict(QWEN3_0_6B, num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
                num_key_value_heads=8, intermediate_size=12288, tie_word_embeddings=False)
QWEN3_32B = dict(QWEN3_0_6B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                 num_key_value_heads=8, intermediate_size=25600, tie_word_embeddings=False)
SHAPES = {"0.6b": ("Qwen3-0.6B shape", QWEN3_0_6B), "8b": ("Qwen3-8B shape", QWEN3_8B),
          "32b": ("Qwen3-32B shape", QWEN3_32B)}
PAGE = 64
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
MAX_POSITION = 40960           # the longest context of the published models of this architecture


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"]))}, "measured"
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS), "fallback"


def flops_peak(pk, ms):
    """The bf16 peak a step of `ms` milliseconds is held against: the burst figure for a short
    step, the figure sustained under the power cap for one of more than a few milliseconds."""
    if ms > 5.0:
        return pk["bf16_tflops_sustained"], "sustained"
    return pk["bf16_tflops"], "burst"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.lines: list[str] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def model_numbers(cfg):
    h, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    nq = cfg["num_attention_heads"] * cfg["head_dim"]
    nk = cfg["num_key_value_heads"] * cfg["head_dim"]
    inter, vocab = cfg["intermediate_size"], cfg["vocab_size"]
    layer_params = (nq + 2 * nk) * h + h * nq + 3 * inter * h
    head_params = vocab * h
    weight_bytes = 2 * (L * layer_params + head_params) + 4 * (L * (2 * h + 2 * cfg["head_dim"]) + h)
    if not cfg["tie_word_embeddings"]:
        pass                                     # the embedding table is gathered, not streamed
    kv_bytes_per_token = L * 2 * nk * 2
    return dict(layer_params=layer_params, head_params=head_params, weight_bytes=weight_bytes,
                kv_bytes_per_token=kv_bytes_per_token, nq=nq)


def prefill_flops(cfg, t):
    n = model_numbers(cfg)
    gemm = 2.0 * t * cfg["num_hidden_layers"] * n["layer_params"] + 2.0 * n["head_params"]
    attn = cfg["num_hidden_layers"] * 4.0 * n["nq"] * t * (t + 1) / 2.0
    return gemm + attn


def fill_requests(engine, batch, context, torch):
    """``batch`` live requests holding ``context`` tokens each, keys and values random."""
    ids = [("bench", i) for i in range(batch)]
    engine.cache.reserve_step([(r, context) for r in ids], engine.plan.max_position)
    for g in engine.cache.groups:
        g.storage.normal_(0.0, 1.0)
    return ids


def decode_device_timed(engine, ids, steps, warmup, torch):
    """K graph-replayed decode steps with the argmax on the device; nothing is read back
    inside the timed region, so host work overlaps the device's."""
    from tinyinfer_b200 import StepEntry
    b = len(ids)
    out = torch.empty(b, dtype=torch.int32, device=engine.device)

    def one():
        logits = engine.decode_step([StepEntry(r, [1], [0]) for r in ids])
        engine.ops.argmax(logits, out)

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    before = engine.ops.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler() as clocks:
        start.record()
        for _ in range(steps):
            one()
        stop.record()
        torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    return ms / steps, clocks.summary(), engine.ops.launches - before


def decode_eager_timed(engine, batch, context, steps, warmup, torch):
    """The same decode steps launched kernel by kernel (no CUDA graph): what the graphs save."""
    from tinyinfer_b200 import StepEntry
    ids = fill_requests(engine, batch, context - (steps + warmup) - 2, torch)
    out = torch.empty(batch, dtype=torch.int32, device=engine.device)
    graphs, engine._step_graphs = engine._step_graphs, None
    try:
        def one():
            engine.ops.argmax(engine.step([StepEntry(r, [1], [0]) for r in ids]), out)
        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            one()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps
    finally:
        engine._step_graphs = graphs
        for r in ids:
            engine.finish(r)


def decode_e2e(llm, batch, context, steps, warmup, torch):
    """The same steps through the Python entry point (``LLM.start`` / ``Session.step``): prompts
    are run first; then every timed step packs the host's token ids, copies them to the device
    from pinned memory, decodes, samples and reads the chosen tokens back."""
    from tinyinfer_b200 import SamplingParams
    g = torch.Generator().manual_seed(1)
    # requests that finish their prompt early decode while the others' prompts still run: room
    # for those tokens, so that nobody reaches its limit inside the timed steps
    slack = -(-batch * context // llm.max_batched_tokens) + batch + 4
    prompt_len = context - (steps + warmup) - slack - 2
    prompts = [torch.randint(0, llm.engine.plan.vocab_size, (prompt_len,), generator=g).tolist()
               for _ in range(batch)]
    session = llm.start(prompts, SamplingParams(max_tokens=steps + warmup + slack + 1))
    while not all(r.output for r in session.requests):      # the prompts, in portions
        session.step()
    for _ in range(warmup):
        session.step()
    torch.cuda.synchronize()
    buckets = llm.engine._graphs.buckets
    copied = sum(bk.copied_ints for bk in buckets.values())
    t0 = time.perf_counter()
    for _ in range(steps):
        made = session.step()
        assert len(made) == batch
    torch.cuda.synchronize()
    sec = time.perf_counter() - t0
    copied = sum(bk.copied_ints for bk in buckets.values()) - copied
    while not session.done:
        session.step()
    session.finish()
    # what a step copies: its tokens, positions, lengths and slots, and the block-table entries
    # its requests gained (a mean over the timed steps), not the whole table
    return sec / steps * 1e3, round(copied * 4 / steps), batch * 4


def measure_decode(engine, batch, context, steps, warmup, torch):
    ids = fill_requests(engine, batch, context - (steps + warmup) - 2, torch)
    try:
        return decode_device_timed(engine, ids, steps, warmup, torch)
    finally:
        for r in ids:
            engine.finish(r)


def measure_prefill(engine, tokens, reps, torch):
    from tinyinfer_b200 import StepEntry
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, engine.plan.vocab_size, (tokens,), generator=g).tolist()
    times = []
    for i in range(reps + 3):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry(("prefill", i), prompt, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.finish(("prefill", i))
        if i >= 3:                       # the first steps run eagerly and capture the step's graph
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


def measure_mixed(engine, decoders, chunk, context, torch):
    """One step with ``decoders`` requests decoding near ``context`` and a portion of ``chunk``
    tokens of another request's prompt beside them (the step shape of chunked prefill under
    load).  The prompt's first tokens run alone; then five portions follow beside the decoders, the
    last one ending at ``context``: the first two steps run eagerly and capture the shape's
    graph, the other three are timed.  Returns ms per step (median)."""
    from tinyinfer_b200 import StepEntry
    g = torch.Generator().manual_seed(2)
    steps, timed = 5, 3
    lead = max(chunk, context - steps * chunk)
    ids = fill_requests(engine, decoders, context - steps - 2, torch)
    prompt = torch.randint(0, engine.plan.vocab_size, (lead + steps * chunk,), generator=g).tolist()
    times = []
    try:
        engine.step([StepEntry(("bench", "prompt"), prompt[:lead], [])])
        for i in range(steps):
            entries = [StepEntry(r, [1], [0]) for r in ids]
            entries.append(StepEntry(("bench", "prompt"), prompt[lead + i * chunk:lead + (i + 1) * chunk], []))
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            engine.step(entries)
            stop.record()
            torch.cuda.synchronize()
            if i >= steps - timed:
                times.append(start.elapsed_time(stop))
    finally:
        for r in ids + [("bench", "prompt")]:
            engine.finish(r)
    return statistics.median(times)


def measure_chains(engine, batch, torch):
    """Each decode product alone: a CUDA graph of 56 dependent launches with distinct weights,
    timed with CUDA events; microseconds per launch."""
    ops, dev, bf = engine.ops, engine.device, torch.bfloat16
    cfg = engine.config
    h, inter = cfg.hidden_size, cfg.intermediate_size
    nq = cfg.num_attention_heads * cfg.head_dim
    nqkv = nq + 2 * cfg.num_key_value_heads * cfg.head_dim

    def rnd(*shape):
        return torch.randn(*shape, device=dev).to(bf)

    x, xb, o, y = torch.randn(batch, h, device=dev), rnd(batch, h), rnd(batch, nq), rnd(batch, inter)
    qkv = torch.empty(batch, nqkv, device=dev)
    yo = torch.empty(batch, inter, device=dev, dtype=bf)
    xn = torch.empty(batch, h, device=dev, dtype=bf)
    norm_w = torch.ones(h, device=dev)
    n = 56
    wq, wo = [rnd(nqkv, h) for _ in range(n)], [rnd(h, nq) for _ in range(n)]
    wg = [ops.pack_gate_up(rnd(inter, h), rnd(inter, h)) for _ in range(n)]
    wd = [rnd(h, inter) for _ in range(n)]
    cases = {
        "qkv": lambda: [ops.linear(xb, w, qkv) for w in wq],
        "o_accumulate": lambda: [ops.linear(o, w, x, accumulate=True) for w in wo],
        "gate_up_swiglu": lambda: [ops.gate_up_swiglu(xb, w, yo) for w in wg],
        "down_accumulate": lambda: [ops.linear(y, w, x, accumulate=True) for w in wd],
        "rmsnorm": lambda: [ops.rmsnorm(x, norm_w, 1e-6, xn) for _ in range(n)],
    }
    out = {}
    for name, fn in cases.items():
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        for _ in range(3):
            graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(20):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        out[name] = round(start.elapsed_time(stop) / 20 / n * 1e3, 2)
    return out


def shape_points(shape_key, page_size, context, steps, warmup, batches, prefill, mixed, pk, torch, prefix):
    """Decode at the given batches, the 2,048-token prefill and the mixed step for another shape
    or page size, each with its fraction of its roofline.  Returns (points, fractions)."""
    import gc
    from tinyinfer_b200 import LLM
    shape_name, shape_cfg = SHAPES[shape_key]
    cfg = dict(shape_cfg, max_position_embeddings=MAX_POSITION)
    nums = model_numbers(cfg)
    max_batch = max(list(batches) + ([64] if mixed else []) + [1])
    llm = LLM(config=cfg, seed=0, dtype="bfloat16", page_size=page_size, max_seq=context,
              max_num_seqs=max_batch + 1, kv_tokens=max_batch * context, cuda_graph=True)
    engine = llm.engine
    points, fracs = {}, {}
    try:
        for b in batches:
            n = min(steps, 32)
            ms, _, _ = measure_decode(engine, b, context, n, warmup, torch)
            points[f"{prefix}decode_b{b}"] = round(b / (ms * 1e-3), 1)
            step_bytes = nums["weight_bytes"] + b * (context - n // 2) * nums["kv_bytes_per_token"]
            fracs[f"{prefix}decode_b{b}"] = round(step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        if prefill:
            ms = measure_prefill(engine, 2048, 3, torch)
            peak, which = flops_peak(pk, ms)
            points[f"{prefix}prefill_2048"] = round(2048 / (ms * 1e-3), 1)
            fracs[f"{prefix}prefill_2048"] = round(prefill_flops(cfg, 2048) / (ms * 1e-3) / (peak * 1e12), 4)
            fracs[f"{prefix}prefill_2048_peak"] = which
        if mixed:
            ms = measure_mixed(engine, 63, 512, context, torch)
            points[f"{prefix}mixed_63_decoding_512_portion"] = round((63 + 512) / (ms * 1e-3), 1)
    finally:
        del engine, llm
        gc.collect()
        torch.cuda.empty_cache()
    return points, fracs


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


# ---- the Kagorax decoder beside the Qwen3 decoder at equal sizes --------------------------------
# (width, heads, kv heads, head size, window, kept first tokens, experts, top, expert size, shared size, layers)
DESIGN_SIZES = {
    "w1024": (1024, 16, 8, 128, 1024, 4, 32, 4, 512, 1024, 8),
    "w2048": (2048, 32, 4, 128, 2048, 4, 64, 8, 768, 768, 6),
    "w4096_h64": (4096, 64, 8, 64, 4096, 16, 32, 2, 2048, 2048, 4),
}
DESIGN_VOCAB = 32768


def kagorax_config(size):
    w, h, g, d, win, keep, experts, top, ff, shared, layers = size
    layer = {"type": "attention",
             "mixer": {"heads": h, "kv_heads": g, "dim": d, "vdim": d, "scale": d ** -0.5, "bias_max": 4 * win,
                       "bias_rows": 32, "mask": {"size": win, "keep_first": keep}},
             "mlp": {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
                     "shared": {"ff": shared}}}
    return {"architecture": "Kagorax", "vocab": DESIGN_VOCAB, "width": w, "embedding": {"scale": float(w) ** 0.5},
            "norm": {"eps": 1e-5}, "layers": [layer] * layers}


def qwen3_like_config(size, context):
    w, h, g, d, win, keep, experts, top, ff, shared, layers = size
    return dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=layers, hidden_size=w,
                num_attention_heads=h, num_key_value_heads=g, head_dim=d, intermediate_size=top * ff + shared,
                vocab_size=DESIGN_VOCAB, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
                max_position_embeddings=context, sliding_window=win, layer_types=["sliding_attention"] * layers)


def timed_ops(engine, names, run, torch):
    """Milliseconds the device spends inside each named call of the kernel set during ``run()``:
    CUDA events around every call, with the device kept busy beforehand so that the host's
    launches run ahead of it."""
    ops = engine.ops
    spans = {n: [] for n in names}
    originals = {n: getattr(ops, n) for n in names}

    def wrap(name, fn):
        def inner(*a, **k):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            out = fn(*a, **k)
            a1.record()
            # a product is told apart by its weight's shape and whether it adds to its output
            what = (tuple(a[1].shape), bool(k.get("accumulate", a[3] if len(a) > 3 else False))) if name == "linear" else None
            spans[name].append((a0, a1, what))
            return out
        return inner

    for n in names:
        setattr(ops, n, wrap(n, originals[n]))
    try:
        torch.cuda.synchronize()
        torch.cuda._sleep(12_000_000)                # about 6 ms: the launches of a whole step queue up behind it
        run()
        torch.cuda.synchronize()
    finally:
        for n in names:
            delattr(ops, n)
    out = {n: [a.elapsed_time(b) for a, b, _ in v] for n, v in spans.items()}
    out["_linear_kinds"] = [what for _, _, what in spans.get("linear", [])]
    return out


def design_arm(args) -> int:
    import torch
    from tinyinfer_b200 import Engine, StepEntry
    pk, pk_kind = peaks()
    prompt_len, batch, context = args.prefill_tokens, args.batch, args.context
    warmup = max(args.warmup, 3)
    out = {"design": "kagorax", "beside": "qwen3 at equal sizes", "peaks": pk_kind, "prefill_tokens": prompt_len,
           "decode_batch": batch, "decode_context": context, "dtype": "bf16", "data": "synthetic", "sizes": {}}
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, DESIGN_VOCAB, (prompt_len,), generator=g).tolist()
    for key, size in DESIGN_SIZES.items():
        if args.design_size and key != args.design_size:
            continue
        w, h, kvh, d, win, keep, experts, top, ff, shared, layers = size
        res = {}
        # rooflines of the kernels that differ, per layer
        seen = sum(min(i + 1, win) + min(keep, max(0, i + 1 - win)) for i in range(prompt_len))
        attn_flops = 4.0 * h * d * seen
        dec_keys = min(context, win + keep)
        attn_bytes = batch * kvh * dec_keys * 2 * d * 2.0
        ffn_flops = {"kagorax": 2.0 * prompt_len * 3 * w * (top * ff + shared), "qwen3": 2.0 * prompt_len * 3 * w * (top * ff + shared)}
        ffn_bytes = {"kagorax": 2.0 * 3 * w * (min(experts, batch * top) * ff + shared), "qwen3": 2.0 * 3 * w * (top * ff + shared)}
        for arm, cfg, calls in (
                ("kagorax", kagorax_config(size), {"attention": ["biased_attention"], "ffn": ["router_topk", "routed_experts"],
                             "inside": ["gate_up_swiglu", "scale_rows"]}),   # the shared expert runs inside routed_experts
                ("qwen3", qwen3_like_config(size, max(context, prompt_len) + 64), {"attention": ["paged_attention"], "ffn": ["swiglu_ffn"]})):
            engine = Engine(config=cfg, seed=0, dtype="bfloat16", page_size=args.page_size,
                            num_pages=-(-max(batch * context, prompt_len) // args.page_size) + batch + 2,
                            max_requests=batch + 1, step_graphs=True)
            pf_ms = measure_prefill(engine, prompt_len, max(1, min(args.steps, 6)), torch)
            ms, clocks, launches = measure_decode(engine, batch, context, args.steps, warmup, torch)
            a = {"prefill_tok_s": round(prompt_len / pf_ms * 1e3), "prefill_ms": round(pf_ms, 3),
                 "decode_tok_s": round(batch / ms * 1e3, 1), "decode_ms_per_step": round(ms, 4),
                 "decode_launches_per_step": launches // max(1, args.steps), "clocks": clocks}
            names = calls["attention"] + calls["ffn"] + calls.get("inside", []) + (["linear"] if arm == "kagorax" else [])
            engine._step_graphs = None
            engine.ops.fuse_decode_tail = engine.ops.fuse_decode_ffn = False   # the feed-forward as a call of its own
            for _ in range(2):        # the first eager step sizes the allocator's pool; the second is read
                spans = timed_ops(engine, names, lambda: engine.step([StepEntry("p", prompt, [prompt_len - 1])]), torch)
                engine.finish("p")
            ids = fill_requests(engine, batch, context - 4, torch)
            for _ in range(2):
                dspans = timed_ops(engine, names, lambda: engine.step([StepEntry(r, [1], [0]) for r in ids]), torch)
            for r in ids:
                engine.finish(r)

            def per_layer(sp, which):
                return sum(sum(sp[n]) for n in calls[which]) / layers

            if arm == "kagorax":          # of a layer's products the router's belongs to the feed-forward
                def ffn_products(sp):     # (the shared expert's are timed inside routed_experts)
                    router_rows = -(-(experts + 1) // 16) * 16
                    return sum(ms_ for ms_, ((n_, k_), acc) in zip(sp["linear"], sp["_linear_kinds"])
                               if n_ == router_rows and k_ == w and not acc) / layers
                extra, dextra = ffn_products(spans), ffn_products(dspans)
            else:
                extra = dextra = 0.0
            pa, da = per_layer(spans, "attention"), per_layer(dspans, "attention")
            pff, dff = per_layer(spans, "ffn") + extra, per_layer(dspans, "ffn") + dextra
            a["per_layer_us"] = {"prompt_attention": round(pa * 1e3, 1), "decode_attention": round(da * 1e3, 1),
                                 "prompt_ffn": round(pff * 1e3, 1), "decode_ffn": round(dff * 1e3, 1)}
            a["calls_per_layer_us"] = {
                "prompt": {n: round(sum(v) / layers * 1e3, 1) for n, v in spans.items() if not n.startswith("_")},
                "decode": {n: round(sum(v) / layers * 1e3, 1) for n, v in dspans.items() if not n.startswith("_")}}
            a["roofline_frac"] = {
                "prompt_attention": round(attn_flops / (pa * 1e-3) / (pk["bf16_tflops"] * 1e12), 3),
                "decode_attention": round(attn_bytes / (da * 1e-3) / (pk["hbm_gbs"] * 1e9), 3),
                "prompt_ffn": round(ffn_flops[arm] / (pff * 1e-3) / (pk["bf16_tflops"] * 1e12), 3),
                "decode_ffn": round(ffn_bytes[arm] / (dff * 1e-3) / (pk["hbm_gbs"] * 1e9), 3)}
            res[arm] = a
            del engine
            torch.cuda.empty_cache()
        out["sizes"][key] = {"width": w, "heads": h, "kv_heads": kvh, "head_dim": d, "window": win, "keep_first": keep,
                             "experts": experts, "top": top, "expert_ff": ff, "shared_ff": shared, "layers": layers, **res}
    print(json.dumps(out))
    return 0


# ---- the Ruvuvik decoder beside the Qwen3 decoder at equal sizes --------------------------------
# (width, heads, kv heads, head size, chunk, latent rank, rotated part, recurrent head size, ff, blocks of
# [attention, latent attention, recurrent] layers)
RUVUVIK_SIZES = {
    "w1024": (1024, 16, 4, 64, 1024, 256, 32, 64, 2816, 2),
    "w2048": (2048, 16, 4, 128, 2048, 512, 64, 64, 5632, 2),
    "w4096": (4096, 32, 8, 128, 4096, 512, 64, 64, 11008, 1),
}


def ruvuvik_config(size):
    w, h, g, d, chunk, rank, dr, rd, ff, blocks = size
    mlp = {"kind": "dense", "ff": ff}
    layers = [
        {"type": "attention", "mlp": mlp,
         "mixer": {"heads": h, "kv_heads": g, "dim": d, "vdim": d, "mask": {"size": chunk},
                   "rot": {"dims": d, "base": 10000.0}, "scale": d ** -0.5, "softcap": 50.0}},
        {"type": "latent_attention", "mlp": mlp,
         "mixer": {"heads": h, "dim": d, "rot_dim": dr, "vdim": d, "kv_rank": rank,
                   "rot": {"dims": dr, "base": 100000.0}, "scale": (d + dr) ** -0.5}},
        {"type": "wkv", "mlp": mlp, "mixer": {"heads": w // rd, "dim": rd, "decay_rank": 64}}]
    return {"architecture": "Ruvuvik", "vocab": DESIGN_VOCAB, "width": w, "norm": {"eps": 1e-5},
            "layers": layers * blocks}


def qwen3_beside_ruvuvik(size, context):
    w, h, g, d, chunk, rank, dr, rd, ff, blocks = size
    return dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3 * blocks, hidden_size=w,
                num_attention_heads=h, num_key_value_heads=g, head_dim=d, intermediate_size=ff * 2 // 3 // 64 * 64,
                vocab_size=DESIGN_VOCAB, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                max_position_embeddings=context)


def ruvuvik_arm(args) -> int:
    """Prefill and decode throughput of the Ruvuvik decoder at sizes of real layers, beside the
    Qwen3 decoder with as many layers of the same width, heads and head size (its feed-forward has
    three matrices of two thirds the inner width, so the feed-forwards move as many bytes), and the
    time the device spends in every kind of kernel call per layer, with the fraction of the
    roofline for the calls that have one."""
    import torch
    from tinyinfer_b200 import Engine, StepEntry
    pk, pk_kind = peaks()
    prompt_len, batch, context = args.prefill_tokens, args.batch, args.context
    warmup = max(args.warmup, 3)
    out = {"design": "ruvuvik", "beside": "qwen3 at equal sizes", "peaks": pk_kind, "prefill_tokens": prompt_len,
           "decode_batch": batch, "decode_context": context, "dtype": "bf16", "data": "synthetic", "sizes": {}}
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, DESIGN_VOCAB, (prompt_len,), generator=g).tolist()
    for key, size in RUVUVIK_SIZES.items():
        if args.design_size and key != args.design_size:
            continue
        w, h, kvh, d, chunk, rank, dr, rd, ff, blocks = size
        res = {}
        calls = {"ruvuvik": ["attention_options", "qk_rownorm_rope_store", "latent_prepare", "head_project",
                             "token_shift_mix", "wkv_recurrence", "tanh_rows", "xielu_rows", "linear", "rmsnorm"],
                 "qwen3": ["paged_attention", "qkv_rope_store", "swiglu_ffn", "linear", "rmsnorm"]}
        for arm, cfg in (("ruvuvik", ruvuvik_config(size)),
                         ("qwen3", qwen3_beside_ruvuvik(size, max(context, prompt_len) + 64))):
            engine = Engine(config=cfg, seed=0, dtype="bfloat16", page_size=args.page_size,
                            num_pages=-(-max(batch * context, prompt_len) // args.page_size) + batch + 2,
                            max_requests=batch + 1, step_graphs=True)
            pf_ms = measure_prefill(engine, prompt_len, max(1, min(args.steps, 6)), torch)
            ms, clocks, launches = measure_decode(engine, batch, context, args.steps, warmup, torch)
            a = {"prefill_tok_s": round(prompt_len / pf_ms * 1e3), "prefill_ms": round(pf_ms, 3),
                 "decode_tok_s": round(batch / ms * 1e3, 1), "decode_ms_per_step": round(ms, 4),
                 "decode_launches_per_step": launches // max(1, args.steps), "clocks": clocks}
            engine._step_graphs = None
            engine.ops.fuse_decode_tail = engine.ops.fuse_decode_ffn = False   # every call of its own
            names = calls[arm]
            for _ in range(2):        # the first eager step sizes the allocator's pool; the second is read
                spans = timed_ops(engine, names, lambda: engine.step([StepEntry("p", prompt, [prompt_len - 1])]), torch)
                engine.finish("p")
            ids = fill_requests(engine, batch, context - 4, torch)
            for _ in range(2):
                dspans = timed_ops(engine, names, lambda: engine.step([StepEntry(r, [1], [0]) for r in ids]), torch)
            for r in ids:
                engine.finish(r)
            n_layers = 3 * blocks
            a["calls_us"] = {
                "prompt": {n: [round(x * 1e3, 1) for x in v[:12]] for n, v in spans.items() if not n.startswith("_") and n != "linear"},
                "decode": {n: [round(x * 1e3, 1) for x in v[:12]] for n, v in dspans.items() if not n.startswith("_") and n != "linear"}}
            a["per_layer_us"] = {
                "prompt": {n: round(sum(v) / n_layers * 1e3, 1) for n, v in spans.items() if not n.startswith("_")},
                "decode": {n: round(sum(v) / n_layers * 1e3, 1) for n, v in dspans.items() if not n.startswith("_")}}
            # rooflines of the attention calls: useful flops of a prompt, cache bytes of a decode step
            if arm == "ruvuvik":
                seen_chunk = sum(i % chunk + 1 for i in range(prompt_len))
                seen_all = prompt_len * (prompt_len + 1) / 2
                att = spans["attention_options"]
                datt = dspans["attention_options"]
                row = rank + dr
                a["roofline_frac"] = {
                    "prompt_chunked_attention": round(4.0 * h * d * seen_chunk / (att[0] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    # the latent form multiplies rows of rank + rotated part and sums rows of rank
                    "prompt_latent_attention": round(2.0 * h * (row + rank) * seen_all / (att[1] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "decode_chunked_attention": round(batch * kvh * ((context - 1) % chunk + 1) * 2 * d * 2.0 / (datt[0] * 1e-3) / (pk["hbm_gbs"] * 1e9), 4),
                    "decode_latent_attention": round(batch * context * row * 2.0 / (datt[1] * 1e-3) / (pk["hbm_gbs"] * 1e9), 4),
                    # the recurrence reads r, k, v, g and the decay's argument (float32) and writes a row
                    "prompt_recurrence_bytes": round(prompt_len * w * (5 * 4 + 2.0) / (spans["wkv_recurrence"][0] * 1e-3) / (pk["hbm_gbs"] * 1e9), 4),
                    "decode_recurrence_state_bytes": round(batch * (w // rd) * rd * rd * 8.0 / (dspans["wkv_recurrence"][0] * 1e-3) / (pk["hbm_gbs"] * 1e9), 4)}
            else:
                att, datt = spans["paged_attention"], dspans["paged_attention"]
                a["roofline_frac"] = {
                    "prompt_attention": round(4.0 * h * d * prompt_len * (prompt_len + 1) / 2 / (att[0] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "decode_attention": round(batch * kvh * context * 2 * d * 2.0 / (datt[0] * 1e-3) / (pk["hbm_gbs"] * 1e9), 4)}
            res[arm] = a
            del engine
            torch.cuda.empty_cache()
        out["sizes"][key] = {"width": w, "heads": h, "kv_heads": kvh, "head_dim": d, "chunk": chunk, "kv_rank": rank,
                             "rot_dim": dr, "recurrent_head": rd, "ff": ff, "layers": 3 * blocks, **res}
    print(json.dumps(out))
    return 0


# ---- the Feruzen decoder beside the Ruvuvik decoder at equal sizes ------------------------------
# (width, attention heads, kv heads, head size, delta heads, delta key heads, delta key size, delta value size,
#  memory heads, memory key size, memory value size, dense ff, experts, top, expert ff, shared ff, blocks of
#  [delta + dense, side by side + experts, side by side + dense] layers)
FERUZEN_SIZES = {
    "w1024": (1024, 16, 4, 64, 8, 4, 64, 128, 4, 64, 128, 2816, 16, 2, 704, 1408, 2),
    "w2048": (2048, 16, 4, 128, 16, 8, 128, 128, 8, 128, 128, 5632, 32, 4, 704, 2816, 2),
    "w4096": (4096, 32, 8, 128, 32, 16, 128, 128, 8, 128, 512, 11008, 64, 4, 1408, 5632, 1),
}


def feruzen_config(size):
    w, h, g, d, dh, dg, dd, dv, mh, md, mv, ff, experts, top, eff, sff, blocks = size
    delta = {"type": "delta", "mixer": {"heads": dh, "kv_heads": dg, "dim": dd, "vdim": dv, "conv": 4}}
    sides = {"type": "parallel", "mixer": {
        "left": {"heads": h, "kv_heads": g, "dim": d, "vdim": d, "rot": {"dims": d, "base": 500000.0}, "scale": d ** -0.5},
        "right": {"heads": mh, "dim": md, "vdim": mv, "gate_cap": 15.0}, "left_scale": 1.0, "right_scale": 1.0}}
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": eff, "limit": 7.0},
           "shared": {"ff": sff, "limit": 7.0}}
    layers = [dict(delta, mlp=dense), dict(sides, mlp=moe), dict(sides, mlp=dense)]
    return {"architecture": "Feruzen", "vocab": DESIGN_VOCAB, "width": w, "norm": {"eps": 1e-6, "groups": 4},
            "canon": {"taps": 4}, "layers": layers * blocks}


def feruzen_arm(args) -> int:
    """Prefill and decode throughput of the Feruzen decoder at sizes of real layers, beside the
    Ruvuvik decoder (the closest design the engine has: attention with options and a recurrent mixer
    with a matrix state) with as many layers of the same width, attention heads and head size, and
    the time the device spends in every kind of kernel call per layer, with the fraction of the
    roofline for the calls that have one."""
    import torch
    from tinyinfer_b200 import Engine, StepEntry
    pk, pk_kind = peaks()
    prompt_len, batch, context = args.prefill_tokens, args.batch, args.context
    warmup = max(args.warmup, 3)
    out = {"design": "feruzen", "beside": "ruvuvik at equal sizes", "peaks": pk_kind, "prefill_tokens": prompt_len,
           "decode_batch": batch, "decode_context": context, "dtype": "bf16", "data": "synthetic", "sizes": {}}
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, DESIGN_VOCAB, (prompt_len,), generator=g).tolist()
    hbm, tc = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    # float32 multiply-adds on the CUDA cores (128 lanes an SM, the clock's maximum): what a walk over a float32 state
    # is held against besides its bytes, since every state element takes a few of them per token
    props = torch.cuda.get_device_properties(0)
    fp32 = props.multi_processor_count * 128 * 2.0 * getattr(props, "clock_rate", 1965000) * 1e3
    for key, size in FERUZEN_SIZES.items():
        if args.design_size and key != args.design_size:
            continue
        w, h, kvh, d, dh, dg, dd, dv, mh, md, mv, ff, experts, top, eff, sff, blocks = size
        beside = (w, h, kvh, d, max(context, prompt_len) + 64, 512, 64, 64, ff, blocks)
        res = {}
        calls = {"feruzen": ["attention_options", "qk_rownorm_rope_store", "matrix_state", "causal_conv", "conv_tail_store",
                             "group_norm", "depth_mix", "add_scaled", "glu_ffn", "glu_rows", "router_topk", "routed_experts", "linear"],
                 "ruvuvik": ["attention_options", "qk_rownorm_rope_store", "latent_prepare", "head_project",
                             "token_shift_mix", "wkv_recurrence", "tanh_rows", "linear_xielu", "xielu_rows", "linear", "rmsnorm"]}
        for arm, cfg in (("feruzen", feruzen_config(size)), ("ruvuvik", ruvuvik_config(beside))):
            engine = Engine(config=cfg, seed=0, dtype="bfloat16", page_size=args.page_size,
                            num_pages=-(-max(batch * context, prompt_len) // args.page_size) + batch + 2,
                            max_requests=batch + 1, step_graphs=True)
            pf_ms = measure_prefill(engine, prompt_len, max(1, min(args.steps, 6)), torch)
            ms, clocks, launches = measure_decode(engine, batch, context, args.steps, warmup, torch)
            a = {"prefill_tok_s": round(prompt_len / pf_ms * 1e3), "prefill_ms": round(pf_ms, 3),
                 "decode_tok_s": round(batch / ms * 1e3, 1), "decode_ms_per_step": round(ms, 4),
                 "decode_launches_per_step": launches // max(1, args.steps), "clocks": clocks}
            engine._step_graphs = None
            engine.ops.fuse_decode_tail = engine.ops.fuse_decode_ffn = False   # every call of its own
            names = calls[arm]
            for _ in range(2):        # the first eager step sizes the allocator's pool; the second is read
                spans = timed_ops(engine, names, lambda: engine.step([StepEntry("p", prompt, [prompt_len - 1])]), torch)
                engine.finish("p")
            ids = fill_requests(engine, batch, context - 4, torch)
            for _ in range(2):
                dspans = timed_ops(engine, names, lambda: engine.step([StepEntry(r, [1], [0]) for r in ids]), torch)
            for r in ids:
                engine.finish(r)
            n_layers = 3 * blocks
            a["calls_us"] = {
                "prompt": {n: [round(x * 1e3, 1) for x in v[:12]] for n, v in spans.items() if not n.startswith("_") and n != "linear"},
                "decode": {n: [round(x * 1e3, 1) for x in v[:12]] for n, v in dspans.items() if not n.startswith("_") and n != "linear"}}
            a["per_layer_us"] = {
                "prompt": {n: round(sum(v) / n_layers * 1e3, 1) for n, v in spans.items() if not n.startswith("_")},
                "decode": {n: round(sum(v) / n_layers * 1e3, 1) for n, v in dspans.items() if not n.startswith("_")}}
            seen_all = prompt_len * (prompt_len + 1) / 2

            def frac(amount, ms_, peak):
                return round(amount / (ms_ * 1e-3) / peak, 4)

            if arm == "feruzen":
                # calls in layer order: the delta layer's recurrence first, then the memories of the two side-by-side layers
                st, dst = spans["matrix_state"], dspans["matrix_state"]
                att, datt = spans["attention_options"], dspans["attention_options"]
                # a prompt's recurrence reads q, k, v, the gate (float32) and two scalars a head, and writes a row;
                # a decoding step reads and writes every request's state
                delta_rows = prompt_len * ((2 * dg * dd + 2 * dh * dv + 2 * dh) * 4 + dh * dv * 2.0)
                mem_rows = prompt_len * ((2 * mh * md + 2 * mh * mv + 2 * mh) * 4 + mh * mv * 2.0)
                # the feed-forwards: a prompt's useful flops; a decoding step's weight bytes (experts: those that are hit)
                ffn = {"prompt": spans["glu_ffn"][0], "decode": dspans["glu_ffn"][0]}      # the first layer's dense one
                a["roofline_frac"] = {
                    "prompt_attention": frac(4.0 * h * d * seen_all, att[0], tc),
                    "decode_attention": frac(batch * kvh * context * 2 * d * 2.0, datt[0], hbm),
                    "prompt_delta_rule_bytes": frac(delta_rows, st[0], hbm),
                    "prompt_matrix_memory_bytes": frac(mem_rows, st[1], hbm),
                    # per state element and token: the delta rule 3 multiply-adds and a product, the memory 2 and a product
                    "prompt_delta_rule_fp32": frac(prompt_len * dh * dd * dv * 7.0, st[0], fp32),
                    "prompt_matrix_memory_fp32": frac(prompt_len * mh * md * (mv + 1) * 5.0, st[1], fp32),
                    "decode_delta_rule_state_bytes": frac(batch * dh * dd * dv * 8.0, dst[0], hbm),
                    "decode_matrix_memory_state_bytes": frac(batch * mh * md * (mv + 1) * 8.0, dst[1], hbm),
                    "prompt_dense_ffn": frac(2.0 * prompt_len * 3 * w * ff, ffn["prompt"], tc),
                    "decode_dense_ffn": frac(2.0 * 3 * w * ff, ffn["decode"], hbm),
                    "prompt_experts": frac(2.0 * prompt_len * top * 3 * w * eff, spans["routed_experts"][0], tc),
                    "decode_experts": frac(2.0 * 3 * w * eff * min(experts, batch * top), dspans["routed_experts"][0], hbm)}
            else:
                att, datt = spans["attention_options"], dspans["attention_options"]
                rd = 64
                # the first layer's feed-forward: the product with the activation, and the first product back to the width
                ffn = {n: sp["linear_xielu"][0] + next(ms_ for ms_, (shape, acc) in zip(sp["linear"], sp["_linear_kinds"])
                                                       if shape == (w, ff))
                       for n, sp in (("prompt", spans), ("decode", dspans))}
                a["roofline_frac"] = {
                    "prompt_attention": frac(4.0 * h * d * seen_all, att[0], tc),
                    "decode_attention": frac(batch * kvh * context * 2 * d * 2.0, datt[0], hbm),
                    "prompt_recurrence_bytes": frac(prompt_len * w * (5 * 4 + 2.0), spans["wkv_recurrence"][0], hbm),
                    # per state element and token: 3 multiply-adds
                    "prompt_recurrence_fp32": frac(prompt_len * (w // rd) * rd * rd * 6.0, spans["wkv_recurrence"][0], fp32),
                    "decode_recurrence_state_bytes": frac(batch * (w // rd) * rd * rd * 8.0, dspans["wkv_recurrence"][0], hbm),
                    "prompt_dense_ffn": frac(2.0 * prompt_len * 2 * w * ff, ffn["prompt"], tc),
                    "decode_dense_ffn": frac(2.0 * 2 * w * ff, ffn["decode"], hbm)}
            res[arm] = a
            del engine
            torch.cuda.empty_cache()
        out["sizes"][key] = {"width": w, "heads": h, "kv_heads": kvh, "head_dim": d, "delta": [dh, dg, dd, dv],
                             "memory": [mh, md, mv], "ff": ff, "experts": experts, "top": top, "expert_ff": eff,
                             "shared_ff": sff, "layers": 3 * blocks, **res}
    print(json.dumps(out))
    return 0


def reference_binary():
    """The reference's command-line program, built with its own CMakeLists if it is not there yet.
    Returns (path, None) or (None, why not)."""
    exe = os.path.join(REF_DIR, "build", "tinyinfer")
    if os.path.isfile(exe) and os.access(exe, os.X_OK):
        return exe, None
    src = os.path.join(REF_DIR, "src")
    if not os.path.isfile(os.path.join(src, "CMakeLists.txt")):
        return None, ("beyondHJM/tinyinfer.cpp is a CMake C++/CUDA project (pip: \"Neither 'setup.py' nor "
                      "'pyproject.toml' found\") and no copy of its tree lies under baseline/_ref/src to build")
    try:
        log = os.path.join(REF_DIR, "build.log")
        with open(log, "w") as fh:
            subprocess.run(["cmake", "-S", src, "-B", os.path.join(REF_DIR, "build"),
                            "-DCMAKE_CUDA_ARCHITECTURES=100", "-DCMAKE_BUILD_TYPE=Release"],
                           stdout=fh, stderr=subprocess.STDOUT, check=True, timeout=600)
            subprocess.run(["cmake", "--build", os.path.join(REF_DIR, "build"), "--target", "tinyinfer", "-j", "8"],
                           stdout=fh, stderr=subprocess.STDOUT, check=True, timeout=1200)
    except (OSError, subprocess.SubprocessError) as exc:
        return None, f"building the reference with its own CMakeLists failed ({type(exc).__name__}; baseline/_ref/build.log)"
    return (exe, None) if os.path.isfile(exe) else (None, "the reference's build left no program")


def reference_gguf(cfg, seed, path):
    """A GGUF file of the configuration with seeded random weights and a tokenizer of single
    letters (so that a prompt of three letters is three tokens); end-of-text is an id no token has."""
    import torch
    from tinyinfer_b200.config import Qwen3Config
    from tinyinfer_b200.config.qwen3 import gguf_metadata, gguf_tensor_name
    from tinyinfer_b200.config.registry import architecture_of
    from tinyinfer_b200.parts.model import CausalLM
    from tinyinfer_b200.weights import write_gguf
    from tinyinfer_b200.weights.random_init import random_tensor
    arch = architecture_of(cfg)
    typed = arch.from_dict(cfg)
    model = CausalLM(arch.build_plan(typed))
    # drawn on the GPU when there is one (the generator gives the same bits there, much sooner)
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    tensors = {gguf_tensor_name(n): random_tensor(seed, n, spec, device=dev).cpu()
               for n, spec in model.expected_tensors().items()}
    meta = gguf_metadata(Qwen3Config.from_dict(cfg))
    letters = [chr(ord("a") + i) for i in range(26)]
    meta["tokenizer.ggml.tokens"] = letters
    meta["tokenizer.ggml.token_type"] = [1] * len(letters)
    meta["tokenizer.ggml.eos_token_id"] = 2 ** 32 - 1
    write_gguf(path, meta, tensors)


def reference_decode(exe, gguf, batch, context, cuda_graph=True):
    """Runs the reference's program: `batch` prompts of three tokens, decoded to `context`.
    Returns (tokens a second as it reports them, generated tokens, decode ms, the tail of its log)."""
    import re
    # its loop ends when all sequences together have made batch + n tokens (src/main.cpp:276)
    n_predict = batch * (context - 4)
    cmd = [exe, "-m", gguf, "-n", str(n_predict), "--max-seq", str(context)]
    for i in range(batch):
        cmd += ["-p", "abc"]
    if cuda_graph:
        cmd.append("--cuda-graph")
    proc = subprocess.run(cmd, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE, text=True, timeout=900)
    tail = proc.stderr[-600:]
    m = re.search(r"main: decode: ([0-9.]+) ms, (\d+) tokens, ([0-9.]+) tok/s", proc.stderr)
    if proc.returncode != 0 or not m:
        raise RuntimeError(f"the reference's program ended with {proc.returncode}: {tail.strip()[-300:]}")
    return float(m.group(3)), int(m.group(2)), float(m.group(1)), tail


def reference_arm(args) -> int:
    shape_name, shape_cfg = SHAPES[args.shape]
    cfg = dict(shape_cfg)
    cfg["max_position_embeddings"] = max(args.context, 2048)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    if not cfg["tie_word_embeddings"]:
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference always ties the head to the embedding (src/inference.cu:70-71); "
                          f"the {shape_name} has a head of its own"}))
        return 0
    if args.batch > 16:
        print(json.dumps({"impl": "reference", "unavailable": "the reference runs at most 16 sequences (src/main.cpp:178)"}))
        return 0
    exe, why = reference_binary()
    if exe is None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    import tempfile
    gguf = os.path.join(tempfile.gettempdir(), f"tinyinfer_ref_{args.shape}_{cfg['num_hidden_layers']}l_{os.getuid()}.gguf")
    try:
        if not os.path.isfile(gguf):
            reference_gguf(cfg, 0, gguf)
        with ClockSampler() as clocks:
            tps, generated, decode_ms, tail = reference_decode(exe, gguf, args.batch, args.context)
        points = {}
        if not args.no_points and args.batch != 1:
            points["decode_b1"] = reference_decode(exe, gguf, 1, args.context)[0]
    except Exception as exc:           # the line must still come out
        print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}))
        return 0
    steps = generated // args.batch
    nums = model_numbers(cfg)
    pk, pk_kind = peaks()
    ctx_mean = args.context // 2
    step_bytes = nums["weight_bytes"] + args.batch * ctx_mean * nums["kv_bytes_per_token"]
    ms_per_step = decode_ms / max(steps, 1)
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    line = {
        "impl": "reference",
        "metric": f"decode tok/s at batch {args.batch}, context {args.context} ({shape_name})",
        "value": tps, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": 0,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights in a GGUF file, prompts of three tokens, greedy decoding",
        "config": {
            "model": shape_name, "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "tied": True, "global_batch": args.batch, "seq_len": args.context,
            "measured_over": "the whole decode, context 3 to seq_len (its own report)",
            "cuda_graph": True, "program": "baseline/_ref/build/tinyinfer (its own CMakeLists, sm_100)",
            "parallelism": "single GPU", "peaks": pk_kind,
        },
        "clocks": clocks.summary(),
        "e2e": {"value": tps, "unit": "tokens/s", "note": "the same run: its command line is its public API"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "at": "mean context seq_len / 2"},
        "prefill": None,
        "points": points,
    }
    print(json.dumps(line))
    return 0



# ---- the Nekorax decoder beside the Ruvuvik decoder at equal sizes ------------------------------
# (width, heads, kv heads, head size, latent rank, query latent rank, rotated part, window of the latent layers,
#  taps, experts, identity experts, top, expert ff, groups (count, keep), blocks of [latent attention, attention]
#  layers; the first block is walked twice)
NEKORAX_SIZES = {
    "w1024": (1024, 16, 4, 64, 256, 384, 32, 4096, 4, 12, 4, 4, 704, (4, 2), 2),
    "w2048": (2048, 16, 4, 128, 512, 768, 64, 4096, 4, 24, 8, 4, 1408, (4, 2), 2),
    "w4096": (4096, 32, 8, 128, 512, 1536, 64, 4096, 4, 48, 16, 4, 1408, (8, 4), 1),
}


def nekorax_config(size):
    w, h, g, d, rank, q_rank, dr, window, taps, experts, identity, top, eff, groups, blocks = size
    mlp = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top,
                                     "groups": {"count": groups[0], "keep": groups[1]}},
           "expert": {"ff": eff, "limit": 7.0}}
    layers = [
        {"type": "latent_attention", "mlp": mlp,
         "mixer": {"heads": h, "dim": d, "rot_dim": dr, "vdim": d, "kv_rank": rank, "q_rank": q_rank,
                   "mask": {"size": window}, "scale": (d + dr) ** -0.5,
                   "rot": {"dims": dr, "base": 10000.0,
                           "scaling": {"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0}}}},
        {"type": "attention", "mlp": mlp,
         "mixer": {"heads": h, "kv_heads": g, "dim": d, "vdim": d, "conv": taps,
                   "rot": {"dims": d // 2, "base": 250000.0}, "scale": d ** -0.5}}]
    return {"architecture": "Nekorax", "vocab": DESIGN_VOCAB, "width": w, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "logit_softcap": 30.0, "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": layers * blocks}


def ruvuvik_beside_nekorax(size, context):
    """As many layers as the Nekorax decoder has layer runs, attention and latent attention in turn (no chunk
    edge inside the context), and a dense feed-forward with as many multiply-adds a token as the chosen experts."""
    w, h, g, d, rank, q_rank, dr, window, taps, experts, identity, top, eff, groups, blocks = size
    mlp = {"kind": "dense", "ff": top * eff * 3 // 2 // 64 * 64}
    layers = [
        {"type": "latent_attention", "mlp": mlp,
         "mixer": {"heads": h, "dim": d, "rot_dim": dr, "vdim": d, "kv_rank": rank,
                   "rot": {"dims": dr, "base": 100000.0}, "scale": (d + dr) ** -0.5}},
        {"type": "attention", "mlp": mlp,
         "mixer": {"heads": h, "kv_heads": g, "dim": d, "vdim": d, "mask": {"size": context},
                   "rot": {"dims": d, "base": 10000.0}, "scale": d ** -0.5, "softcap": 50.0}}]
    return {"architecture": "Ruvuvik", "vocab": DESIGN_VOCAB, "width": w, "norm": {"eps": 1e-5},
            "layers": layers * (blocks + 1)}


def nekorax_arm(args) -> int:
    """Prefill and decode throughput of the Nekorax decoder at sizes of real layers, beside the Ruvuvik
    decoder (the closest design the engine has: the same two attention kernels) with as many layers as
    Nekorax has layer runs, of the same width, heads, head size and latent rank, and the time the device
    spends in every kind of kernel call per layer run, with the fraction of the roofline for the calls
    that have one."""
    import torch
    from tinyinfer_b200 import Engine, StepEntry
    pk, pk_kind = peaks()
    prompt_len, batch, context = args.prefill_tokens, args.batch, args.context
    warmup = max(args.warmup, 3)
    out = {"design": "nekorax", "beside": "ruvuvik at equal sizes", "peaks": pk_kind, "prefill_tokens": prompt_len,
           "decode_batch": batch, "decode_context": context, "dtype": "bf16", "data": "synthetic", "sizes": {}}
    gen = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, DESIGN_VOCAB, (prompt_len,), generator=gen).tolist()
    hbm, tc = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    for key, size in NEKORAX_SIZES.items():
        if args.design_size and key != args.design_size:
            continue
        w, h, kvh, d, rank, q_rank, dr, window, taps, experts, identity, top, eff, groups, blocks = size
        runs = 2 * (blocks + 1)
        res = {}
        calls = {"nekorax": ["attention_options", "qkv_turn_store", "turn_rows", "latent_prepare", "head_project",
                             "causal_conv", "conv_tail_store", "tanh_norm", "tanh_norm_pair", "router_choose", "routed_experts", "add_row",
                             "cap_rows", "slice_rmsnorm", "linear"],
                 "ruvuvik": ["attention_options", "qk_rownorm_rope_store", "latent_prepare", "head_project",
                             "linear_xielu", "xielu_rows", "linear", "rmsnorm"]}
        for arm, cfg in (("nekorax", nekorax_config(size)),
                         ("ruvuvik", ruvuvik_beside_nekorax(size, max(context, prompt_len) + 64))):
            engine = Engine(config=cfg, seed=0, dtype="bfloat16", page_size=args.page_size,
                            num_pages=-(-max(batch * context, prompt_len) // args.page_size) + batch + 2,
                            max_requests=batch + 1, step_graphs=True)
            if arm == "nekorax":
                # seeded weights are small: every token's scores would be nearly equal and the seeded correction alone
                # would send all tokens to the same experts.  Larger router rows and no correction make the choice
                # differ from token to token.
                for block in engine.model.blocks:
                    block.ffn.w_router.mul_(6.0)
                    block.ffn.correction.zero_()
            pf_ms = measure_prefill(engine, prompt_len, max(1, min(args.steps, 6)), torch)
            ms, clocks, launches = measure_decode(engine, batch, context, args.steps, warmup, torch)
            a = {"prefill_tok_s": round(prompt_len / pf_ms * 1e3), "prefill_ms": round(pf_ms, 3),
                 "decode_tok_s": round(batch / ms * 1e3, 1), "decode_ms_per_step": round(ms, 4),
                 "decode_launches_per_step": launches // max(1, args.steps), "clocks": clocks}
            engine._step_graphs = None
            engine.ops.fuse_decode_tail = engine.ops.fuse_decode_ffn = False   # every call of its own
            names = calls[arm]
            for _ in range(2):        # the first eager step sizes the allocator's pool; the second is read
                spans = timed_ops(engine, names, lambda: engine.step([StepEntry("p", prompt, [prompt_len - 1])]), torch)
                engine.finish("p")
            ids = fill_requests(engine, batch, context - 4, torch)
            for _ in range(2):
                # a token of its own for every request, so that the routers' choices differ between them
                dspans = timed_ops(engine, names, lambda: engine.step([StepEntry(r, [1 + 37 * i], [0]) for i, r in enumerate(ids)]), torch)
            chosen = {"prompt": [], "decode": []}
            if arm == "nekorax":
                # which experts the first feed-forward's router chose, in a prompt and in a decoding step: the
                # pairs that have tensors (the rest are identity experts) and how many different experts they hit
                inner = engine.ops.routed_experts

                def noting(h_, w_, ids_, *rest, **kw):
                    chosen[phase].append(ids_.clone())
                    return inner(h_, w_, ids_, *rest, **kw)

                engine.ops.routed_experts = noting
                phase = "decode"
                engine.step([StepEntry(r, [1 + 37 * i], [0]) for i, r in enumerate(ids)])
            for r in ids:
                engine.finish(r)
            if arm == "nekorax":
                phase = "prompt"
                engine.step([StepEntry("p", prompt, [prompt_len - 1])])
                engine.finish("p")
                del engine.ops.routed_experts
            a["calls_us"] = {
                "prompt": {n: [round(x * 1e3, 1) for x in v[:12]] for n, v in spans.items() if not n.startswith("_") and n != "linear"},
                "decode": {n: [round(x * 1e3, 1) for x in v[:12]] for n, v in dspans.items() if not n.startswith("_") and n != "linear"}}
            a["per_layer_us"] = {
                "prompt": {n: round(sum(v) / runs * 1e3, 1) for n, v in spans.items() if not n.startswith("_")},
                "decode": {n: round(sum(v) / runs * 1e3, 1) for n, v in dspans.items() if not n.startswith("_")}}
            seen_all = prompt_len * (prompt_len + 1) / 2
            row = rank + dr

            def frac(amount, ms_, peak):
                return round(amount / (ms_ * 1e-3) / peak, 4)

            # calls in layer order: the latent layer first, then the attention layer
            att, datt = spans["attention_options"], dspans["attention_options"]
            if arm == "nekorax":
                seen_window = sum(min(i + 1, window) for i in range(prompt_len))
                first = {k: v[0][v[0] < experts] for k, v in chosen.items()}
                real_pairs, hit = int(first["prompt"].numel()), int(first["decode"].unique().numel())
                a["first_router"] = {"prompt_pairs_with_tensors": real_pairs, "of": prompt_len * top,
                                     "decode_experts_hit": hit, "decode_pairs_with_tensors": int(first["decode"].numel())}
                cols = (h + 2 * kvh) * d
                a["roofline_frac"] = {
                    "prompt_latent_attention": frac(2.0 * h * (row + rank) * seen_window, att[0], tc),
                    "prompt_attention": frac(4.0 * h * d * seen_all, att[1], tc),
                    "decode_latent_attention": frac(batch * min(context, window) * row * 2.0, datt[0], hbm),
                    "decode_attention": frac(batch * kvh * context * 2 * d * 2.0, datt[1], hbm),
                    "prompt_experts": frac(2.0 * real_pairs * 3 * w * eff, spans["routed_experts"][0], tc),
                    "decode_experts": frac(2.0 * 3 * w * eff * hit, dspans["routed_experts"][0], hbm),
                    # the row kernels, by the bytes they must move: float32 rows in, rows of the activation dtype or
                    # float32 rows out
                    "prompt_norm_by_tanh": frac(prompt_len * w * (4 + 2.0), spans["tanh_norm"][0], hbm),
                    "prompt_norm_pair": frac(prompt_len * w * (4 + 4 + 4 + 2.0), spans["tanh_norm_pair"][0], hbm),
                    "prompt_convolution": frac(prompt_len * cols * 8.0, spans["causal_conv"][2], hbm),      # behind the junction's two conversions
                    "prompt_turn_and_store": frac(prompt_len * cols * (4 + 2.0), spans["qkv_turn_store"][0], hbm),
                    "prompt_turn_back_and_gate": frac(prompt_len * h * d * (2 + 4 + 2.0), spans["turn_rows"][0], hbm)}
            else:
                ffn = {n: sp["linear_xielu"][0] for n, sp in (("prompt", spans), ("decode", dspans))}
                a["roofline_frac"] = {
                    "prompt_latent_attention": frac(2.0 * h * (row + rank) * seen_all, att[0], tc),
                    "prompt_attention": frac(4.0 * h * d * seen_all, att[1], tc),
                    "decode_latent_attention": frac(batch * context * row * 2.0, datt[0], hbm),
                    "decode_attention": frac(batch * kvh * context * 2 * d * 2.0, datt[1], hbm),
                    "prompt_ffn_first_product": frac(2.0 * prompt_len * w * (top * eff * 3 // 2 // 64 * 64), ffn["prompt"], tc),
                    "decode_ffn_first_product": frac(2.0 * w * (top * eff * 3 // 2 // 64 * 64), ffn["decode"], hbm),
                    "prompt_norm": frac(prompt_len * w * (4 + 2.0), spans["rmsnorm"][0], hbm),
                    "prompt_norm_turn_and_store": frac(prompt_len * (h + 2 * kvh) * d * (4 + 2.0), spans["qk_rownorm_rope_store"][0], hbm)}
            res[arm] = a
            del engine
            torch.cuda.empty_cache()
        out["sizes"][key] = {"width": w, "heads": h, "kv_heads": kvh, "head_dim": d, "kv_rank": rank, "q_rank": q_rank,
                             "rot_dim": dr, "window": window, "taps": taps, "experts": experts, "identity": identity,
                             "top": top, "expert_ff": eff, "groups": list(groups), "layer_runs": runs, **res}
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers (named in config)")
    ap.add_argument("--shape", choices=list(SHAPES), default="0.6b", help="layer sizes of the model")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64 and the other shapes")
    ap.add_argument("--no-shapes", action="store_true", help="skip the 8B and 32B shapes and the page-16 run")
    ap.add_argument("--page-size", type=int, default=PAGE, help="tokens per cache page")
    ap.add_argument("--prefill-tokens", type=int, default=2048,
                    help="with --only prefill: the length of the prompt (the default run's is 2,048)")
    ap.add_argument("--mixed-decoders", type=int, default=63,
                    help="with --only mixed: the number of decoding requests beside the 512-token portion")
    ap.add_argument("--attention-in-turn", action="store_true",
                    help="with --only mixed: flash-decoding behind the prompt attention kernel, not beside it")
    ap.add_argument("--design", choices=["kagorax", "ruvuvik", "feruzen", "nekorax"], default=None,
                    help="set this decoder beside the closest one the engine has (Qwen3; for feruzen and nekorax: Ruvuvik) at equal sizes instead of the default run")
    ap.add_argument("--design-size", choices=sorted(set(DESIGN_SIZES) | set(RUVUVIK_SIZES) | set(FERUZEN_SIZES) | set(NEKORAX_SIZES)), default=None,
                    help="one of the sizes only")
    ap.add_argument("--only", choices=["decode", "prefill", "chains", "mixed"], default=None,
                    help="run one part only and print a short line (for profiling small cases)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU; this engine does no work on several (asked for {args.gpus})")
        return 2
    warmup = max(args.warmup, 3)
    if args.design == "ruvuvik":
        return ruvuvik_arm(args)
    if args.design == "feruzen":
        return feruzen_arm(args)
    if args.design == "nekorax":
        return nekorax_arm(args)
    if args.design:
        return design_arm(args)

    import torch
    from tinyinfer_b200 import LLM

    shape_name, shape_cfg = SHAPES[args.shape]
    cfg = dict(shape_cfg)
    cfg["max_position_embeddings"] = max(args.context, MAX_POSITION)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk, pk_kind = peaks()
    nums = model_numbers(cfg)
    max_batch = max(args.batch, 1 if (args.no_points or args.only not in (None, "mixed")) else 64)
    longest = max(args.context, args.prefill_tokens + args.page_size if args.only == "prefill" else 0)
    llm = LLM(config=cfg, seed=0, dtype="bfloat16", page_size=args.page_size, max_seq=longest,
              max_num_seqs=max_batch + 1, kv_tokens=max(max_batch * args.context, longest), cuda_graph=True)
    engine = llm.engine

    if args.only == "decode":
        ms, _, launches = measure_decode(engine, args.batch, args.context, args.steps, warmup, torch)
        print(json.dumps({"only": "decode", "batch": args.batch, "context": args.context,
                          "ms_per_step": round(ms, 4), "gpu_launches": launches}))
        return 0
    if args.only == "chains":
        print(json.dumps({"only": "chains", "batch": args.batch, "us_per_launch":
                          measure_chains(engine, args.batch, torch)}))
        return 0
    if args.only == "mixed":
        engine.ops.attention_side_by_side = not args.attention_in_turn
        mx_ms = measure_mixed(engine, args.mixed_decoders, 512, args.context, torch)
        print(json.dumps({"only": "mixed", "decoding": args.mixed_decoders, "portion": 512, "ms": round(mx_ms, 3),
                          "attention": "in turn" if args.attention_in_turn else "side by side"}))
        return 0
    if args.only == "prefill":
        pf_ms = measure_prefill(engine, args.prefill_tokens, max(1, min(args.steps, 8)), torch)
        print(json.dumps({"only": "prefill", "tokens": args.prefill_tokens, "ms": round(pf_ms, 3)}))
        return 0
    ms, clocks, launches = measure_decode(engine, args.batch, args.context, args.steps, warmup, torch)
    e2e_ms, h2d, d2h = decode_e2e(llm, args.batch, args.context, args.steps, warmup, torch)
    ctx_mid = args.context - args.steps // 2
    step_bytes = nums["weight_bytes"] + args.batch * ctx_mid * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9

    points, fracs = {}, {}
    if not args.no_points:
        for b in (1, 64):
            n = min(args.steps, 32)
            pms, _, _ = measure_decode(engine, b, args.context, n, warmup, torch)
            points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
            b_bytes = nums["weight_bytes"] + b * (args.context - n // 2) * nums["kv_bytes_per_token"]
            fracs[f"decode_b{b}"] = round(b_bytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        eager_ms = decode_eager_timed(engine, args.batch, args.context, min(args.steps, 32), warmup, torch)
        points[f"decode_b{args.batch}_no_graph"] = round(args.batch / (eager_ms * 1e-3), 1)
        # chunked prefill under load: 63 requests decode beside a 512-token portion of a prompt
        mx_ms = measure_mixed(engine, 63, 512, args.context, torch)
        points["mixed_63_decoding_512_portion"] = round((63 + 512) / (mx_ms * 1e-3), 1)

    pf_tokens = 2048
    pf_ms = measure_prefill(engine, pf_tokens, 3, torch)
    pf_peak, pf_which = flops_peak(pk, pf_ms)
    pf_frac = prefill_flops(cfg, pf_tokens) / (pf_ms * 1e-3) / (pf_peak * 1e12)

    if not args.no_points and not args.no_shapes and args.shape == "0.6b" and not args.layers:
        # the page size and the two larger shapes that the baseline names, as points of their own
        import gc
        del engine, llm
        gc.collect()
        torch.cuda.empty_cache()
        for key, page, batches, pre, mix, prefix in (
                ("0.6b", 16, (8,), True, False, "page16_"),
                ("8b", args.page_size, (1, 8, 64), True, True, "8b_"),
                ("32b", args.page_size, (1, 8, 64), True, False, "32b_")):
            try:
                p2, f2 = shape_points(key, page, args.context, args.steps, warmup, batches, pre, mix, pk, torch, prefix)
            except Exception as exc:                    # a point that fails must not lose the line
                p2, f2 = {f"{prefix}error": f"{type(exc).__name__}: {str(exc)[:120]}"}, {}
            points.update(p2)
            fracs.update(f2)

    value = args.batch / (ms * 1e-3)
    line = {
        "metric": f"decode tok/s at batch {args.batch}, context {args.context} ({shape_name})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights, random token ids, random keys and values",
        "config": {
            "model": shape_name, "layers": cfg["num_hidden_layers"],
            "layers_full": full_layers, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "tied": cfg["tie_word_embeddings"], "global_batch": args.batch,
            "seq_len": args.context, "page_size": args.page_size, "max_position": cfg["max_position_embeddings"],
            "parallelism": "single GPU", "cuda_graph": True, "l2": "working set > L2, no flush", "peaks": pk_kind,
        },
        "clocks": clocks,
        "e2e": {"value": round(args.batch / (e2e_ms * 1e-3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(pf_tokens / (pf_ms * 1e-3), 1), "tokens": pf_tokens,
                    "ms": round(pf_ms, 3), "frac": round(pf_frac, 4), "peak": pf_which},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "points_frac": fracs,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
