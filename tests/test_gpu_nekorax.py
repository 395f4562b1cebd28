"""Nekorax on the GPU against the plain implementation: every kernel alone, each mixer alone over
requests cut into portions (also with inputs made so that one key, or the unit in the softmax's
denominator, carries the answer), whole prompts, the same requests cut in different ways, long
decoding, reused pages and state slots, and greedy generation through the entry point.

float32 is the sharp comparison: a mechanism alone agrees to 2e-5 of its largest output, the whole
model to 6e-5 of the largest logit.  In bfloat16 a mechanism alone agrees to 3e-2; in the whole model
an expert chosen differently moves a row, so the bound is 3e-2 for half the rows and 0.12 for nine
out of ten."""
import copy
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import plain_nekorax as plain
import traces
from nekorax_util import SMALL, attention, latent, make_model, mixer_weights, mlp_weights, moe
from test_gpu_feruzen import MODEL_RTOL, _compare, _run, _run_mixer
from test_gpu_ruvuvik import _fill, _paged
from util import assert_close_logits, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
LENGTHS = {"A": [70, 45, 120, 33, 17, 2, 64, 1], "B": [40, 9, 130, 1], "C": [300, 33, 150, 64, 217, 17], "D": [50, 3]}


@pytest.fixture(scope="module")
def ops():
    from tinyinfer_b200.kernels import cuda_ops
    return cuda_ops(DEV)


def _requests(name):
    vocab = SMALL[name]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, seed=700 + i) for i, n in enumerate(LENGTHS[name])}


_PLAIN = {}


def _plain(model_dir, name):
    if name not in _PLAIN:
        cfg, w = plain.load_folder(model_dir)
        _PLAIN[name] = {r: plain.forward(cfg, w, t) for r, t in _requests(name).items()}
    return _PLAIN[name]


def _close(got, want, dtype, what):
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    err = (got.double().cpu() - want).abs().max() / want.abs().max()
    assert err < tol, f"{what}: off by {float(err):.3g} of the largest value"


# ---- kernels alone ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(5, 48), (1, 36), (70, 256), (3, 2049)])
def test_norm_by_tanh(ops, sizes, dtype):
    t, n = sizes
    g = torch.Generator().manual_seed(n)
    x = torch.randn((t, n), generator=g) * 3
    w = {"n": 1 + 0.3 * torch.randn((n,), generator=g), "n.b": 0.2 * torch.randn((n,), generator=g),
         "n.alpha": torch.tensor(0.37)}
    want = plain.dyt(x.double(), {k: v.double() for k, v in w.items()}, "n")
    xd, wd, bd = x.to(DEV), w["n"].to(DEV), w["n.b"].to(DEV)
    out = torch.empty((t, n), dtype=dtype, device=DEV)
    ops.tanh_norm(xd, 0.37, wd, bd, out=out)
    _close(out, want, dtype, "rows")
    rows = torch.tensor([t - 1, 0], dtype=torch.int32, device=DEV)
    some = torch.empty((2, n), dtype=dtype, device=DEV)
    ops.tanh_norm(xd, 0.37, wd, bd, out=some, rows=rows)
    assert torch.equal(some, out[[t - 1, 0]])
    residual = torch.randn((t, n), generator=g).to(DEV)
    before = residual.clone()
    ops.tanh_norm(xd, 0.37, wd, bd, residual=residual)
    _close(residual - before, want, torch.float32, "added to a residual")
    ops.tanh_norm(xd, 0.37, wd, None, out=out)
    _close(out, want - w["n.b"].double(), dtype, "without a bias")
    # the norm behind a sublayer and the norm in front of the next in one launch: the same bits
    w2, b2 = (1 + 0.3 * torch.randn((n,), generator=g)).to(DEV), (0.2 * torch.randn((n,), generator=g)).to(DEV)
    first, second = before.clone(), before.clone()
    ops.tanh_norm(xd, 0.37, wd, bd, residual=first)
    ops.tanh_norm(first, 1.4, w2, b2, out=out)
    both = torch.empty_like(out)
    ops.tanh_norm_pair(xd, 0.37, wd, bd, second, 1.4, w2, b2, both)
    assert torch.equal(first, second) and torch.equal(out, both)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_of_a_column_slice(ops, dtype):
    g = torch.Generator().manual_seed(4)
    wide = torch.randn((37, 150), generator=g) * 2
    w = 1 + 0.3 * torch.randn((40,), generator=g)
    for lo, weight in ((0, w), (64, w), (110, None)):
        x = wide[:, lo:lo + 40]
        want = plain.unit_rms(x.double(), 1e-5) * (1.0 if weight is None else weight.double())
        out = torch.empty((37, 40), dtype=dtype, device=DEV)
        ops.slice_rmsnorm(wide.to(DEV)[:, lo:lo + 40], None if weight is None else weight.to(DEV), 1e-5, out)
        _close(out, want, dtype, f"columns from {lo}")


def test_cap_and_added_row(ops):
    g = torch.Generator().manual_seed(1)
    x = torch.randn((7, 131), generator=g) * 20
    d = x.to(DEV)
    ops.cap_rows(d, 9.0)
    _close(d, 9.0 * torch.tanh(x.double() / 9.0), torch.float32, "cap")
    wide = torch.randn((5, 40), generator=g).to(DEV)
    view, row = wide[:, 8:32], torch.randn((24,), generator=g)
    want = wide.cpu().double()
    want[:, 8:32] += row.double()
    ops.add_row(view, row.to(DEV))
    _close(wide, want, torch.float32, "row added to a column slice")


@pytest.mark.parametrize("case", [(6, 2, None, None), (12, 3, (2, 1), 0.05), (12, 3, (3, 2), 0.05), (9, 9, (3, 3), 0.1),
                                  (40, 6, (8, 3), 0.02), (5, 1, (5, 1), 0.3), (300, 8, (10, 4), 0.01), (1, 1, (1, 1), 0.0)])
def test_router_choice(ops, case):
    total, top, groups, corr = case
    g = torch.Generator().manual_seed(total * 7 + top)
    t = 133
    z = torch.randn((t, total + 3), generator=g) * 2.5
    z[5] = 0.0                                            # all scores equal: the correction alone decides
    z[6, :total] = z[6, 0]
    correction = None if corr is None else torch.randn((total,), generator=g) * corr
    ids = torch.empty((t, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((t, top), dtype=torch.float32, device=DEV)
    ops.router_choose(z.to(DEV), total, top, ids, weights, None if correction is None else correction.to(DEV),
                      *(groups or (1, 1)))
    r = {"top": top, "groups": None if groups is None else {"count": groups[0], "keep": groups[1]}}
    # the float32 scores decide; the plain choice is made from them in float64
    s = torch.softmax(z[:, :total].to(DEV), dim=-1).cpu().double()
    zero = torch.zeros((total,), dtype=F64) if correction is None else correction.double()
    for i in range(t):
        want = plain.route(torch.log(s[i]), zero, r)
        gaps = sorted(float(x) for x in (s[i] + zero))
        if min((b - a for a, b in zip(gaps, gaps[1:])), default=1.0) < 1e-6 and i not in (5, 6):
            continue                                      # a close call between two outputs
        assert ids[i].tolist() == [e for e, _ in want], f"row {i}"
        assert torch.allclose(weights[i].cpu().double(), torch.stack([x for _, x in want]), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("geom", [(4, 2, 12, 8, 6, 8, "neox"), (1, 1, 16, 16, 16, 16, "neox"), (6, 3, 10, 24, 0, 16, "neox"),
                                  (8, 1, 80, 64, 40, 16, "neox"), (2, 2, 8, 6, 4, 8, "interleaved")])
def test_turned_heads_values_and_the_way_back(ops, geom, dtype):
    from tinyinfer_b200.parts.rope import NoPosition, RopeInterleaved, RopeNeox
    heads, kv, dk, dv, rot, ps, kind = geom
    ctx, ql = [37, 5, 300], [9, 5, 1]
    step, cache, bt, positions, req = _paged(ctx, ql, ps, kv * (dk + dv), dtype)
    g = torch.Generator().manual_seed(3)
    t = len(positions)
    nq, nk, nv = heads * dk, kv * dk, kv * dv
    proj = torch.randn((t, nq + nk + nv + 5), generator=g)
    cls = RopeNeox if kind == "neox" else RopeInterleaved
    layout = "halves" if kind == "neox" else "pairs"
    rotation = (cls(dk, 777.0, rot) if rot else NoPosition()).rotation(DEV)
    v_rotation = cls(dv, 777.0).rotation(DEV)
    q_out = torch.empty((t, nq), dtype=dtype, device=DEV)
    ops.qkv_turn_store(proj.to(DEV), rotation, v_rotation, step, cache, q_out, heads, kv, dk, dv)
    pos = torch.tensor(positions)
    p64 = proj.double()
    fq, fv = plain.frequencies(777.0, rot) if rot else None, plain.frequencies(777.0, dv)
    want_q = p64[:, :nq].reshape(t, heads, dk)
    want_k = p64[:, nq:nq + nk].reshape(t, kv, dk)
    if rot:
        want_q, want_k = plain.turn(want_q, pos, fq, rot, layout), plain.turn(want_k, pos, fq, rot, layout)
    want_v = plain.turn(p64[:, nq + nk:nq + nk + nv].reshape(t, kv, dv), pos, fv, dv, layout)
    _close(q_out.view(t, heads, dk), want_q, dtype, "queries")
    for i in range(t):
        page = cache.pages[int(bt[req[i], positions[i] // ps])]
        slot = positions[i] % ps
        _close(page[: kv * ps * dk].view(kv, ps, dk)[:, slot], want_k[i], dtype, f"key of token {i}")
        _close(page[kv * ps * dk:].view(kv, ps, dv)[:, slot], want_v[i], dtype, f"value of token {i}")
    # the way back, with a gate: rows of heads * dv turned by minus the position
    rows = torch.randn((t, heads * dv), generator=g)
    gate = torch.randn((t, heads * dv + 3), generator=g)
    want = plain.turn(rows.to(dtype).double().reshape(t, heads, dv), -pos, fv, dv, layout).reshape(t, -1) \
        * torch.sigmoid(gate[:, :heads * dv].double())
    d = rows.to(dtype).to(DEV)
    ops.turn_rows(d, step, v_rotation, heads, dv, back=True, gate=gate.to(DEV)[:, :heads * dv])
    _close(d, want, dtype, "turned back in place")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [False, True])
def test_one_more_unit_in_the_denominator(ops, decoded, dtype):
    """One visible key whose score is 0 shares the weight with the unit: half its value comes out.  A
    key with a large score takes nearly everything, hundreds of positions back too; keys with very
    negative scores leave nearly nothing."""
    heads, kv, dk, dv, ps = 4, 2, 16, 32, 16
    sink = torch.zeros((heads,), dtype=torch.float32, device=DEV)
    for pos, target in ((0, 0), (700, 0), (700, 352), (700, 700), (17, 16)):
        ctx = pos + 1
        n = 1 if decoded else min(ctx, 40)
        step, cache, bt, positions, req = _paged([ctx], [n], ps, kv * (dk + dv), dtype, seed=pos)
        g = torch.Generator().manual_seed(target)
        direction = torch.nn.functional.normalize(torch.randn((dk,), generator=g), dim=0)
        keys = -direction.repeat(ctx, kv, 1) * 8               # every other key: score -64
        keys[target] = direction * 8
        values = torch.zeros((ctx, kv, dv))
        values[:, :, 1] = 1.0
        values[target, :, :2] = torch.tensor([1.0, 0.0])
        _fill(cache, bt, [keys], [values], kv, dk, dv)
        for strength, share in ((8.0, 1.0), (0.0, 0.5 if pos == 0 else None), (-8.0, 0.0)):
            if share is None:
                continue
            q = torch.zeros((n, heads, dk))
            q[-1] = direction * strength
            out = torch.empty((n, heads * dv), dtype=dtype, device=DEV)
            ops.attention_options(q.reshape(n, -1).to(dtype).to(DEV), step, cache, out, heads, kv, dk, dv, 1.0, sink=sink)
            rows = out.float().view(n, heads, dv)
            if strength < 0 and pos > 0:                        # the other keys now score +64: the target is lost among them
                assert (rows[-1, :, 0] < 0.01).all()
            else:
                assert ((rows[-1, :, 0] - share).abs() < 0.01).all(), f"query {pos}, key {target}, strength {strength}: {rows[-1, :, 0].tolist()}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [False, True])
def test_the_windows_edge_over_shared_rows(ops, decoded, dtype):
    """Rows that are key and value at once, one key carrying all the weight: the last position the window
    keeps is seen, the one before it is not; at page borders, far back, and at the sequence's start."""
    heads, row, dv, ps = 4, 48, 32, 16
    for pos, window in ((300, 96), (300, 17), (300, 16), (40, 41), (40, 40), (5, 1), (700, 690)):
        ctx = pos + 1
        for target, seen in ((pos - window + 1, True), (pos - window, False)):
            if target < 0:
                continue
            n = 1 if decoded else min(ctx, 40)
            step, cache, bt, positions, req = _paged([ctx], [n], ps, row, dtype, seed=pos)
            g = torch.Generator().manual_seed(target)
            direction = torch.zeros((row,))
            direction[dv:] = torch.nn.functional.normalize(torch.randn((row - dv,), generator=g), dim=0)
            rows = torch.randn((ctx, 1, row), generator=g) * 0.05
            rows[:, :, 1] = 1.0
            rows[:, :, 0] = 0.0
            rows[target, 0] = direction * 8
            rows[target, 0, 0], rows[target, 0, 1] = 1.0, 0.0
            _fill(cache, bt, [rows], [None], 1, row, 0)
            q = torch.zeros((n, heads, row))
            q[-1, :, dv:] = direction[dv:] * 8
            out = torch.empty((n, heads * dv), dtype=dtype, device=DEV)
            ops.attention_options(q.reshape(n, -1).to(dtype).to(DEV), step, cache, out, heads, 1, row, dv, 1.0,
                                  window=window, shared_rows=True)
            got = out.float().view(n, heads, dv)[-1, :, 0]
            assert ((got > 0.99) if seen else (got < 0.01)).all(), f"query {pos}, window {window}, key {target}: {got.tolist()}"


# ---- parts alone ---------------------------------------------------------------------------------
def _part(ops, category, spec, w):
    from tinyinfer_b200.parts.base import build_part
    part = build_part(category, spec)
    part.load_weights({k: v.to(DEV) for k, v in w.items()}, ops)
    return part


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mlp", [moe(4, 2, 24, 1.5, identity=2, groups=(3, 2)), moe(6, 3, 16, 2.5, identity=3, groups=(3, 1)),
                                 moe(1, 1, 24, 3.0), moe(4, 4, 8, 1.0), moe(12, 3, 32, 1.5, identity=4, groups=(2, 1)),
                                 moe(2, 2, 64, 0.5, identity=6, groups=(4, 2))])
@pytest.mark.parametrize("t", [1, 7, 150, 700])      # 150 and 700 rows: the grouped products on the tensor cores
def test_experts_with_identity_among_them(ops, mlp, t, dtype):
    from tinyinfer_b200.config import nekorax
    width = 64
    g = torch.Generator().manual_seed(t)
    w = mlp_weights(mlp, width, g)
    cfg = SimpleNamespace(width=width)
    part = _part(ops, "ffn", nekorax._ffn_spec(cfg, nekorax._mlp({"mlp": mlp}, "here")), w)
    h = (torch.randn((t, width), generator=g) * 1.5).to(dtype)
    want = plain.moe({k: v.double() for k, v in w.items()}, "", h.double(), mlp)
    residual = torch.zeros((t, width), dtype=torch.float32, device=DEV)
    part.forward(ops, h.to(DEV), residual, SimpleNamespace(scratch={}))
    ops.flush()
    err = (residual.cpu().double() - want).abs().max(dim=-1).values / want.abs().max()
    if dtype == torch.float32:
        assert err.max() < 2e-5, f"off by {float(err.max()):.3g}"
    else:                                                # a near-tie in the choice may fall the other way
        assert err.median() < 3e-2 and torch.quantile(err, 0.9) < 3e-2 if t >= 10 else err.median() < 3e-2


MIXER_CASES = [attention(4, 2, 12, 8, 6, 1000.0, 0.29, conv=3), attention(1, 1, 16, 16, 0, 7.0, 0.25, conv=1),
               attention(3, 3, 8, 8, 2, 30.0, 0.35), attention(4, 2, 64, 64, 32, 20000.0, 0.125, conv=4),
               attention(2, 1, 128, 128, 128, 300000.0, 0.09, conv=2), attention(6, 6, 80, 32, 40, 250.0, 0.1, conv=7),
               latent(3, 8, 4, 10, 12, 20, 100.0, 0.3, window=20, scaling=(4.0, 16, 8.0, 1.0)),
               latent(2, 6, 8, 6, 10, 8, 3000.0, 0.35, window=7), latent(1, 16, 2, 16, 8, 8, 30.0, 0.25),
               latent(4, 64, 32, 64, 128, 96, 20000.0, 0.1, window=33, scaling=(16.0, 64, 32.0, 1.0)),
               latent(2, 128, 64, 128, 64, 64, 1000.0, 0.07, window=16),
               attention(6, 2, 32, 16, 16, 900.0, 0.18, conv=3), latent(6, 32, 16, 48, 64, 40, 500.0, 0.15, window=50)]
CUTS = [[("a", 30), ("b", 1)], [("b", 2), ("c", 5)], [("a", 1), ("b", 30), ("c", 1)], [("a", 2), ("c", 1)],
        [("a", 17), ("b", 7), ("c", 33)], [("a", 1)], [("a", 1), ("c", 2)], [("b", 0), ("d", 70)], [("d", 1), ("a", 1)]]
TOTAL = {"a": 53, "b": 40, "c": 42, "d": 71}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", MIXER_CASES)
def test_each_mixer_alone_in_portions(ops, case, dtype):
    """Four requests in portions down to one token; the fourth takes the state slot that the second
    gave back."""
    from tinyinfer_b200.config import nekorax
    kind, m = case["type"], case["mixer"]
    width = 64
    g = torch.Generator().manual_seed(5)
    w = mixer_weights(kind, m, width, g)
    cfg = SimpleNamespace(width=width, norm_eps=1e-5)
    layer = nekorax.NekoraxLayer(kind, nekorax._mixer(case, "here", kind), None)
    part = _part(ops, "mixer", nekorax._mixer_spec(cfg, layer), w)
    inputs = {r: (torch.randn((n, width), generator=g)).to(dtype).float() for r, n in TOTAL.items()}
    got = _run_mixer(ops, part, inputs, CUTS, dtype)
    w64 = {k: v.double() for k, v in w.items()}
    for r, x in inputs.items():
        want = plain.attention(w64, "", x.double(), m) if kind == "attention" else \
            plain.latent_attention(w64, "", x.double(), m, 1e-5)
        _close(got[r], want, dtype, f"{kind} request {r}")


def test_the_junction_in_front_of_a_pass(ops):
    from tinyinfer_b200.config.plan import PartSpec
    width, passes, t = 40, 3, 9
    g = torch.Generator().manual_seed(2)
    w = {"in": (torch.randn((width, 2 * width), generator=g) / width ** 0.5).to(torch.bfloat16),
         "step": torch.randn((passes, width), generator=g).to(torch.bfloat16)}
    for dtype in (torch.float32, torch.bfloat16):
        part = _part(ops, "junction", PartSpec("loop_input", {"hidden_size": width, "passes": passes}), w)
        x, x0 = torch.randn((t, width), generator=g), torch.randn((t, width), generator=g)
        step = SimpleNamespace(scratch={}, act_dtype=dtype, req_of_tok=torch.zeros(t, dtype=torch.int32, device=DEV),
                               cu_q=torch.tensor([0, t], dtype=torch.int32, device=DEV), num_requests=1, max_q_len=t)
        d, d0 = x.to(DEV), x0.to(DEV)
        for index in (0, 2):
            both = torch.cat([d.cpu().to(dtype).double(), x0.to(dtype).double()], dim=1)
            want = both @ w["in"].double().T + w["step"][index].double()
            part.forward(ops, d, d0, index, step)
            _close(d, want, torch.float32 if dtype == torch.float32 else torch.bfloat16, f"pass {index}")


# ---- whole models ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts(tmp_path_factory, name, dtype):
    d = make_model(tmp_path_factory.getbasetemp(), name)
    steps = traces.whole(_requests(name))
    out = _run(d, dtype, steps, traces.max_live_tokens(steps))
    _compare(steps, out, _plain(d, name), dtype, f"{name} whole")


def test_every_layer_run_against_the_plain_rows(tmp_path_factory):
    """What each layer run hands on, in float32: the first that differs names the mechanism."""
    from tinyinfer_b200 import Engine, StepEntry
    for name in ("A", "C"):
        d = make_model(tmp_path_factory.getbasetemp(), name)
        cfg, w = plain.load_folder(d)
        tokens = _requests(name)["r1"]
        want = []
        plain.forward(cfg, w, tokens, layers_out=want)
        eng = Engine(d, dtype="float32", page_size=16, num_pages=8, max_requests=1)
        got = []
        for block in eng.model.blocks:
            inner = block.forward
            block.forward = lambda ops, x, step, cache, inner=inner: (inner(ops, x, step, cache), got.append(x.clone()))[0]
        eng.step([StepEntry("x", tokens, [0])])
        assert len(got) == len(want) == len(plain.order_of_layers(cfg))
        for i, (a, b) in enumerate(zip(got, want)):
            assert (a.cpu().double() - b).abs().max() < MODEL_RTOL * b.abs().max(), f"{name}: layer run {i}"


@pytest.mark.parametrize("name, family, dtype", [
    ("A", "tail", "float32"), ("A", "portions", "float32"), ("A", "mixed", "float32"), ("A", "mixed", "bfloat16"),
    ("B", "portions", "float32"), ("B", "mixed", "float32"), ("B", "tail", "bfloat16"),
    ("C", "tail", "float32"), ("C", "portions", "bfloat16"), ("C", "mixed", "float32"), ("C", "mixed", "bfloat16"),
    ("C", "long portions", "bfloat16"), ("C", "long portions", "float32"), ("D", "mixed", "float32")])
def test_cuttings_agree_with_the_plain_implementation(tmp_path_factory, name, family, dtype):
    """Prefill against token-by-token decoding, portions down to two tokens, and up to four live
    requests of unequal length in a pool so small that pages and state slots are used again."""
    d = make_model(tmp_path_factory.getbasetemp(), name)
    reqs = _requests(name)
    steps = {"tail": lambda: traces.tail_decoded(reqs, tail=40), "portions": lambda: traces.portions(reqs),
             "long portions": lambda: traces.portions(reqs, sizes=(150, 2, 71, 70, 128, 3)),
             "mixed": lambda: traces.mixed(reqs, seed=5)}[family]()
    out = _run(d, dtype, steps, traces.max_live_tokens(steps))
    _compare(steps, out, _plain(d, name), dtype, f"{name} {family}")


@pytest.mark.parametrize("seed", range(12))
def test_drawn_configurations(tmp_path_factory, seed):
    """Sizes, constants, options and the order of layers drawn from a seed: mixed batches in a small pool in
    float32, whole prompts in bfloat16."""
    from nekorax_util import make_drawn_model
    d = make_drawn_model(tmp_path_factory.getbasetemp(), seed)
    cfg, w = plain.load_folder(d)
    reqs = {f"r{i}": random_tokens(cfg["vocab"], n, seed=seed * 10 + i) for i, n in enumerate([70, 45, 33, 2, 97, 1])}
    want = {r: plain.forward(cfg, w, t) for r, t in reqs.items()}
    steps = traces.mixed(reqs, seed=seed)
    _compare(steps, _run(d, "float32", steps, traces.max_live_tokens(steps)), want, "float32", f"drawn {seed} mixed")
    steps = traces.whole(reqs)
    _compare(steps, _run(d, "bfloat16", steps, traces.max_live_tokens(steps)), want, "bfloat16", f"drawn {seed} whole")


def test_one_state_slot_used_by_every_request_in_turn(tmp_path_factory):
    d = make_model(tmp_path_factory.getbasetemp(), "A")
    steps = traces.portions(_requests("A"), sizes=(40, 2, 9))
    out = _run(d, "float32", steps, traces.max_live_tokens(steps), max_requests=1)
    _compare(steps, out, _plain(d, "A"), "float32", "one slot")


def test_float32_cuttings_give_the_same_bits(tmp_path_factory):
    d = make_model(tmp_path_factory.getbasetemp(), "A")
    reqs = _requests("A")
    seen = {}
    for family in (traces.whole(reqs), traces.portions(reqs), traces.mixed(reqs, seed=2)):
        out = _run(d, "float32", family, traces.max_live_tokens(family))
        for r, rows in traces.collect(family, out).items():
            for p, x in rows:
                if (r, p) in seen:
                    assert torch.equal(seen[(r, p)], x), f"request {r} position {p}"
                seen[(r, p)] = x


def test_long_decoding_and_pages_given_back(tmp_path_factory):
    """170 tokens one by one through the decode graphs; the layers with a window give their pages back
    as it passes, the others hold eleven."""
    from tinyinfer_b200 import Engine, StepEntry
    d = make_model(tmp_path_factory.getbasetemp(), "A")
    tokens = random_tokens(SMALL["A"]["vocab"], 170, seed=77)
    cfg, w = plain.load_folder(d)
    want = plain.forward(cfg, w, tokens)
    eng = Engine(d, dtype="float32", page_size=16, num_pages=11, max_requests=2)
    got = [eng.step([StepEntry("x", tokens[:4], [3])])[0].cpu()]
    for p in range(4, len(tokens)):
        got.append(eng.decode_step([StepEntry("x", [tokens[p]], [0])])[0].cpu().clone())
        eng.cache.check()
    assert_close_logits(torch.stack(got), want[3:], MODEL_RTOL, "long decoding")
    free = {g.spec.window: n for g, n in zip(eng.cache.groups, eng.cache.free_pages())}
    assert free[None] == 0 and free[20] >= 8 and free[7] >= 9, free
    eng.finish("x")
    assert all(n == 11 for n in eng.cache.free_pages())


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tmp_path_factory, name, graphs):
    from tinyinfer_b200 import LLM, SamplingParams
    d = make_model(tmp_path_factory.getbasetemp(), name)
    cfg, w = plain.load_folder(d)
    prompts = [random_tokens(cfg["vocab"], n, seed=n) for n in (5, 31, 12)]
    llm = LLM(d, dtype="float32", max_seq=128, max_num_seqs=2, max_batched_tokens=24, page_size=16,
              cuda_graph=graphs)
    outs = llm.generate(prompts, SamplingParams(max_tokens=8))
    for prompt, out in zip(prompts, outs):
        assert out.tokens == plain.greedy(cfg, w, prompt, 8), f"prompt of {len(prompt)} tokens"


def test_random_weights_from_a_configuration(tmp_path):
    from tinyinfer_b200 import Engine, StepEntry, write_random_model
    cfg = copy.deepcopy(SMALL["C"])
    tokens = random_tokens(cfg["vocab"], 90, seed=1)
    a = Engine(config=cfg, seed=5, dtype="bfloat16", page_size=16, num_pages=16, max_requests=2)
    la = a.step([StepEntry("a", tokens, [0, 50, 89])])
    d = os.path.join(str(tmp_path), "written")
    write_random_model(d, cfg, seed=5)
    b = Engine(d, dtype="bfloat16", page_size=16, num_pages=16, max_requests=2)
    lb = b.step([StepEntry("a", tokens, [0, 50, 89])])
    assert torch.isfinite(la).all() and torch.equal(la, lb)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(tmp_path_factory, tmp_path, dtype):
    """The replay program as a user starts it: steps on standard input, logits in files."""
    import numpy as np
    d = make_model(tmp_path_factory.getbasetemp(), "C")
    steps = traces.mixed(_requests("C"), seed=9)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "out")
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out,
         "--max-tokens", str(traces.max_live_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
    vocab = SMALL["C"]["vocab"]
    outputs = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted:
            data = np.fromfile(os.path.join(out, f"{s['step']}.f32"), dtype="<f4")
            outputs[s["step"]] = torch.from_numpy(data.reshape(wanted, vocab).copy())
    _compare(steps, outputs, _plain(d, "C"), dtype, f"replay {dtype}")


def test_command_line_with_token_ids(tmp_path_factory, capsys):
    from tinyinfer_b200 import cli
    d = make_model(tmp_path_factory.getbasetemp(), "B")
    cfg, w = plain.load_folder(d)
    prompt = random_tokens(cfg["vocab"], 9, seed=4)
    rc = cli.main(["-m", d, "--tokens", "-p", " ".join(map(str, prompt)), "-n", "6", "--dtype", "float32",
                   "--max-seq", "64", "--max-num-seqs", "2", "--page-size", "16"])
    assert rc == 0
    out = capsys.readouterr().out
    line = [ln for ln in out.splitlines() if ln.startswith("[output]")][0]
    assert [int(x) for x in line.split()[1:]] == plain.greedy(cfg, w, prompt, 6)
