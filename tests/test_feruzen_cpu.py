"""Feruzen without a GPU: configuration errors, the plan, tensor names and shapes, what each
layer keeps per request (pages beside fixed-size state under one cache slot), and the plain
implementation's mechanisms at their edges."""
import copy
import math

import pytest
import torch

import plain_feruzen as plain
from feruzen_util import SMALL, SMALL_A, SMALL_B, random_weights
from tinyinfer_b200.cache import CacheManager
from tinyinfer_b200.config.registry import ConfigError, architecture_of
from tinyinfer_b200.parts.base import CompositeSpec, FixedStateSpec, PagedKVSpec
from tinyinfer_b200.parts.model import CausalLM
from tinyinfer_b200.weights.loader import check_tensors
from util import random_tokens


def _plan(cfg):
    arch = architecture_of(cfg)
    return arch.build_plan(arch.from_dict(cfg))


def test_registry_names_the_design():
    assert architecture_of({"architecture": "Feruzen"}).name == "Feruzen"


@pytest.mark.parametrize("path,value,text", [
    (("layers", 0, "type"), "conv", "known:"),
    (("layers", 1, "mixer", "kv_heads"), 3, "kv heads"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv heads"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 5, "even"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 14, "at most"),
    (("layers", 0, "mixer", "left", "scale"), None, "lacks"),
    (("layers", 0, "mixer", "right", "gate_cap"), 0.0, "positive"),
    (("layers", 0, "mixer", "right_scale"), "1", "number"),
    (("layers", 1, "mixer", "conv"), 0, ">= 1"),
    (("layers", 0, "mlp", "kind"), "glu", "known:"),
    (("layers", 1, "mlp", "router", "top"), 6, "top 6 of 5"),
    (("layers", 1, "mlp", "expert", "limit"), -1.0, "positive"),
    (("norm", "groups"), 5, "equal groups"),
    (("norm", "eps"), 0, "positive"),
    (("canon", "taps"), None, "lacks"),
])
def test_configuration_errors(path, value, text):
    cfg = copy.deepcopy(SMALL_A)
    node = cfg
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = value
    with pytest.raises(ConfigError, match=text):
        _plan(cfg)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_tensor_names_and_shapes(name):
    cfg = SMALL[name]
    model = CausalLM(_plan(cfg))
    want = model.expected_tensors()
    have = {k: tuple(v.shape) for k, v in random_weights(cfg, 0).items()}
    assert set(want) == set(have)
    check_tensors("here", want, have)


def test_what_a_layer_keeps():
    plan = _plan(SMALL_A)
    assert [e.cache_slot for e in plan.schedule] == [0, 1, 2, 3] and all(e.writes_cache for e in plan.schedule)
    assert plan.layers[2].ffn is None and plan.layers[2].ffn_norm is None
    specs = CausalLM(plan).cache_specs()
    # layer 0: one kept row in front of the mixers; pages of 2 kv heads; three heads of S [8, 12 + 1] and their maxima
    assert isinstance(specs[0], CompositeSpec)
    flat = dict(specs[0].flat())
    assert flat["conv"] == FixedStateSpec((48,), torch.float32)
    assert isinstance(flat["mixer.left"], PagedKVSpec) and flat["mixer.left"].num_kv_heads == 2
    assert flat["mixer.right"] == FixedStateSpec((3 * 8 * 13 + 3,), torch.float32)
    # layer 1: four heads of S [8, 12] and two kept rows of the q, k, v channels (16 + 16 + 48)
    assert dict(specs[1].flat())["mixer"] == FixedStateSpec((4 * 8 * 12 + 2 * 80,), torch.float32)
    # one tap keeps nothing
    flat_b = dict(CausalLM(_plan(SMALL_B)).cache_specs()[0].flat())
    assert "conv" not in flat_b and flat_b["mixer"] == FixedStateSpec((16 * 16,), torch.float32)


def test_composite_slots_in_the_cache_manager():
    specs = CausalLM(_plan(SMALL_A)).cache_specs()
    cm = CacheManager(specs, page_size=8, num_pages=6, max_requests=2, device="cpu")
    cm.reserve_step([("a", 19), ("b", 3)])
    slots = torch.tensor([cm.state_slot("a"), cm.state_slot("b")], dtype=torch.int32)
    tables = [torch.tensor([cm.block_table(g, r) + [-1] * (3 - len(cm.block_table(g, r))) for r in "ab"], dtype=torch.int32)
              for g in range(len(cm.groups))]
    view = cm.view(0, True, tables, slots)
    assert view["conv"].state.shape[-1] == 48 and view.child("mixer")["right"].state.shape[-1] == 3 * 8 * 13 + 3
    assert view.child("mixer")["left"].page_size == 8
    view["conv"].state[cm.state_slot("a")].fill_(3.0)
    view.child("mixer")["right"].state[cm.state_slot("a")].fill_(2.0)
    cm.check()
    cm.free_request("a")
    cm.reserve_step([("c", 1)])                                   # takes a's slot: the state starts at zero again
    assert cm.state_slot("c") == int(slots[0])
    view = cm.view(0, True, tables, slots)
    assert float(view["conv"].state[cm.state_slot("c")].abs().max()) == 0.0
    assert float(view.child("mixer")["right"].state[cm.state_slot("c")].abs().max()) == 0.0
    cm.free_request("b")
    cm.free_request("c")
    assert cm.free_pages() == [6] * len(cm.groups)


def test_plain_mechanisms_at_their_edges():
    F = torch.float64
    # norm in groups: every part has unit root mean square of its own
    x = torch.tensor([[3.0, 4.0, 0.0, -2.0, 1.0, 1.0]], dtype=F)
    y = plain.group_norm(x, torch.tensor([1.0, 1.0, 1.0, 1.0, 1.0, 3.0], dtype=F), 3, 0.0)
    assert torch.allclose(y, torch.tensor([[3 / 12.5 ** 0.5, 4 / 12.5 ** 0.5, 0.0, -(2 ** 0.5), 1.0, 3.0]], dtype=F))
    # the convolution's last column is the token's own; earlier columns reach back; zeros before the start
    h = torch.arange(1.0, 5.0, dtype=F).view(4, 1)
    assert plain.time_conv(h, torch.tensor([[100.0, 10.0, 1.0]], dtype=F)).view(-1).tolist() == [1.0, 12.0, 123.0, 234.0]
    # the clamps: the gate from above only, the other branch on both sides
    one = torch.ones((1, 1), dtype=F)
    big = plain.clamped_glu(torch.tensor([[10.0]], dtype=F), one, one, one, 2.0)
    assert abs(big.item() - 2.0 * torch.sigmoid(torch.tensor(1.702 * 2.0, dtype=F)).item() * 3.0) < 1e-12
    low = plain.clamped_glu(torch.tensor([[-10.0]], dtype=F), one, one, one, 2.0)
    assert abs(low.item() - (-10.0) * torch.sigmoid(torch.tensor(-17.02, dtype=F)).item() * (-1.0)) < 1e-12
    # rotation of neighbouring pairs: a quarter turn of the first pair, the rest as it was
    v = torch.tensor([[[1.0, 0.0, 5.0, 6.0]]], dtype=F)
    out = plain.turn_pairs(v, torch.tensor([1]), 2, math.e)       # one pair, frequency base^0 = 1
    assert torch.allclose(out, torch.tensor([[[math.cos(1.0), math.sin(1.0), 5.0, 6.0]]], dtype=F))


def test_plain_recurrences_by_hand():
    F = torch.float64
    width = 2
    # the delta rule with k = q along one axis: the second write replaces what the first left
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2}
    eye = torch.eye(2, dtype=F)
    w = {"x.q": eye * 50, "x.k": eye * 50, "x.v": eye, "x.q.conv": torch.ones((2, 1), dtype=F),
         "x.k.conv": torch.ones((2, 1), dtype=F), "x.v.conv": torch.ones((2, 1), dtype=F),
         "x.b": torch.full((1, 2), 40.0, dtype=F), "x.a": torch.full((1, 2), -40.0, dtype=F),
         "x.A_log": torch.zeros(1, dtype=F), "x.dt_bias": torch.zeros(1, dtype=F), "x.norm": torch.ones(2, dtype=F),
         "x.g": eye, "x.o": eye}
    h = torch.tensor([[1.0, 0.0], [1.0, 0.0]], dtype=F)
    # beta = 1, no decay: token 0 writes v under k, token 1 finds it there (u = 0) and reads the same;
    # the unit root mean square leaves the direction, sqrt 2 on the first axis, times silu(1) of the gate
    silu1 = 1.0 / (1.0 + math.exp(-1.0))
    out = plain.gated_delta(w, "x.", h, m, 0.0)
    assert torch.allclose(out, torch.tensor([[2 ** 0.5 * silu1, 0.0]] * 2, dtype=F), atol=1e-8)
    # the matrix memory with one token: S = e^(i - m) k v^T, n = e^(i - m) k, and m = max(f + 0, i)
    mm = {"heads": 1, "dim": 2, "vdim": 2, "gate_cap": 100.0}
    w2 = {"y.q": eye, "y.k": eye, "y.v": eye, "y.g": eye * 0, "y.i": torch.zeros((1, 2), dtype=F),
          "y.i.b": torch.tensor([-3.0], dtype=F), "y.f": torch.zeros((1, 2), dtype=F), "y.f.b": torch.tensor([0.0], dtype=F),
          "y.norm": torch.ones(2, dtype=F), "y.o": eye}
    out = plain.matrix_memory(w2, "y.", torch.tensor([[2.0, 0.0]], dtype=F), mm, 0.0)
    # m = max(logsigmoid(0), -3) = -ln 2; o = e^(i-m) 2 * 2 / sqrt 2 * (1, 0) / (max(|n.q|, e^(-m)) + 1e-6):
    # only its direction survives the unit root mean square: (sqrt 2, 0) times sigmoid(0)
    assert torch.allclose(out, torch.tensor([[2 ** 0.5 * 0.5, 0.0]], dtype=F), atol=1e-9)


def test_plain_router_takes_shares_as_they_are():
    F = torch.float64
    mlp = {"kind": "moe", "router": {"experts": 3, "top": 1}, "expert": {"ff": 1, "limit": 9.0}}
    w = {"m.router": torch.tensor([[0.0], [1.0], [0.5]], dtype=F)}
    for e in range(3):
        w[f"m.e{e}.gate"] = torch.ones((1, 1), dtype=F)
        w[f"m.e{e}.up"] = torch.zeros((1, 1), dtype=F)
        w[f"m.e{e}.down"] = torch.full((1, 1), float(e + 1), dtype=F)
    out = plain.feed_forward(w, "m.", torch.tensor([[1.0]], dtype=F), mlp)
    share = math.e / (1 + math.e + math.e ** 0.5)                 # expert 1's share of the softmax, not 1
    assert abs(out.item() - share * 2.0 * 1.0 / (1 + math.exp(-1.702))) < 1e-12


def test_plain_whole_equals_token_by_token_greedy():
    cfg = SMALL_B
    w = {k: v.double() for k, v in random_weights(cfg, 1).items()}
    tokens = random_tokens(cfg["vocab"], 12, seed=2)
    whole = plain.forward(cfg, w, tokens)
    for n in (1, 5, 12):                                          # causal: a prefix gives the same rows
        assert (plain.forward(cfg, w, tokens[:n]) - whole[:n]).abs().max() < 1e-9
    rows = []
    plain.forward(cfg, w, tokens, layer_rows=rows)
    assert len(rows) == len(cfg["layers"]) and rows[0].shape == (12, cfg["width"])
