"""Nekorax without a GPU: its configuration and plan, tensor names, what every layer run keeps per
request, and the plain implementation against itself at the edges of its mechanisms."""
import copy
import math

import pytest
import torch

import plain_nekorax as plain
from nekorax_util import SMALL, attention, latent, make_model, mixer_weights, moe, random_weights

F64 = torch.float64


def _plan(cfg):
    from tinyinfer_b200.config import architecture_of
    arch = architecture_of(cfg)
    return arch.build_plan(arch.from_dict(cfg))


def test_registered_under_its_name():
    from tinyinfer_b200.config import get_architecture
    assert get_architecture("Nekorax") is get_architecture("nekorax")


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_tensor_names_and_shapes(name):
    from tinyinfer_b200.parts.model import CausalLM
    cfg = SMALL[name]
    model = CausalLM(_plan(cfg))
    want = random_weights(cfg, 1)
    expected = model.expected_tensors()
    assert set(expected) == set(want)
    for n, spec in expected.items():
        assert tuple(spec.shape) == tuple(want[n].shape), n


def test_schedule_follows_the_loop():
    plan = _plan(SMALL["A"])                       # layers 1 and 2 twice
    runs = [(e.layer, e.enter) for e in plan.schedule]
    assert runs == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert [e.cache_slot for e in plan.schedule] == list(range(6))
    assert runs == [(i, t if i == 1 else None) for i, t in plain.order_of_layers(SMALL["A"])]
    assert [e.enter for e in _plan(SMALL["B"]).schedule] == [0, None, None, None]
    assert [e.enter for e in _plan(SMALL["C"]).schedule] == [0, None, None, 1, None, None, 2, None, None, None]
    plan = _plan(SMALL["D"])
    assert plan.junction is None and all(e.enter is None for e in plan.schedule)


def test_what_every_layer_run_keeps():
    from tinyinfer_b200.parts.base import CompositeSpec, FixedStateSpec, PagedKVSpec
    from tinyinfer_b200.parts.model import CausalLM
    specs = CausalLM(_plan(SMALL["A"])).cache_specs()
    assert len(specs) == 6
    a = SMALL["A"]["layers"][0]["mixer"]
    channels = (a["heads"] + a["kv_heads"]) * a["dim"] + a["kv_heads"] * a["vdim"]
    assert specs[0] == CompositeSpec((("conv", FixedStateSpec((2 * channels,), torch.float32)),
                                      ("kv", PagedKVSpec(2, 12, None, 8))))
    assert specs[1] == specs[3] == PagedKVSpec(1, 12 + 4, 20, 0)        # one row of latent and key part, a window
    assert specs[5] == PagedKVSpec(1, 10 + 8, 7, 0)
    b = CausalLM(_plan(SMALL["B"])).cache_specs()
    assert b[0] == PagedKVSpec(1, 16, None, None)                        # one tap keeps nothing
    assert b[3] == PagedKVSpec(1, 6 + 4, None, 0)                        # no mask: every key


def test_pages_behind_a_window_go_back():
    from tinyinfer_b200.cache import CacheManager
    from tinyinfer_b200.parts.model import CausalLM
    cm = CacheManager(CausalLM(_plan(SMALL["A"])).cache_specs(), page_size=16, num_pages=8, max_requests=2)
    cm.reserve_step([("x", 100)])
    cm.release_passed("x")
    free = {g.spec.window: n for g, n in zip(cm.groups, cm.free_pages())}
    assert free == {None: 1, 20: 8 - 2, 7: 8 - 2}          # tokens 81 .. 99 and 94 .. 99 lie on the last two pages
    cm.free_request("x")
    assert cm.free_pages() == [8] * len(cm.groups)
    cm.check()


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].__setitem__("type", "wkv"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("vdim", 9), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 6), "rot_dim"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 4), "groups"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c["loop"].__setitem__("times", 0), "times"),
    (lambda c: c.pop("embedding"), "embedding"),
    (lambda c: c.__setitem__("logit_softcap", -1.0), "logit_softcap")])
def test_configuration_errors(change, message):
    from tinyinfer_b200.config import ConfigError
    cfg = copy.deepcopy(SMALL["A"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        _plan(cfg)


# ---- the plain implementation at its edges -----------------------------------------------------------
def test_turned_values_depend_on_distances_alone():
    """Shifting every position by the same amount leaves the attention mixer's output as it is, though
    keys, queries and values are all turned by absolute positions."""
    m = attention(2, 1, 8, 6, 4, 50.0, 0.3)["mixer"]
    g = torch.Generator().manual_seed(0)
    w = {k: v.double() for k, v in mixer_weights("attention", m, 16, g).items()}
    h = torch.randn((9, 16), generator=g, dtype=F64)
    whole = plain.attention(w, "", h, m)
    # the same rows behind three tokens that the queries cannot tell apart from nothing: zero rows
    # have zero keys (score 0) and zero values, so only the unit in the denominator grows
    pad = torch.zeros((3, 16), dtype=F64)
    shifted = plain.attention(w, "", torch.cat([pad, h]), m)[3:]
    assert not torch.allclose(whole, shifted)               # three more zero scores in the denominator
    fv = plain.frequencies(50.0, 6)
    v = torch.randn((5, 1, 6), generator=g, dtype=F64)
    there = plain.turn(v, torch.arange(5), fv, 6, "halves")
    back = plain.turn(there, -torch.arange(5), fv, 6, "halves")
    assert torch.allclose(back, v)
    moved = plain.turn(plain.turn(v, torch.arange(5) + 40, fv, 6, "halves"), -(torch.arange(5) + 47), fv, 6, "halves")
    assert torch.allclose(moved, plain.turn(v, torch.full((5,), -7), fv, 6, "halves"))


def test_the_unit_in_the_denominator():
    m = attention(1, 1, 4, 4, 0, 10.0, 1.0)["mixer"]
    w = {"q": torch.zeros((4, 4), dtype=F64), "k": torch.zeros((4, 4), dtype=F64), "v": torch.eye(4, dtype=F64),
         "g": torch.zeros((4, 4), dtype=F64), "o": torch.eye(4, dtype=F64)}
    h = torch.tensor([[2.0, 0.0, 0.0, 0.0]], dtype=F64)
    # one key of score 0 against the unit: half the value; the gate's sigmoid(0) halves it again
    assert torch.allclose(plain.attention(w, "", h, m), torch.tensor([[0.5, 0.0, 0.0, 0.0]], dtype=F64))


def test_window_edges_of_the_latent_mixer():
    m = latent(2, 6, 4, 6, 8, 8, 100.0, 0.4, window=5)["mixer"]
    g = torch.Generator().manual_seed(1)
    w = {k: v.double() for k, v in mixer_weights("latent_attention", m, 12, g).items()}
    h = torch.randn((12, 12), generator=g, dtype=F64)
    base = plain.latent_attention(w, "", h, m, 1e-6)
    moved = h.clone()
    moved[3] += 1.0                       # position 3 is seen by 3 .. 7, not by 8
    out = plain.latent_attention(w, "", moved, m, 1e-6)
    changed = [(out[i] - base[i]).abs().max() > 1e-9 for i in range(12)]
    assert changed == [False] * 3 + [True] * 5 + [False] * 4


def test_stretched_frequencies():
    from tinyinfer_b200.parts.rope import RopeStretched
    for dims, base, scaling in ((8, 100.0, (4.0, 16, 8.0, 1.0)), (32, 20000.0, (16.0, 64, 32.0, 1.0)), (4, 10.0, (2.0, 8, 1.0, 1.0))):
        named = dict(zip(("factor", "original", "fast", "slow"), scaling))
        want, mag = plain.yarn(plain.frequencies(base, dims), base, dims, named)
        part = RopeStretched(dims, base, *scaling)
        assert torch.allclose(part.inv_freq().double(), want, rtol=1e-6)
        assert math.isclose(part.rotation("cpu").scale, mag)
    # fast pairs stay, slow ones are divided by the factor
    plain_f = plain.frequencies(20000.0, 32)
    got, _ = plain.yarn(plain_f, 20000.0, 32, {"factor": 16.0, "original": 64, "fast": 32.0, "slow": 1.0})
    assert got[0] == plain_f[0] and math.isclose(got[-1], plain_f[-1] / 16.0)


def test_groups_correction_and_identity_in_the_plain_router():
    r = {"experts": 2, "identity": 2, "top": 2, "groups": {"count": 2, "keep": 1}}
    z = torch.log(torch.tensor([0.4, 0.1, 0.3, 0.2], dtype=F64))
    none = torch.zeros(4, dtype=F64)
    assert [e for e, _ in plain.route(z, none, r)] == [0, 1]              # the group of the largest score
    corr = torch.tensor([0.0, 0.0, 0.0, 0.3], dtype=F64)
    picked = plain.route(z, corr, r)
    assert [e for e, _ in picked] == [3, 2]                                # the correction moves the choice ...
    assert torch.allclose(torch.stack([x for _, x in picked]), torch.tensor([0.2, 0.3], dtype=F64))   # ... not the weights
    negative = torch.tensor([-1.0, -1.0, -2.0, -2.0], dtype=F64)
    assert [e for e, _ in plain.route(z, negative, r)] == [0, 1]          # outside the kept group: not 0 but never


def test_identity_experts_hand_the_input_on():
    mlp = moe(1, 2, 4, 1.0, identity=2)
    w = {"router": torch.tensor([[-9.0], [1.0], [1.0]], dtype=F64).repeat(1, 3), "correction": torch.zeros(3, dtype=F64),
         "e0.gate": torch.zeros((4, 3), dtype=F64), "e0.up": torch.zeros((4, 3), dtype=F64),
         "e0.down": torch.zeros((3, 4), dtype=F64)}
    h = torch.tensor([[1.0, 2.0, 3.0]], dtype=F64)
    out = plain.moe(w, "", h, mlp)
    assert torch.allclose(out, h, atol=1e-6)             # two identity experts of nearly half the weight each


def test_model_folder_round_trip(tmp_path):
    d = make_model(tmp_path, "D")
    cfg, w = plain.load_folder(d)
    assert cfg == SMALL["D"]
    rows = []
    logits = plain.forward(cfg, w, [1, 2, 3, 4], layers_out=rows)
    assert logits.shape == (4, 61) and len(rows) == 2 and logits.abs().max() <= cfg["logit_softcap"]
