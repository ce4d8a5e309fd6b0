"""Pupopel on the CPU: configuration, registry, declared tensors, the looped schedule with the products that open its
passes, cache needs, and the plain implementation against itself and against small cases worked out by hand."""
import copy
import math

import pytest
import torch

from logssms_b200.config import ConfigError, make_model_config
from logssms_b200.config.pupopel import PupopelConfig
from logssms_b200.models import build_model

from plain import pupopel_plain as P
from tiny_pupopel import PUPO, make_pupopel_dir, plain_model


def test_config_is_chosen_by_the_architecture_string_and_round_trips():
    cfg = make_model_config(PUPO["A"])
    assert isinstance(cfg, PupopelConfig) and cfg.architectures == ("Pupopel",)
    assert make_model_config(cfg.to_dict()).to_dict() == cfg.to_dict() == PUPO["A"]
    spec = cfg.model_spec()
    assert [b.kind for b in spec.layers] == ["parallel_stream"] * 4
    assert [b.mixer.spec.kind for b in spec.layers] == ["channel_delta", "mixer_pair", "channel_delta", "mixer_pair"]
    assert [None if b.feed_forward is None else b.feed_forward.kind for b in spec.layers] == ["glu", "routed_mlp", "routed_mlp", None]
    d = spec.layers[0].mixer.spec
    assert (d.num_heads, d.num_key_heads, d.key_dim, d.value_dim, d.conv_kernel, d.unit_eps) == (4, 2, 16, 24, 3, 1e-6)
    pair = spec.layers[1].mixer.spec
    left, right = pair.left.spec, pair.right.spec
    assert (pair.left.out_scale, pair.right.out_scale) == (0.7, 1.3)
    assert (left.num_heads, left.num_kv_heads, left.head_dim, left.value_dim, left.softmax_scale) == (6, 2, 16, 24, 0.3)
    assert (left.temp_coef, left.temp_every, left.slope_span, left.sink) == (0.4, 7, 8.0, True)
    assert (right.num_heads, right.key_dim, right.value_dim, right.decay) == (3, 16, 8, (0.5, 0.9, 0.995))
    no_temp = spec.layers[3].mixer.spec.left.spec
    assert (no_temp.temp_coef, no_temp.temp_every) == (0.0, 0)
    r = spec.layers[1].feed_forward
    assert (r.score, r.expert, r.weigh, r.router_bias, r.shared_size, r.top, r.num_experts) == ("softmax_chosen", "silu", "output", True, 40, 2, 5)
    assert spec.layers[2].feed_forward.shared_size == 0
    assert spec.final_norm.offset == 1.0 and spec.layers[0].norm.offset == 1.0


def test_the_loop_becomes_a_schedule_whose_passes_open_with_the_stream_input():
    spec = make_model_config(PUPO["A"]).model_spec()
    # layers 1 and 2 three times in a row, every run with a cache layer of its own; a pass opens right before layer 1
    assert [(e.layer, e.cache, e.opens) for e in spec.schedule] == [
        (0, 0, None), (1, 1, 0), (2, 2, None), (1, 3, 0), (2, 4, None), (1, 5, 0), (2, 6, None), (3, 7, None)]
    assert [s.name for s in spec.stream_inputs] == ["loop.in"]
    # no loop: no product at all; an empty range: the tensor exists, nothing opens; one layer once: it opens once
    none = make_model_config(PUPO["C"]).model_spec()
    assert none.stream_inputs == () and [e.opens for e in none.schedule] == [None, None]
    empty = make_model_config(PUPO["E"]).model_spec()
    assert [e.layer for e in empty.schedule] == [0, 1, 2] and all(e.opens is None for e in empty.schedule)
    once = make_model_config(PUPO["D"]).model_spec()
    assert [(e.layer, e.opens) for e in once.schedule] == [(0, None), (1, 0)]
    whole = make_model_config(PUPO["B"]).model_spec()
    assert [(e.layer, e.opens) for e in whole.schedule] == [(0, 0), (1, None), (2, None), (0, 0), (1, None), (2, None)]


@pytest.mark.parametrize("edit, message", [
    (lambda r: r["layers"][0].update(type="conv"), "not a mixer"),
    (lambda r: r["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda r: r["layers"][0]["mixer"].update(conv=9), "conv"),
    (lambda r: r["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda r: r["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda r: r["layers"][1]["mixer"]["right"].update(decay=[0.5, 0.9]), "decay"),
    (lambda r: r["layers"][1]["mixer"]["right"].update(decay=[0.5, 0.9, 1.5]), "decay"),
    (lambda r: r["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda r: r["layers"][0]["mlp"].update(kind="glu"), "neither"),
    (lambda r: r["loop"].update(stop=9), "loop"),
    (lambda r: r["loop"].update(times=0), "loop"),
    (lambda r: r["norm"].update(eps=0.0), "eps"),
    (lambda r: r.pop("layers"), "layers"),
])
def test_config_refuses_what_it_cannot_run(edit, message):
    raw = copy.deepcopy(PUPO["A"])
    edit(raw)
    with pytest.raises(ConfigError, match=message):
        make_model_config(raw)


def test_declared_tensors_carry_the_design_names():
    model = build_model(make_model_config(PUPO["A"]))
    names = {n: tuple(s.shape) for n, s in model.named_param_specs()}
    assert names["embed"] == (211, 64) and names["head"] == (211, 64) and names["final.norm"] == (64,)
    assert names["loop.in"] == (64, 128)
    assert names["l0.norm1"] == (64,)
    assert names["l0.mix.q"] == (32, 64) and names["l0.mix.k"] == (32, 64) and names["l0.mix.v"] == (96, 64)
    assert names["l0.mix.q.conv"] == (32, 3) and names["l0.mix.v.conv"] == (96, 3)
    assert names["l0.mix.b"] == (4, 64) and names["l0.mix.A_log"] == (4,) and names["l0.mix.dt_bias"] == (64,)
    assert names["l0.mix.a2"][0] == 64 and names["l0.mix.a1"][0] == names["l0.mix.a2"][1]
    assert names["l0.mix.g2"][0] == 96 and names["l0.mix.norm"] == (24,) and names["l0.mix.o"] == (64, 96)
    assert names["l0.mlp.gate"] == (96, 64) and names["l0.mlp.down"] == (64, 96)
    assert names["l1.mix.left.q"] == (96, 64) and names["l1.mix.left.k"] == (32, 64) and names["l1.mix.left.v"] == (48, 64)
    assert names["l1.mix.left.q.norm"] == (16,) and names["l1.mix.left.sink"] == (6,) and names["l1.mix.left.o"] == (64, 144)
    assert names["l1.mix.right.q"] == (48, 64) and names["l1.mix.right.v"] == (24, 64) and names["l1.mix.right.g"] == (24, 64)
    assert names["l1.mix.right.norm"] == (24,) and names["l1.mix.right.o"] == (64, 24)
    assert names["l1.mlp.router"] == (5, 64) and names["l1.mlp.router.b"] == (5,)
    assert names["l1.mlp.e4.gate"] == (24, 64) and names["l1.mlp.shared.down"] == (64, 40)
    assert "l2.mlp.shared.gate" not in names and not any(n.startswith("l3.mlp.") for n in names)
    assert "loop.in" not in {n for n, _ in build_model(make_model_config(PUPO["C"])).named_param_specs()}


def test_cache_needs_of_both_mixers_and_a_cache_layer_per_run():
    model = build_model(make_model_config(PUPO["A"]))
    needs = model.cache_needs()
    assert len(needs) == 8                                               # 1 + 2 layers x 3 passes + 1
    delta = {s.name: (tuple(s.shape), s.dtype) for s in needs[0].states}
    assert needs[0].kv is None
    assert delta["conv"] == ((2 * 2 * 16 + 4 * 24, 2), None) and delta["delta"] == ((4, 16, 24), torch.float32)
    pair = needs[1]
    assert pair.kv is not None and pair.kv.window is None                # keys and values for the request's whole life
    assert {s.name: tuple(s.shape) for s in pair.states} == {"lightning": (3, 16, 8)}
    assert needs[1] == needs[3] == needs[5] and needs[2] == needs[4] == needs[6]
    # one tap: no convolution window to carry; recurrent layers only: nothing is paged
    one_tap = build_model(make_model_config(PUPO["B"])).cache_needs()[1]
    assert [s.name for s in one_tap.states] == ["delta"]
    assert all(n.kv is None for n in build_model(make_model_config(PUPO["D"])).cache_needs())


# --------------------------------------------------------------------------- the plain implementation
@pytest.mark.parametrize("name", ["A", "B", "F"])
def test_plain_model_in_portions_equals_the_plain_model_at_once(tmp_path, name):
    folder = make_pupopel_dir(tmp_path / name, PUPO[name], seed=3)
    m = plain_model(folder)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, PUPO[name]["vocab"], (23,), generator=g).tolist()
    whole = m.forward(ids, m.new_state())
    state, parts = m.new_state(), []
    for lo, hi in ((0, 9), (9, 10), (10, 12), (12, 23)):
        parts.append(m.forward(ids[lo:hi], state))
    assert torch.allclose(torch.cat(parts), whole, rtol=1e-9, atol=1e-9)
    # a later token changes no earlier logits; an earlier one changes the later ones
    other = list(ids)
    other[15] = (other[15] + 1) % PUPO[name]["vocab"]
    moved = m.forward(other, m.new_state())
    assert torch.equal(moved[:15], whole[:15]) and not torch.allclose(moved[16:], whole[16:])


def _attention_weights(dim, heads, sink):
    eye = torch.eye(heads * dim, dtype=torch.float64)
    return {"q": eye.clone(), "k": eye[:dim].clone(), "v": eye[:dim].clone(), "q.norm": torch.ones(dim, dtype=torch.float64),
            "k.norm": torch.ones(dim, dtype=torch.float64), "sink": torch.tensor(sink, dtype=torch.float64),
            "o": torch.eye(heads * dim, dtype=torch.float64)}


def test_plain_sink_takes_its_share_without_a_value():
    """One token, one head: the score of the token on itself is scale * |q~|^2 = scale * dim (normed vectors), and the
    output is the value times e^s / (e^s + e^sink)."""
    dim, scale, sink = 4, 0.25, 0.7
    h = torch.tensor([[1.0, -2.0, 0.5, 3.0]], dtype=torch.float64)
    y = P.sink_attention(h, _attention_weights(dim, 1, [sink]), {}, heads=1, kv_heads=1, dim=dim, vdim=dim, scale=scale,
                         temp_coef=0.0, temp_every=1, eps=1e-12)
    s = scale * dim
    assert torch.allclose(y, h * math.exp(s) / (math.exp(s) + math.exp(sink)), rtol=1e-9)


def test_plain_bias_by_distance_and_query_factor_by_position():
    """Two equal tokens, two heads on one key head: both keys score alike, so head h weighs the older one e^(-slope_h) to
    1 (slope_h = 2^(-8 (h + 1) / 2)); with a sink far below that is all.  The query factor 1 + c ln(floor((p + 1) / every)
    + 1) scales position 1's score by 1 + c ln 2 when `every` is 2 and leaves position 0's alone."""
    dim = 2
    h = torch.tensor([[3.0, 4.0, 3.0, 4.0]] * 2, dtype=torch.float64)          # both heads read the same query
    W = _attention_weights(dim, 2, [-200.0, -200.0])
    W["v"] = torch.zeros(dim, 2 * dim, dtype=torch.float64)
    kw = dict(heads=2, kv_heads=1, dim=dim, vdim=dim, scale=0.5, eps=1e-12)
    # the cache as position 0 left it (normed key, value (0, 1)); position 1 brings the value (1, 1)
    k = P.rms(h[:1, :dim].view(1, 1, dim), 1e-12)
    for coef, every in ((0.0, 1), (0.6, 2)):
        state = {"k": k.clone(), "v": torch.tensor([[[0.0, 1.0]]], dtype=torch.float64)}
        Wv = dict(W)
        Wv["v"] = torch.tensor([[1.0 / 3.0, 0.0, 0.0, 0.0], [1.0 / 3.0, 0.0, 0.0, 0.0]], dtype=torch.float64)   # value (1, 1) for the new token
        y = P.sink_attention(h[1:2], Wv, state, temp_coef=coef, temp_every=every, **kw).view(2, dim)
        for hd in range(2):
            slope = 2.0 ** (-8.0 * (hd + 1) / 2)
            older = math.exp(-slope) / (1.0 + math.exp(-slope))               # equal scores whatever the query factor is
            assert abs(float(y[hd, 0]) - (1.0 - older)) < 1e-9 and abs(float(y[hd, 1]) - 1.0) < 1e-9
    # the factor itself: one key, a sink level with the unscaled score
    s = 0.5 * dim
    for p, factor in ((0, 1.0), (1, 1.0 + 0.6 * math.log(2.0))):
        state = {} if p == 0 else {"k": torch.zeros(1, 1, dim, dtype=torch.float64), "v": torch.zeros(1, 1, dim, dtype=torch.float64)}
        W1 = _attention_weights(dim, 1, [s])
        y = P.sink_attention(torch.tensor([[3.0, 4.0]], dtype=torch.float64), W1, state, heads=1, kv_heads=1, dim=dim, vdim=dim,
                             scale=0.5, temp_coef=0.6, temp_every=2, eps=1e-12)
        slope = 2.0 ** -8.0
        mine = math.exp(s * factor)
        rest = math.exp(s) + (math.exp(0.0 - slope) if p else 0.0)            # the sink, and at position 1 the zero key one step back
        assert torch.allclose(y, torch.tensor([[3.0, 4.0]], dtype=torch.float64) * mine / (mine + rest), rtol=1e-9)


def test_plain_router_weighs_the_chosen_experts_by_a_softmax_over_them_alone():
    width, ff = 3, 2
    W = {"router": torch.tensor([[1.0, 0, 0], [0, 1.0, 0], [0, 0, 1.0], [0, 0, 0]], dtype=torch.float64),
         "router.b": torch.tensor([0.0, 0.0, 0.0, 1.5], dtype=torch.float64)}
    for e in range(4):
        W[f"e{e}.gate"] = torch.full((ff, width), 0.1 * (e + 1), dtype=torch.float64)
        W[f"e{e}.up"] = torch.ones(ff, width, dtype=torch.float64)
        W[f"e{e}.down"] = torch.ones(width, ff, dtype=torch.float64) * (e + 1)
    h = torch.tensor([[2.0, 1.0, -1.0]], dtype=torch.float64)                 # logits 2, 1, -1 and the bias alone: 1.5
    y = P.moe_ff(h, W, experts=4, top=2, shared=False)
    w0, w3 = math.exp(2.0) / (math.exp(2.0) + math.exp(1.5)), math.exp(1.5) / (math.exp(2.0) + math.exp(1.5))
    one = lambda e: float(P.glu(h, W, f"e{e}.", P.silu)[0, 0])
    assert torch.allclose(y, torch.full((1, width), w0 * one(0) + w3 * one(3), dtype=torch.float64), rtol=1e-12)
