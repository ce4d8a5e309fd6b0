"""Zarisun on the CPU: configuration and its refusals, tensor names, cache layers of layers that read another layer's
latents, cache needs, the stretched rotation frequencies, and the plain functions against cases worked out by hand."""
import copy
import math

import pytest
import torch

from logssms_b200.config import ConfigError, make_model_config
from logssms_b200.models import build_model
from plain import zarisun_plain as P
from tiny_zarisun import ZARI, ZARI_A, ZARI_B, ZARI_E


def test_config_round_trip_and_specs():
    cfg = make_model_config(ZARI_A)
    assert cfg.to_dict() == ZARI_A and cfg.architectures == ("Zarisun",)
    spec = cfg.model_spec()
    assert [b.mixer.spec.kind for b in spec.layers] == ["conv_attention", "latent_attention", "latent_attention", "gated_delta", "latent_attention"]
    assert spec.lm_head_multiplier == 1.5 and spec.tie_word_embeddings
    a, l1, l2 = spec.layers[0].mixer.spec, spec.layers[1].mixer.spec, spec.layers[2].mixer.spec
    assert (a.window, a.conv_kernel, a.softmax_scale, a.position.rotary_dim, a.position.theta) == (20, 3, 0.3, 8, 500.0)
    assert dict(a.position.scaling) == {"factor": 8.0, "original": 32.0, "fast": 16.0, "slow": 2.0}
    assert l1.own_latents and not l2.own_latents and l1.pairing == "neighbours" and l1.sink and l1.head_gate and l1.window is None
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None
    assert spec.layers[0].feed_forward.activation == "silu"
    # a layer that reads another layer's latents uses that layer's cache layer and does not write it
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 1, False), (3, 2, True), (4, 1, False)]
    assert [(e.cache, e.writes_cache) for e in make_model_config(ZARI_E).model_spec().schedule] == \
        [(0, True), (1, True), (2, True), (3, True), (1, False), (4, True), (3, False)]
    no_mask = make_model_config(ZARI_E).model_spec().layers[2].mixer.spec
    assert no_mask.window is None
    assert make_model_config(ZARI_B).model_spec().layers[3].mixer.spec.position is None


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "convolution", "not a mixer"),
    (("layers", 0, "mixer", "heads"), 5, "multiple of kv_heads"),
    (("layers", 0, "mixer", "vdim"), 8, "vdim must equal dim"),
    (("layers", 0, "mixer", "conv"), 9, "taps"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "even"),
    (("layers", 0, "mixer", "rot", "dims"), 18, "at most"),
    (("layers", 0, "mixer", "rot", "scaling", "factor"), 0.0, "positive"),
    (("layers", 2, "mixer", "kv_from"), 0, "earlier latent_attention"),
    (("layers", 2, "mixer", "kv_from"), 2, "earlier latent_attention"),
    (("layers", 4, "mixer", "kv_from"), 2, "latents of its own"),
    (("layers", 2, "mixer", "kv_rank"), 16, "must equal those of layer 1"),
    (("layers", 1, "mixer", "rot_dim"), 7, "even"),
    (("layers", 0, "mlp", "kind"), "moe", "not 'dense'"),
    (("norm", "eps"), 0.0, "positive"),
    (("vocab",), 0, "positive"),
])
def test_config_refusals(path, value, word):
    raw = copy.deepcopy(ZARI_A)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        make_model_config(raw)


def test_missing_keys_are_refused():
    for drop in (("layers",), ("width",), ("norm",), ("layers", 0, "mixer", "scale"), ("layers", 1, "mixer", "kv_rank"), ("layers", 3, "mixer", "conv")):
        raw = copy.deepcopy(ZARI_A)
        at = raw
        for key in drop[:-1]:
            at = at[key]
        del at[drop[-1]]
        with pytest.raises(ConfigError):
            make_model_config(raw)


def test_tensor_names_and_shapes():
    model = build_model(make_model_config(ZARI_A))
    shapes = {n: tuple(s.shape) for n, s in model.named_param_specs()}
    assert shapes["embed"] == (211, 64) and shapes["final.norm"] == (64,) and "head.weight" not in shapes and "head" not in shapes
    assert shapes["l0.mix.q"] == (96, 64) and shapes["l0.mix.k"] == (32, 64) and shapes["l0.mix.q.conv"] == (96, 3)
    assert shapes["l0.mix.q.norm"] == (96,) and shapes["l0.mix.k.norm"] == (32,) and shapes["l0.mix.sink"] == (6,)
    assert shapes["l0.mix.g"] == (6, 64) and shapes["l0.mix.o"] == (64, 96) and "l0.mix.v" not in shapes
    assert shapes["l1.mix.q"] == (3 * 40, 64) and shapes["l1.mix.dkv"] == (48, 64) and shapes["l1.mix.dkv.norm"] == (32,)
    assert shapes["l1.mix.uk"] == (72, 32) and shapes["l1.mix.uv"] == (24, 32) and shapes["l1.mix.g"] == (3, 64)
    assert "l2.mix.dkv" not in shapes and "l2.mix.dkv.norm" not in shapes and shapes["l2.mix.uk"] == (16, 32)
    assert "l2.norm2" not in shapes and "l2.mlp.gate" not in shapes and shapes["l2.norm1"] == (64,)
    assert shapes["l3.mix.a"] == (4, 64) and shapes["l3.mix.b"] == (4, 64) and shapes["l3.mix.dt_bias"] == (4,) and shapes["l3.mix.A_log"] == (4,)
    assert shapes["l3.mix.g"] == (96, 64) and shapes["l3.mix.norm"] == (24,) and shapes["l3.mix.v.conv"] == (96, 4)
    assert shapes["l0.mlp.gate"] == (96, 64) and shapes["l0.mlp.down"] == (64, 96)


def test_cache_needs():
    needs = build_model(make_model_config(ZARI_A)).cache_needs()
    assert len(needs) == 3
    assert needs[0].kv.window == 20 and [t.shape for t in needs[0].kv.tensors] == [(2, 16), (2, 16)]
    assert [(s.name, s.shape) for s in needs[0].states] == [("conv", (128, 2))]
    assert needs[1].kv.window is None and [(t.name, t.shape) for t in needs[1].kv.tensors] == [("c", (32,)), ("kr", (16,))]
    assert [(s.name, s.shape, s.dtype) for s in needs[2].states] == [("conv", (160, 3), None), ("delta", (4, 16, 24), torch.float32)]
    one_tap = build_model(make_model_config(ZARI_B)).cache_needs()
    assert [s.name for s in one_tap[0].states] == ["delta"] and one_tap[3].states == ()


def test_every_tiny_configuration_builds():
    for name, raw in ZARI.items():
        model = build_model(make_model_config(raw))
        assert len(model.cache_needs()) == model.num_cache_layers, name


def test_ramp_frequencies_by_hand():
    from logssms_b200.parts.rope import ramp_frequencies
    # 8 columns, base 16: plain frequencies 16^(-i/4) = 1, 1/2, 1/4, 1/8
    f, mag = ramp_frequencies(8, 16.0, None)
    assert torch.allclose(f, torch.tensor([1.0, 0.5, 0.25, 0.125])) and mag == 1.0
    # factor 4, original 64, fast 4, slow 1: dim(4) = 8 ln(64 / (8 pi)) / (2 ln 16) = 1.348.., dim(1) = 8 ln(64 / (2 pi)) / (2 ln 16) = 3.348..
    # lo = 1, hi = min(4, 7) = 4: ramp = (i - 1) / 3 clamped = 0, 0, 1/3, 2/3
    f, mag = ramp_frequencies(8, 16.0, (("factor", 4.0), ("original", 64.0), ("fast", 4.0), ("slow", 1.0)))
    want = [1.0, 0.5, 0.25 / 4 / 3 + 0.25 * 2 / 3, 0.125 / 4 * 2 / 3 + 0.125 / 3]
    assert torch.allclose(f, torch.tensor(want), rtol=1e-6) and abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-12
    # the plain function says the same
    g, m2 = P.yarn_frequencies({"dims": 8, "base": 16.0, "scaling": {"factor": 4.0, "original": 64.0, "fast": 4.0, "slow": 1.0}})
    assert torch.allclose(g.float(), f) and abs(m2 - mag) < 1e-12
    # hi == lo: the ramp is a step (the divisor is 0.001, not 1)
    f, _ = ramp_frequencies(4, 100.0, (("factor", 2.0), ("original", 2 * math.pi), ("fast", 1.0), ("slow", 1.0)))
    assert torch.allclose(f, torch.tensor([1.0, 0.1 / 2]))


def test_plain_functions_by_hand():
    # convolution: the last column is the current token's, zeros before the start
    u = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    y = P.short_conv(u, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))
    assert y.flatten().tolist() == [1.0, 12.0, 124.0]
    # norm with eps inside the root
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(P.rms_norm(x, torch.tensor([1.0, 2.0], dtype=torch.float64), 0.5), x / math.sqrt(12.5 + 0.5) * torch.tensor([1.0, 2.0]))
    # rotation of neighbours: a quarter turn at position 1 with frequency pi/2 ... by the formula (u cos - v sin, v cos + u sin)
    q = torch.tensor([[[1.0, 0.0, 5.0]]], dtype=torch.float64).repeat(2, 1, 1)
    r = P.rotate(q, torch.tensor([0, 3]), {"dims": 2, "base": 7.0})
    assert torch.allclose(r[0], q[0]) and torch.allclose(r[1, 0], torch.tensor([math.cos(3.0), math.sin(3.0), 5.0], dtype=torch.float64))
    # sink softmax: equal scores over a window of 2, sink ln 2: weights 1 / (n + 2)
    k = torch.zeros(3, 1, 1, dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[2.0]], [[4.0]]], dtype=torch.float64)
    o = P.sink_softmax_attention(k, k, v, 1.0, torch.tensor([math.log(2.0)], dtype=torch.float64), 2)
    assert torch.allclose(o.flatten(), torch.tensor([1 / 3, 3 / 4, 6 / 4], dtype=torch.float64))
    o = P.sink_softmax_attention(k, k, v, 1.0, torch.tensor([math.log(2.0)], dtype=torch.float64), None)
    assert torch.allclose(o.flatten(), torch.tensor([1 / 3, 3 / 4, 7 / 5], dtype=torch.float64))


def test_plain_delta_rule_by_hand():
    # one head, one key channel, one value channel, one tap of 1: q = k = silu(h w) made unit (sign), S scalar
    W = 1
    p = {n: torch.ones(1, W, dtype=torch.float64) for n in ("q", "k", "v", "g")}
    p.update({"q.conv": torch.ones(1, 1, dtype=torch.float64), "k.conv": torch.ones(1, 1, dtype=torch.float64), "v.conv": torch.ones(1, 1, dtype=torch.float64),
              "a": torch.zeros(1, W, dtype=torch.float64), "b": torch.zeros(1, W, dtype=torch.float64), "A_log": torch.zeros(1, dtype=torch.float64),
              "dt_bias": torch.zeros(1, dtype=torch.float64), "norm": torch.ones(1, dtype=torch.float64), "o": torch.ones(1, 1, dtype=torch.float64)})
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1}
    h = torch.tensor([[2.0], [3.0]], dtype=torch.float64)
    silu = lambda z: z / (1 + math.exp(-z))
    unit = lambda z: z / math.sqrt(z * z + 1e-6)
    g = math.exp(-math.log(2.0))                      # exp(-exp(0) softplus(0)) = 1/2
    S, outs = 0.0, []
    for t in range(2):
        z = silu(float(h[t]))
        k = unit(z)
        S = g * S
        S = S + k * 0.5 * (z - S * k)                 # beta = sigmoid(0) = 1/2, v = silu(h)
        o = S * k                                      # q = unit * dim^-1/2 = unit
        outs.append(o / math.sqrt(o * o + 1e-5) * z)   # head norm over one channel, times silu(g h)
    got = P.delta_rule(h, p, m, 1e-5)
    assert torch.allclose(got.flatten(), torch.tensor(outs, dtype=torch.float64), rtol=1e-12)
