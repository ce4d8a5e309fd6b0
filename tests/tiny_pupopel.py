"""Small Pupopel configurations (sizes unlike any real model's, several values of every option), a writer of random model
folders for them, and the plain implementation's logits."""
from __future__ import annotations

import os

import torch

from logssms_b200.config import make_model_config
from logssms_b200.weights import write_random_model

from plain.pupopel_plain import PlainPupopel


def _delta(heads, kv_heads, dim, vdim, conv, decay_rank=8, gate_rank=6):
    return {"type": "channel_delta",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank, "gate_rank": gate_rank}}


def _pair(heads, kv_heads, dim, vdim, scale, temp, r_heads, r_dim, r_vdim, decay, left_scale=1.0, right_scale=1.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if temp is not None:
        left["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "parallel",
            "mixer": {"left": left, "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": list(decay)},
                      "left_scale": left_scale, "right_scale": right_scale}}


def _moe(ff, experts, top, shared):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _model(width, vocab, eps, loop, layers):
    raw = {"architecture": "Pupopel", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop is not None:
        raw["loop"] = dict(zip(("start", "stop", "times"), loop))
    return raw


# A: both mixers and both feed-forwards; value heads that share query/key heads (2 per key head), 3 taps; grouped queries
# (3 query heads per key head) with head sizes that differ between keys and values, a query factor that steps every 7
# tokens; decays from short to nearly none; the middle two layers run three times
PUPO_A = _model(64, 211, 1e-5, (1, 3, 3), [
    {**_delta(4, 2, 16, 24, 3), "mlp": _dense(96)},
    {**_pair(6, 2, 16, 24, 0.3, (0.4, 7), 3, 16, 8, (0.5, 0.9, 0.995), 0.7, 1.3), "mlp": _moe(24, 5, 2, 40)},
    {**_delta(2, 2, 32, 16, 4), "mlp": _moe(16, 3, 1, 0)},
    {**_pair(2, 2, 24, 8, 0.2, None, 1, 32, 40, (1.0,)), "mlp": None},
])

# B: the attention pair first and looped (its keys and values once per pass), one tap (nothing carried), two taps, a
# value head wider than 128 on the recurrent side, no loop product shared with anything else: the whole model twice
PUPO_B = _model(96, 333, 1e-6, (0, 3, 2), [
    {**_pair(4, 1, 8, 40, 0.35, (1.0, 1), 2, 8, 136, (0.97, 0.6), 1.0, 0.5), "mlp": _dense(50)},
    {**_delta(3, 3, 8, 136, 1), "mlp": None},
    {**_delta(6, 1, 24, 8, 2), "mlp": _moe(16, 8, 3, 24)},
])

# C: sizes of 1 where the design allows them; no loop at all (no product that opens a pass)
PUPO_C = _model(48, 130, 1e-5, None, [
    {**_delta(1, 1, 2, 1, 2, decay_rank=1, gate_rank=1), "mlp": _moe(8, 1, 1, 8)},
    {**_pair(1, 1, 4, 2, 0.5, (0.3, 1000), 1, 1, 1, (0.8,)), "mlp": None},
])

# D: recurrent layers only (no paged cache at all), the loop over one layer, once (a pass still opens with its product)
PUPO_D = _model(40, 90, 1e-5, (1, 2, 1), [
    {**_delta(2, 1, 40, 72, 4), "mlp": _dense(64)},
    {**_delta(4, 4, 16, 16, 3), "mlp": _moe(16, 4, 4, 16)},
])

# E: attention pairs only, two of them with equal cache needs (one page group) and one with others; an empty loop range
PUPO_E = _model(48, 77, 1e-5, (1, 1, 3), [
    {**_pair(4, 2, 8, 16, 0.4, (0.2, 16), 2, 16, 16, (0.9, 0.99)), "mlp": None},
    {**_pair(4, 2, 8, 16, 0.4, None, 1, 16, 32, (0.75,)), "mlp": _dense(64)},
    {**_pair(2, 1, 16, 24, 0.25, (0.5, 3), 2, 8, 8, (0.3, 1.0)), "mlp": _moe(24, 6, 2, 8)},
])

# F: nothing is a multiple of 8, or even of 2 where the design allows it: odd width, vocabulary, feed-forward sizes, ranks
# and head sizes (no 16-byte rows anywhere)
PUPO_F = _model(45, 101, 1e-5, (0, 2, 2), [
    {**_delta(3, 1, 12, 5, 3, decay_rank=5, gate_rank=3), "mlp": _dense(31)},
    {**_pair(3, 1, 6, 10, 0.4, (0.3, 5), 3, 5, 7, (0.9, 0.95, 0.5)), "mlp": _moe(19, 3, 2, 11)},
    {**_delta(2, 2, 20, 12, 5, decay_rank=7, gate_rank=9), "mlp": None},
])


def random_pupopel(seed: int) -> dict:
    """A configuration with every size and option drawn at random within what config.json allows."""
    import random
    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(2, 5)):
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3])
            mixer = _delta(kv * rng.choice([1, 2]), kv, rng.choice([8, 16, 24, 64, 72]), rng.choice([4, 8, 24, 40]), rng.randint(1, 5),
                           rng.choice([2, 8, 12]), rng.choice([3, 8]))
        else:
            kv = rng.choice([1, 2, 3])
            rh = rng.randint(1, 3)
            mixer = _pair(kv * rng.choice([1, 2, 4]), kv, rng.choice([8, 16, 24, 32, 64]), 2 * rng.randint(2, 40), rng.choice([0.1, 0.3]),
                          rng.choice([None, (0.3, 4), (0.1, 64)]), rh, rng.choice([8, 16, 32]), rng.choice([8, 24, 64]),
                          [rng.choice([0.5, 0.9, 0.99, 1.0]) for _ in range(rh)], rng.choice([0.5, 1.0]), rng.choice([0.8, 1.0]))
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            mlp = None
        elif kind == "dense":
            mlp = _dense(2 * rng.randint(8, 60))
        else:
            experts = rng.randint(1, 9)
            mlp = _moe(2 * rng.randint(4, 30), experts, rng.randint(1, min(experts, 3)), rng.choice([0, 8, 30]))
        layers.append({**mixer, "mlp": mlp})
    a = rng.randint(0, len(layers))
    b = rng.randint(a, len(layers))
    return _model(2 * rng.randint(16, 48), rng.randint(60, 400), rng.choice([1e-5, 1e-6]), rng.choice([None, (a, b, rng.randint(1, 3))]), layers)


PUPO = {"A": PUPO_A, "B": PUPO_B, "C": PUPO_C, "D": PUPO_D, "E": PUPO_E, "F": PUPO_F}
PUPO.update({f"R{seed}": random_pupopel(seed) for seed in range(1, 9)})


def make_pupopel_dir(path, raw: dict, seed: int = 0, dtype=torch.float32, sharp: float = 1.0) -> str:
    """Random weights for `raw` in `path`.  `sharp` scales the query norms of the softmax attentions so that the softmax
    picks single keys (a missing or surplus key then moves the logits far beyond any tolerance)."""
    from safetensors.torch import load_file, save_file
    out = write_random_model(make_model_config(raw), str(path), seed=seed, dtype=dtype, perturb=True)
    file = os.path.join(out, "model.safetensors")
    t = load_file(file)
    for name in list(t):
        if sharp != 1.0 and name.endswith(".left.q.norm"):
            t[name] = (t[name].float() * sharp).to(t[name].dtype)
    save_file(t, file)
    return out


def plain_model(model_dir: str) -> PlainPupopel:
    return PlainPupopel.from_folder(model_dir, torch.float64)


def plain_logits(model_dir: str, ids, dtype=torch.float64) -> torch.Tensor:
    m = PlainPupopel.from_folder(model_dir, dtype)
    return m.forward(list(ids), m.new_state()).double()


def without_close_calls(raw: dict) -> dict:
    """The same configuration with routers that choose all their experts (their weights still differ token by token): in a
    bfloat16 engine rounding turns a close call of a router now and then, which no tolerance on the logits allows for.
    The float32 runs keep the choice."""
    import copy
    raw = copy.deepcopy(raw)
    for layer in raw["layers"]:
        if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return raw


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per position: root mean square of the logits' difference (its mean over the vocabulary taken off) over the root
    mean square of the wanted logits."""
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all(), "engine produced non-finite logits"
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)


TOL = {"float32": 1e-4, "bfloat16": 5e-2}
