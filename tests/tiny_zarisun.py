"""Small Zarisun configurations (sizes unlike any real model's, several values of every option), a writer of random model
folders for them, and the plain implementation's logits."""
from __future__ import annotations

import json
import os

import torch

from logssms_b200.config import make_model_config
from logssms_b200.weights import write_random_model

from plain import zarisun_plain as P


def _rot(dims, base, scaling=None):
    rot = {"dims": dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return rot


def _attention(heads, kv_heads, dim, conv, window, scale, rot):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": conv, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = rot
    return {"type": "attention", "mixer": m}


def _latent(heads, dim, rot_dim, vdim, rank, scale, rot, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _model(width, vocab, eps, logit_scale, layers):
    return {"architecture": "Zarisun", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width, "logit_scale": logit_scale}


# A: all three mixers; a window (20) shorter than a page of 64 and crossed many times; grouped queries 3 to 1; a rotation
# over part of the head with a ramp; two layers that read the latents of layer 1, one right behind it and one further on;
# a layer without feed-forward
_ROT_A = _rot(16, 10000.0, (4.0, 64, 8.0, 1.0))
ZARI_A = _model(64, 211, 1e-5, 1.5, [
    {**_attention(6, 2, 16, 3, 20, 0.3, _rot(8, 500.0, (8.0, 32, 16.0, 2.0))), "mlp": _dense(96)},
    {**_latent(3, 24, 16, 8, 32, 0.2, _ROT_A), "mlp": _dense(40)},
    {**_latent(2, 8, 16, 24, 32, 0.25, _ROT_A, kv_from=1), "mlp": None},
    {**_delta(4, 2, 16, 24, 4), "mlp": _dense(72)},
    {**_latent(4, 16, 16, 16, 32, 0.15, _ROT_A, kv_from=1), "mlp": _dense(48)},
])

# B: the recurrent layer first; a window (70) just past a page; one tap and two taps; the whole head rotated, without
# scaling; sizes that take the tensor-core attentions (head 32, rank 64, rotated part 16)
ZARI_B = _model(96, 333, 1e-6, 0.7, [
    {**_delta(3, 3, 8, 136, 1), "mlp": None},
    {**_attention(4, 1, 32, 2, 70, 0.2, _rot(32, 10000.0)), "mlp": _dense(50)},
    {**_latent(4, 16, 16, 16, 64, 0.2, _rot(16, 30000.0, (2.0, 16, 4.0, 0.5))), "mlp": _dense(64)},
    {**_attention(2, 2, 16, 1, 1, 0.4, None), "mlp": None},
])

# C: sizes of 1 where the design allows them: one head, one key channel pair, one value channel, a window of 1 and one of
# 2, a one-tap convolution; a latent layer whose rotated part has two columns
ZARI_C = _model(48, 130, 1e-5, 1.0, [
    {**_attention(1, 1, 2, 1, 2, 0.5, _rot(2, 100.0)), "mlp": None},
    {**_delta(1, 1, 2, 1, 2), "mlp": _dense(8)},
    {**_latent(1, 1, 2, 1, 3, 0.5, _rot(2, 50.0, (3.0, 8, 2.0, 1.0))), "mlp": _dense(8)},
])

# D: recurrent layers only (no paged cache at all)
ZARI_D = _model(40, 90, 1e-5, 2.5, [
    {**_delta(2, 1, 40, 72, 4), "mlp": _dense(64)},
    {**_delta(4, 4, 16, 16, 3), "mlp": None},
])

# E: attention layers only, no mask on one of them (every earlier token is seen), windows of 64 (a page) and 400 (never
# reached); two latent layers with latents of their own and different ranks, each with a reader; nothing is a multiple
# of 8 in layer 3
ZARI_E = _model(56, 177, 1e-5, 1.0, [
    {**_attention(4, 2, 8, 4, 64, 0.35, _rot(4, 1000.0)), "mlp": _dense(64)},
    {**_latent(2, 8, 8, 8, 16, 0.3, _rot(8, 2000.0)), "mlp": None},
    {**_attention(2, 1, 24, 5, None, 0.2, _rot(24, 8000.0, (16.0, 128, 32.0, 1.0))), "mlp": _dense(30)},
    {**_latent(3, 5, 6, 7, 11, 0.3, _rot(6, 3000.0, (8.0, 20, 4.0, 1.0))), "mlp": _dense(31)},
    {**_latent(2, 8, 8, 4, 16, 0.3, _rot(8, 2000.0), kv_from=1), "mlp": _dense(16)},
    {**_attention(3, 3, 16, 3, 400, 0.25, _rot(16, 10000.0)), "mlp": None},
    {**_latent(5, 3, 6, 9, 11, 0.3, _rot(6, 3000.0, (8.0, 20, 4.0, 1.0)), kv_from=3), "mlp": None},
])


def random_zarisun(seed: int) -> dict:
    """A configuration with every size and option drawn at random within what config.json allows."""
    import random
    rng = random.Random(seed)
    layers, latents = [], []

    def rotation(limit):
        if rng.random() < 0.15:
            return None
        dims = 2 * rng.randint(1, limit // 2)
        sc = None if rng.random() < 0.4 else (rng.choice([2.0, 4.0, 8.0, 32.0]), rng.choice([16, 64, 512]), rng.choice([4.0, 32.0]), rng.choice([0.5, 1.0]))
        return _rot(dims, rng.choice([100.0, 10000.0, 40000.0]), sc)
    for i in range(rng.randint(2, 6)):
        r = rng.random()
        if r < 0.3:
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 24, 32, 64])
            mixer = _attention(kv * rng.choice([1, 2, 4]), kv, dim, rng.randint(1, 5), rng.choice([None, 1, 3, 17, 64, 65, 100, 300]),
                               rng.choice([0.1, 0.3]), rotation(dim))
        elif r < 0.6:
            kv = rng.choice([1, 2, 3])
            mixer = _delta(kv * rng.choice([1, 2]), kv, rng.choice([8, 16, 24, 64, 72]), rng.choice([4, 8, 24, 40]), rng.randint(1, 5))
        elif latents and rng.random() < 0.5:
            src = rng.choice(latents)
            theirs = layers[src]["mixer"]
            mixer = _latent(rng.randint(1, 5), rng.choice([4, 8, 16, 24]), theirs["rot_dim"], rng.choice([4, 8, 24]), theirs["kv_rank"],
                            rng.choice([0.1, 0.3]), theirs.get("rot"), kv_from=src)
        else:
            rot_dim = rng.choice([4, 8, 16, 32])
            mixer = _latent(rng.randint(1, 5), rng.choice([4, 8, 16, 24]), rot_dim, rng.choice([4, 8, 24]), rng.choice([8, 32, 40, 64]),
                            rng.choice([0.1, 0.3]), rotation(rot_dim))
            latents.append(i)
        layers.append({**mixer, "mlp": None if rng.random() < 0.3 else _dense(2 * rng.randint(8, 60))})
    return _model(2 * rng.randint(16, 48), rng.randint(60, 400), rng.choice([1e-5, 1e-6]), rng.choice([0.5, 1.0, 3.0]), layers)


ZARI = {"A": ZARI_A, "B": ZARI_B, "C": ZARI_C, "D": ZARI_D, "E": ZARI_E}
ZARI.update({f"R{seed}": random_zarisun(seed) for seed in range(1, 9)})


def make_zarisun_dir(path, raw: dict, seed: int = 0, dtype=torch.float32, sharp: float = 1.0) -> str:
    """Random weights for `raw` in `path`.  `sharp` scales the attentions' queries (the query norm's weight; the query
    projection of a latent attention) so that the softmax picks single keys: a missing or surplus key, or a sink that is
    left out, then moves the logits far beyond any tolerance."""
    from safetensors.torch import load_file, save_file
    out = write_random_model(make_model_config(raw), str(path), seed=seed, dtype=dtype, perturb=True)
    file = os.path.join(out, "model.safetensors")
    t = load_file(file)
    for i, layer in enumerate(raw["layers"]):
        if sharp == 1.0:
            break
        if layer["type"] == "attention":
            name = f"l{i}.mix.q.norm"
        elif layer["type"] == "latent_attention":
            name = f"l{i}.mix.q"
        else:
            continue
        t[name] = (t[name].float() * sharp).to(t[name].dtype)
    save_file(t, file)
    return out


def read_folder(model_dir: str):
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    return config, load_file(os.path.join(model_dir, "model.safetensors"))


def plain_logits(model_dir: str, ids, dtype=torch.float64) -> torch.Tensor:
    """The plain model's logits at every position, from the folder's stored weights (in `dtype` throughout)."""
    config, tensors = read_folder(model_dir)
    return P.forward(config, tensors, list(ids), dtype=dtype).double()


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per position: root mean square of the logits' difference (its mean over the vocabulary taken off) over the root
    mean square of the wanted logits."""
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all(), "engine produced non-finite logits"
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)


TOL = {"float32": 3e-4, "bfloat16": 5e-2}
