"""A plain, slow Zarisun: one function per mechanism, written from the design's equations in float64 tensor operations,
token by token where the design is a recurrence.  It shares no code with the engine; the engine's tests compare against it.

A model is (config mapping, {tensor name: tensor}); a request is a list of token ids.  `forward` returns the logits at
every position and, on request, the stream after every layer.  With another `dtype` than float64 every tensor and every
intermediate result is of that dtype (angles excepted): what rounding alone does to a model.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the sequence's start."""
    T, taps = u.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


def yarn_frequencies(rot):
    """The rotation's frequencies per pair and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((torch.arange(dims // 2, dtype=F) - lo) / max(hi - lo, 0.001), 0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, d]: neighbouring pairs of the first rot.dims columns of every head turn by position * frequency
    (`rot` None: nothing turns)."""
    if rot is None:
        return x
    dims = int(rot["dims"])
    f, m = yarn_frequencies(rot)
    a = positions.to(F)[:, None] * f[None, :]
    cos, sin = (torch.cos(a) * m)[:, None, :].to(x.dtype), (torch.sin(a) * m)[:, None, :].to(x.dtype)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def sink_softmax_attention(q, k, v, scale, sink, window):
    """q [T, H, d], k [T, H, d], v [T, H, dv] (keys already repeated per query head); position i sees j with
    0 <= i - j < window (None: every j <= i); the denominator also holds exp(sink_h)."""
    T, H = q.shape[0], q.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for h in range(H):
            s = (k[lo:i + 1, h] @ q[i, h]) * scale
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            out[i, h] = (e[:, None] * v[lo:i + 1, h]).sum(0) / (e.sum() + torch.exp(sink[h] - m))
    return out


def conv_attention(h, p, m, eps):
    """The 'attention' mixer on one sequence h [T, width]; p: its tensors by short name."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = short_conv(h @ p["q"].T, p["q.conv"])
    k = short_conv(h @ p["k"].T, p["k.conv"])
    v = k.view(T, G, d)                                     # the values are the keys as they leave the convolution
    q = rms_norm(q, p["q.norm"], eps).view(T, H, d)
    k = rms_norm(k, p["k.norm"], eps).view(T, G, d)
    pos = torch.arange(T)
    q, k = rotate(q, pos, m.get("rot")), rotate(k, pos, m.get("rot"))
    rep = H // G
    o = sink_softmax_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1), float(m["scale"]), p["sink"],
                               None if m.get("mask") is None else int(m["mask"]["size"]))
    o = o * torch.sigmoid(h @ p["g"].T)[:, :, None]
    return o.reshape(T, -1) @ p["o"].T


def latent_kv(h, p, m, eps):
    """The cached pair of a latent-attention layer: the normed latent c [T, rank] and the rotated key part [T, rot_dim]."""
    T, rank = h.shape[0], int(m["kv_rank"])
    d = h @ p["dkv"].T
    c = rms_norm(d[:, :rank], p["dkv.norm"], eps)
    kr = rotate(d[:, None, rank:], torch.arange(T), m.get("rot"))[:, 0]
    return c, kr


def latent_attention(h, p, m, eps, c, kr):
    T = h.shape[0]
    H, d, r, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    q = (h @ p["q"].T).view(T, H, d + r)
    q_rot = rotate(q[..., d:], torch.arange(T), m.get("rot"))
    k_nope = (c @ p["uk"].T).view(T, H, d)
    v = (c @ p["uv"].T).view(T, H, dv)
    qq = torch.cat([q[..., :d], q_rot], -1)
    kk = torch.cat([k_nope, kr[:, None, :].expand(T, H, r)], -1)
    o = sink_softmax_attention(qq, kk, v, float(m["scale"]), p["sink"], None)
    o = o * torch.sigmoid(h @ p["g"].T)[:, :, None]
    return o.reshape(T, -1) @ p["o"].T


def delta_rule(h, p, m, eps):
    T = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    silu = torch.nn.functional.silu
    q = silu(short_conv(h @ p["q"].T, p["q.conv"])).view(T, G, dk)
    k = silu(short_conv(h @ p["k"].T, p["k.conv"])).view(T, G, dk)
    v = silu(short_conv(h @ p["v"].T, p["v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ p["b"].T)
    g = torch.exp(-torch.exp(p["A_log"]) * torch.nn.functional.softplus(h @ p["a"].T + p["dt_bias"]))
    gate = silu(h @ p["g"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    for t in range(T):
        for j in range(H):
            kj, qj = k[t, j // (H // G)], q[t, j // (H // G)]
            S[j] = g[t, j] * S[j]
            u = beta[t, j] * (v[t, j] - S[j].T @ kj)
            S[j] = S[j] + torch.outer(kj, u)
            o[t, j] = S[j].T @ qj
    o = rms_norm(o, p["norm"], eps) * gate
    return o.reshape(T, -1) @ p["o"].T


def dense_ff(h, p):
    return (torch.nn.functional.silu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


def layer_tensors(tensors, prefix, dtype=F):
    return {k[len(prefix):]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, want_layers=False, dtype=F):
    """Logits [T, vocab] of one sequence (and the stream after every layer, [layers, T, width])."""
    eps = float(config["norm"]["eps"])
    embed = tensors["embed"].to(dtype)
    x = embed[torch.tensor(tokens)]
    streams, latents = [], {}
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        p = layer_tensors(tensors, f"l{i}.mix.", dtype)
        if layer["type"] == "attention":
            y = conv_attention(x, p, m, eps)
        elif layer["type"] == "delta":
            y = delta_rule(x, p, m, eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_kv(x, p, m, eps)
            y = latent_attention(x, p, m, eps, *latents[i if src is None else int(src)])
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, tensors[f"l{i}.norm1"].to(dtype), eps)
        if layer.get("mlp") is not None:
            y = dense_ff(x, layer_tensors(tensors, f"l{i}.mlp.", dtype))
            x = x + rms_norm(y, tensors[f"l{i}.norm2"].to(dtype), eps)
        streams.append(x)
    logits = rms_norm(x, tensors["final.norm"].to(dtype), eps) @ embed.T * float(config["logit_scale"])
    if want_layers:
        return logits, torch.stack(streams)
    return logits


def greedy(config, tensors, prompt, n):
    """The n tokens that greedy decoding appends to the prompt."""
    tokens, out = list(prompt), []
    for _ in range(n):
        nxt = int(forward(config, tensors, tokens)[-1].argmax())
        tokens.append(nxt)
        out.append(nxt)
    return out
