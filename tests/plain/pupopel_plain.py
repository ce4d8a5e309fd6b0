"""Plain, slow Pupopel: one function per mechanism, written from the design's equations.

Everything runs on the CPU in one dtype (float64 by default), token by token or with explicit loops over the keys;
nothing of the engine is imported.  Notation: h [T, width] is a sublayer's input, rows are tokens of ONE sequence in
order.  A sequence's carried state is a plain dict, so that a prompt may be fed in pieces.

    layer        h = RMS(x) (1 + w);  x <- x + mixer(h) + ff(h)           (one norm, both sublayers read it)
    loop         the layers [a, b) run n times, every pass with states of its own; each pass opens with
                 x <- W_in [x ; x0], x0 the token embeddings
    delta mixer  q, k, v through a short causal convolution and silu; q^, k^ unit vectors per head, q^ / sqrt(dim);
                 S <- diag(g_t) S;  u = b_t (v_t - S^T k^_t);  S <- S + k^_t u^T;  o_t = S^T q^_t
                 g_t = exp(-exp(A) softplus(a2 (a1 h) + dt)) per key channel, b_t = sigmoid(W_b h) per head;
                 y = W_o [RMS_head(o) w * sigmoid(g2 (g1 h))]
    pair mixer   cl * softmax attention + cr * linear attention, both on h
       softmax   RMS-normed q, k per head; q times 1 + c ln(floor((p + 1) / e) + 1); score s (q . k) - m_h (i - j),
                 m_h = 2^(-8 (h + 1) / H); the softmax's denominator also holds exp(sink_h)
       linear    q, k, v = silu(.); S <- d_h S + k v^T; o = S^T q; y = W_o [RMS(o) w * sigmoid(W_g h)]
    dense ff     W_d (gelu_tanh(W_g h) * W_u h)
    moe          z = W_r h + b; the `top` largest z are chosen, weights softmax over the chosen z;
                 y = sum_e w_e W_d,e (silu(W_g,e h) * W_u,e h) + the same form once more for every token ("shared")
"""
from __future__ import annotations

import json
import math
import os

import torch


# --------------------------------------------------------------------------- small pieces
def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def short_conv(x, taps, state, key):
    """y_t[c] = sum_j taps[c, j] x_{t - (n - 1) + j}[c], zeros before the sequence's start; the last n - 1 inputs are
    carried in state[key]."""
    n = taps.shape[1]
    past = state.get(key)
    if past is None:
        past = torch.zeros(n - 1, x.shape[1], dtype=x.dtype)
    full = torch.cat([past, x])
    state[key] = full[full.shape[0] - (n - 1):].clone()
    rows = [(full[t:t + n] * taps.T).sum(0) for t in range(x.shape[0])]
    return torch.stack(rows)


# --------------------------------------------------------------------------- delta rule with a decay per key channel
def channel_delta(h, W, state, *, heads, kv_heads, dim, vdim, eps):
    T = h.shape[0]
    q = silu(short_conv(h @ W["q"].T, W["q.conv"], state, "conv_q")).view(T, kv_heads, dim)
    k = silu(short_conv(h @ W["k"].T, W["k.conv"], state, "conv_k")).view(T, kv_heads, dim)
    v = silu(short_conv(h @ W["v"].T, W["v.conv"], state, "conv_v")).view(T, heads, vdim)
    unit = lambda a: a / torch.sqrt((a * a).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(q) * dim ** -0.5, unit(k)
    beta = torch.sigmoid(h @ W["b"].T)                                                     # [T, heads]
    step = softplus((h @ W["a1"].T) @ W["a2"].T + W["dt_bias"]).view(T, heads, dim)
    decay = torch.exp(-torch.exp(W["A_log"]).view(1, heads, 1) * step)                     # [T, heads, dim]
    gate = torch.sigmoid((h @ W["g1"].T) @ W["g2"].T).view(T, heads, vdim)
    S = state.get("S")
    if S is None:
        S = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    per = heads // kv_heads
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        for hd in range(heads):
            kk, qq = k[t, hd // per], q[t, hd // per]
            Sh = decay[t, hd].unsqueeze(1) * S[hd]
            u = beta[t, hd] * (v[t, hd] - Sh.T @ kk)
            Sh = Sh + torch.outer(kk, u)
            S[hd] = Sh
            out[t, hd] = Sh.T @ qq
    state["S"] = S
    y = rms(out, eps) * W["norm"] * gate
    return y.reshape(T, heads * vdim) @ W["o"].T


# --------------------------------------------------------------------------- softmax attention: bias by distance, sink
def sink_attention(h, W, state, *, heads, kv_heads, dim, vdim, scale, temp_coef, temp_every, eps):
    T = h.shape[0]
    start = 0 if "k" not in state else state["k"].shape[0]
    q = rms((h @ W["q"].T).view(T, heads, dim), eps) * W["q.norm"]
    k = rms((h @ W["k"].T).view(T, kv_heads, dim), eps) * W["k.norm"]
    v = (h @ W["v"].T).view(T, kv_heads, vdim)
    if start:
        k, v = torch.cat([state["k"], k]), torch.cat([state["v"], v])
    state["k"], state["v"] = k, v
    per = heads // kv_heads
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        i = start + t
        temp = 1.0 + temp_coef * math.log((i + 1) // temp_every + 1)
        dist = torch.arange(i, -1, -1, dtype=h.dtype)                   # i - j for j = 0 .. i
        for hd in range(heads):
            g = hd // per
            slope = 2.0 ** (-8.0 * (hd + 1) / heads)
            s = (k[:i + 1, g] @ (q[t, hd] * temp)) * scale - slope * dist
            sink = W["sink"][hd]
            top = torch.maximum(s.max(), sink)
            e = torch.exp(s - top)
            out[t, hd] = (e @ v[:i + 1, g]) / (e.sum() + torch.exp(sink - top))
    return out.reshape(T, heads * vdim) @ W["o"].T


# --------------------------------------------------------------------------- linear attention with a fixed decay per head
def lightning(h, W, state, *, heads, dim, vdim, decay, eps):
    T = h.shape[0]
    q = silu(h @ W["q"].T).view(T, heads, dim)
    k = silu(h @ W["k"].T).view(T, heads, dim)
    v = silu(h @ W["v"].T).view(T, heads, vdim)
    S = state.get("L")
    if S is None:
        S = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        for hd in range(heads):
            S[hd] = decay[hd] * S[hd] + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S[hd].T @ q[t, hd]
    state["L"] = S
    y = rms(out.reshape(T, heads * vdim), eps) * W["norm"] * torch.sigmoid(h @ W["g"].T)
    return y @ W["o"].T


def pair_mixer(h, W, state, m, eps):
    sub = lambda p: {k[len(p):]: v for k, v in W.items() if k.startswith(p)}
    L, R = m["left"], m["right"]
    temp = L.get("q_temp") or {"coef": 0.0, "every": 1}           # no query factor: times 1
    left = sink_attention(h, sub("left."), state, heads=L["heads"], kv_heads=L["kv_heads"], dim=L["dim"], vdim=L["vdim"],
                          scale=L["scale"], temp_coef=temp["coef"], temp_every=temp["every"], eps=eps)
    right = lightning(h, sub("right."), state, heads=R["heads"], dim=R["dim"], vdim=R["vdim"], decay=R["decay"], eps=eps)
    return m["left_scale"] * left + m["right_scale"] * right


# --------------------------------------------------------------------------- feed-forwards
def glu(h, W, prefix, act):
    return (act(h @ W[prefix + "gate"].T) * (h @ W[prefix + "up"].T)) @ W[prefix + "down"].T


def moe_ff(h, W, *, experts, top, shared, margins=None):
    z = h @ W["router"].T + W["router.b"]                       # [T, experts]
    if margins is not None:
        ranked = z.sort(-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if experts > top else torch.ones_like(z[:, 0]))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        best = torch.topk(z[t], top)
        weights = torch.softmax(best.values, 0)
        for w, e in zip(weights, best.indices.tolist()):
            out[t] += w * glu(h[t:t + 1], W, f"e{e}.", silu)[0]
    if shared:
        out = out + glu(h, W, "shared.", silu)
    return out


# --------------------------------------------------------------------------- the model
class PlainPupopel:
    def __init__(self, cfg: dict, tensors: dict, dtype=torch.float64):
        self.cfg = cfg
        self.w = {k: (v if v.dtype in (torch.int32, torch.int64) else v.to(dtype)) for k, v in tensors.items()}
        self.dtype = dtype
        n = len(cfg["layers"])
        loop = cfg.get("loop")
        # (layer, does a pass open here)
        if loop is None:
            self.runs = [(i, False) for i in range(n)]
        else:
            a, b, times = loop["start"], loop["stop"], loop["times"]
            inner = [(i, i == a) for i in range(a, b)]
            self.runs = [(i, False) for i in range(a)] + inner * times + [(i, False) for i in range(b, n)]

    @classmethod
    def from_folder(cls, folder: str, dtype=torch.float64):
        from safetensors import safe_open
        with open(os.path.join(folder, "config.json")) as f:
            cfg = json.load(f)
        tensors = {}
        with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name)
        return cls(cfg, tensors, dtype)

    def _sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self):
        return {"runs": [dict() for _ in self.runs]}

    def forward(self, ids, state, layer_outputs=None, margins=None):
        """Logits [T, vocab] of the next `ids` of a sequence whose earlier tokens left `state`."""
        cfg, eps = self.cfg, self.cfg["norm"]["eps"]
        x0 = self.w["embed"][torch.as_tensor(list(ids))]
        x = x0
        for run, (i, opens) in enumerate(self.runs):
            layer, st = cfg["layers"][i], state["runs"][run]
            if opens:
                x = torch.cat([x, x0], -1) @ self.w["loop.in"].T
            m = layer["mixer"]
            W = self._sub(f"l{i}.mix.")
            h = rms(x, eps) * (1.0 + self.w[f"l{i}.norm1"])
            if layer["type"] == "channel_delta":
                y = channel_delta(h, W, st, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], eps=eps)
            elif layer["type"] == "parallel":
                y = pair_mixer(h, W, st, m, eps)
            else:
                raise ValueError(layer["type"])
            ff = layer.get("mlp")
            if ff is not None:
                W = self._sub(f"l{i}.mlp.")
                if ff["kind"] == "dense":
                    y = y + glu(h, W, "", gelu_tanh)
                else:
                    y = y + moe_ff(h, W, experts=ff["router"]["experts"], top=ff["router"]["top"],
                                   shared=ff.get("shared") is not None, margins=margins)
            x = x + y
            if layer_outputs is not None:
                layer_outputs.append(x)
        return (rms(x, eps) * (1.0 + self.w["final.norm"])) @ self.w["head"].T
