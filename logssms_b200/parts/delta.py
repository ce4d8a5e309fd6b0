"""Gated delta rule with a decay per key channel."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, StateNeed
from ..ops import kernels as K
from ..registry import MIXERS
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init, ones_init


def _uniform(lo: float, hi: float):
    def init(gen, shape):
        return lo + (hi - lo) * torch.rand(shape, generator=gen, dtype=torch.float32)
    return init


@MIXERS.register("channel_delta")
class ChannelDelta(Part):
    """q, k [key heads, key_dim] and v [heads, value_dim] from the input h, each through a short causal convolution per
    channel (no bias, zeros before the sequence's start) and silu; value head j reads query/key head j // (heads / key heads).
    q and k become unit vectors per head, q also times key_dim^-1/2.  Per head, with g = exp(-exp(A_log) softplus(a2 (a1 h) +
    dt_bias)) per key channel and b = sigmoid(W_b h):  S <- diag(g) S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q (the
    read-out sees the token's own write).  o is RMS-normed per head (one weight [value_dim] for all heads), times
    sigmoid(g2 (g1 h)), then the output projection.

    Per-request state: the convolution's last taps - 1 inputs per channel (activation dtype) and S [heads, key_dim,
    value_dim] in float32.  The six input products are one (rows q | k | v | a1 | g1 | b, merged at bind time); the unit
    vectors, decays, gates, the state and the head norm are 32-bit in every engine dtype (`K.delta_scan` token by token for
    decoded tokens and short portions, `K.delta_scan_chunks` for long portions, `K.delta_scan_rows` for those past 256 key
    channels).
    Tensors: q, q.conv, k, k.conv, v, v.conv, b, A_log, dt_bias, a1, a2, g1, g2, norm, o."""
    kernels = ("delta", "conv", "gla", "moe", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if spec.num_heads % spec.num_key_heads:
            raise ValueError("value heads must be a multiple of query/key heads")
        if not 1 <= spec.conv_kernel <= 8:
            raise ValueError("the short convolution takes 1 .. 8 taps")
        self.spec = spec
        self._jitter = 0.1 if perturb_init else 0.0
        self.in_w = self.conv_w = self.a2_w = self.g2_w = self.o_w = self.norm_w = self.A_log = self.dt_bias = None
        self.rank_a = -1 if spec.decay_rank is None else spec.decay_rank
        self.rank_g = -1 if spec.gate_rank is None else spec.gate_rank

    def param_specs(self):
        s = self.spec
        qk, vv = s.num_key_heads * s.key_dim, s.num_heads * s.value_dim
        fan = normal_init(s.hidden_size ** -0.5)          # random weights: products of unit-size rows stay of unit size
        taps = normal_init(0.5)
        return {
            "q": ParamSpec((qk, s.hidden_size), MATRIX, fan), "q.conv": ParamSpec((qk, s.conv_kernel), VECTOR, taps),
            "k": ParamSpec((qk, s.hidden_size), MATRIX, fan), "k.conv": ParamSpec((qk, s.conv_kernel), VECTOR, taps),
            "v": ParamSpec((vv, s.hidden_size), MATRIX, fan), "v.conv": ParamSpec((vv, s.conv_kernel), VECTOR, taps),
            "b": ParamSpec((s.num_heads, s.hidden_size), MATRIX, fan),
            "A_log": ParamSpec((s.num_heads,), VECTOR, _uniform(-3.0, 0.5)),
            "dt_bias": ParamSpec((s.num_heads * s.key_dim,), VECTOR, normal_init(1.0)),
            "a1": ParamSpec((self.rank_a, s.hidden_size), MATRIX, fan),
            "a2": ParamSpec((s.num_heads * s.key_dim, self.rank_a), MATRIX, normal_init(max(self.rank_a, 1) ** -0.5)),
            "g1": ParamSpec((self.rank_g, s.hidden_size), MATRIX, fan),
            "g2": ParamSpec((vv, self.rank_g), MATRIX, normal_init(max(self.rank_g, 1) ** -0.5)),
            "norm": ParamSpec((s.value_dim,), VECTOR, ones_init(self._jitter)),
            "o": ParamSpec((s.hidden_size, vv), MATRIX, normal_init(2.0 * vv ** -0.5)),
        }

    def bind(self, t):
        for lo, hi in (("a1", "a2"), ("g1", "g2")):
            if t[lo].shape[0] != t[hi].shape[1]:
                raise ValueError(f"the two projections {lo}, {hi} disagree on their rank: {tuple(t[lo].shape)} and {tuple(t[hi].shape)}")
        self.rank_a, self.rank_g = t["a1"].shape[0], t["g1"].shape[0]
        self.in_w = torch.cat([t["q"], t["k"], t["v"], t["a1"], t["g1"], t["b"]], 0).contiguous()
        self.conv_w = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], 0).contiguous()
        self.a2_w, self.g2_w, self.o_w, self.norm_w = t["a2"].contiguous(), t["g2"].contiguous(), t["o"], t["norm"]
        self.A_log, self.dt_bias = t["A_log"], t["dt_bias"]

    def setup(self, rt) -> None:
        pass

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        C = 2 * s.num_key_heads * s.key_dim + s.num_heads * s.value_dim
        states = [StateNeed("delta", (s.num_heads, s.key_dim, s.value_dim), torch.float32)]
        if s.conv_kernel > 1:
            states.insert(0, StateNeed("conv", (C, s.conv_kernel - 1), None))
        return CacheNeeds(states=tuple(states))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True) -> torch.Tensor:
        s = self.spec
        H, Hk, dk, dv = s.num_heads, s.num_key_heads, s.key_dim, s.value_dim
        C = 2 * Hk * dk + H * dv
        proj = K.linear(x, self.in_w)                                     # q | k | v | low-rank decay, gate inputs | write gate
        states = ctx.cache.states[cache_layer]
        if s.conv_kernel > 1:
            conv = K.causal_conv1d(proj[:, :C], self.conv_w, None, states["conv"], ctx.cu_seqlens, ctx.start_pos, ctx.slots,
                                   ctx.num_requests, ctx.max_len, (C, C), (1.0, 1.0, 1.0))
        else:
            conv = K.silu_columns(proj, C, scale=self.conv_w.view(-1))           # one tap: a scale per channel, nothing carried
        ra, rg = self.rank_a, self.rank_g
        z = K.linear(proj[:, C:C + ra], self.a2_w, out_f32=True)
        gate = K.linear(proj[:, C + ra:C + ra + rg], self.g2_w)
        beta = proj[:, C + ra + rg:]
        args = (conv, z, self.dt_bias, self.A_log, beta, states["delta"], ctx.cu_seqlens, ctx.start_pos, ctx.slots, ctx.num_requests,
                H, Hk, dk, dv, dk ** -0.5, s.unit_eps)
        if ctx.has_long_portions and (K.delta_scan_chunks_ok(dk) or K.delta_scan_rows_ok(dk)):
            # long portions: what the recurrence reads is made for all tokens at once (in chunks of tokens that share one
            # reduction round, or, past 256 key channels, token by token with the state's update alone in the loop);
            # decoded tokens and short portions beside them token by token
            long_list, _, short_list, n_short = ctx.requests_by_portion()
            if K.delta_scan_chunks_ok(dk):
                chunks, n_chunks, per_request, n_long = ctx.long_portion_chunks(K.DELTA_CHUNK)
                o = K.delta_scan_chunks(*args[:9], chunks, n_chunks, per_request, n_long, *args[10:])
            else:
                o = K.delta_scan_rows(*args, request_list=long_list)
            if n_short > 0:
                K.delta_scan(*args, request_list=short_list, out=o)
        else:
            o = K.delta_scan(*args)
        y = K.gla_norm_gate(o, gate, self.norm_w, s.norm_eps, H, sigmoid_gate=True)
        return K.linear(y, self.o_w)


@MIXERS.register("gated_delta")
class GatedDelta(Part):
    """The gated delta rule with ONE decay per head.  q, k [key heads, key_dim] and v [heads, value_dim] from the input h, each
    through a short causal convolution per channel (no bias, zeros before the sequence's start) and silu; value head j reads
    query/key head j // (heads / key heads).  q and k become unit vectors per head, q also times key_dim^-1/2.  Per head, with
    g = exp(-exp(A_log) softplus(W_a h + dt_bias)) and b = sigmoid(W_b h), a number per head each:  S <- g S;  u = b (v - S^T k);
    S <- S + k u^T;  o = S^T q (the read-out sees the token's own write).  o is RMS-normed per head (one weight [value_dim] for
    all heads), times silu(W_g h), then the output projection.

    Per-request state: the convolution's last taps - 1 inputs per channel (activation dtype) and S [heads, key_dim,
    value_dim] in float32.  The products q | k | v | g | b are one; the decay's input comes from a second small product
    whose sums stay 32-bit.  It runs on `ChannelDelta`'s kernels with their `head_decay` option.
    Tensors: q, q.conv, k, k.conv, v, v.conv, a, dt_bias, A_log, b, g, norm, o."""
    kernels = ("delta", "conv", "gla", "moe", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if spec.num_heads % spec.num_key_heads:
            raise ValueError("value heads must be a multiple of query/key heads")
        if not 1 <= spec.conv_kernel <= 8:
            raise ValueError("the short convolution takes 1 .. 8 taps")
        self.spec = spec
        self._jitter = 0.1 if perturb_init else 0.0
        self.in_w = self.a_w = self.conv_w = self.o_w = self.norm_w = self.A_log = self.dt_bias = None

    def param_specs(self):
        s = self.spec
        qk, vv = s.num_key_heads * s.key_dim, s.num_heads * s.value_dim
        fan = normal_init(s.hidden_size ** -0.5)          # random weights: products of unit-size rows stay of unit size
        taps = normal_init(0.5)
        return {
            "q": ParamSpec((qk, s.hidden_size), MATRIX, fan), "q.conv": ParamSpec((qk, s.conv_kernel), VECTOR, taps),
            "k": ParamSpec((qk, s.hidden_size), MATRIX, fan), "k.conv": ParamSpec((qk, s.conv_kernel), VECTOR, taps),
            "v": ParamSpec((vv, s.hidden_size), MATRIX, fan), "v.conv": ParamSpec((vv, s.conv_kernel), VECTOR, taps),
            "a": ParamSpec((s.num_heads, s.hidden_size), MATRIX, fan),
            "b": ParamSpec((s.num_heads, s.hidden_size), MATRIX, fan),
            "A_log": ParamSpec((s.num_heads,), VECTOR, _uniform(-3.0, 0.5)),
            "dt_bias": ParamSpec((s.num_heads,), VECTOR, normal_init(1.0)),
            "g": ParamSpec((vv, s.hidden_size), MATRIX, fan),
            "norm": ParamSpec((s.value_dim,), VECTOR, ones_init(self._jitter)),
            "o": ParamSpec((s.hidden_size, vv), MATRIX, normal_init(2.0 * vv ** -0.5)),
        }

    def bind(self, t):
        self.in_w = torch.cat([t["q"], t["k"], t["v"], t["g"], t["b"]], 0).contiguous()
        self.a_w = t["a"].contiguous()
        self.conv_w = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], 0).contiguous()
        self.o_w, self.norm_w, self.A_log, self.dt_bias = t["o"], t["norm"], t["A_log"], t["dt_bias"]

    def setup(self, rt) -> None:
        pass

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        C = 2 * s.num_key_heads * s.key_dim + s.num_heads * s.value_dim
        states = [StateNeed("delta", (s.num_heads, s.key_dim, s.value_dim), torch.float32)]
        if s.conv_kernel > 1:
            states.insert(0, StateNeed("conv", (C, s.conv_kernel - 1), None))
        return CacheNeeds(states=tuple(states))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True) -> torch.Tensor:
        s = self.spec
        H, Hk, dk, dv = s.num_heads, s.num_key_heads, s.key_dim, s.value_dim
        C = 2 * Hk * dk + H * dv
        G = H * dv
        proj = K.linear(x, self.in_w)                                     # q | k | v | output gate | write gate
        z = K.linear_f32(x, self.a_w)                                     # the decay's input: sums handed on unrounded
        states = ctx.cache.states[cache_layer]
        conv = K.causal_conv1d(proj[:, :C], self.conv_w, None, states["conv"] if s.conv_kernel > 1 else None, ctx.cu_seqlens,
                               ctx.start_pos, ctx.slots, ctx.num_requests, ctx.max_len, (C, C), (1.0, 1.0, 1.0))
        beta = proj[:, C + G:]
        args = (conv, z, self.dt_bias, self.A_log, beta, states["delta"], ctx.cu_seqlens, ctx.start_pos, ctx.slots, ctx.num_requests,
                H, Hk, dk, dv, dk ** -0.5, s.unit_eps)
        if ctx.has_long_portions and (K.delta_scan_chunks_ok(dk) or K.delta_scan_rows_ok(dk)):
            # long portions in chunks of tokens (token by token past 256 key channels), decoded tokens and short portions
            # beside them token by token
            long_list, _, short_list, n_short = ctx.requests_by_portion()
            if K.delta_scan_chunks_ok(dk):
                chunks, n_chunks, per_request, n_long = ctx.long_portion_chunks(K.DELTA_CHUNK)
                o = K.delta_scan_chunks(*args[:9], chunks, n_chunks, per_request, n_long, *args[10:], head_decay=True)
            else:
                o = K.delta_scan_rows(*args, request_list=long_list, head_decay=True)
            if n_short > 0:
                K.delta_scan(*args, request_list=short_list, out=o, head_decay=True)
        else:
            o = K.delta_scan(*args, head_decay=True)
        y = K.gla_norm_gate(o, proj[:, C:C + G], self.norm_w, s.norm_eps, H)
        return K.linear(y, self.o_w)
