"""Causal grouped-query attention with normed queries and keys, a bias by distance and a sink; and two mixers side by side."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, KVNeed
from ..ops import kernels as K
from ..registry import MIXERS
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init, ones_init

NO_WINDOW = 1 << 30      # a window that no position reaches: every earlier token is seen


@MIXERS.register("sink_attention")
class SinkAttention(Part):
    """q [heads, head_dim], k [kv_heads, head_dim], v [kv_heads, value_dim] from the input; query head h reads key/value head
    h // (heads / kv_heads).  Queries and keys are RMS-normed per head with a weight each that the heads share; there is no
    rotation: the position enters through the query's factor 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) and through
    the bias slope_h * (i - j) that is taken off the scaled score of query i and key j, slope_h = 2^(-slope_span (h + 1) /
    heads).  Position i sees every j <= i.  The softmax's denominator also holds exp(sink_h), a stored number per head
    without key or value.

    Keys (normed) and values are cached in pages for the request's life.  It runs on the kernels of the attention over a
    window and pooled blocks, with no blocks, a window that is never reached, and their two options for the bias and the
    sink: prompt portions of a bfloat16 engine on the tensor cores (`K.pooled_attention_tile`), decoded tokens, short
    portions and float32 engines with key ranges side by side (`K.pooled_attention_split`) or a warp per (token, head)
    (`K.pooled_attention`).  Norms, the query's factor, scores and weights are 32-bit.
    Tensors: q, q.norm, k, k.norm, v, sink, o."""
    kernels = ("attention_pooled", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        self.spec = spec
        self._jitter = 0.1 if perturb_init else 0.0
        self.in_w = self.o_w = self.q_norm = self.k_norm = self.sinks = self.slopes = None

    def param_specs(self):
        s = self.spec
        fan = normal_init(s.hidden_size ** -0.5)          # random weights: products of unit-size rows stay of unit size
        specs = {
            "q": ParamSpec((s.num_heads * s.head_dim, s.hidden_size), MATRIX, fan),
            "q.norm": ParamSpec((s.head_dim,), VECTOR, ones_init(self._jitter)),
            "k": ParamSpec((s.num_kv_heads * s.head_dim, s.hidden_size), MATRIX, fan),
            "k.norm": ParamSpec((s.head_dim,), VECTOR, ones_init(self._jitter)),
            "v": ParamSpec((s.num_kv_heads * s.value_dim, s.hidden_size), MATRIX, fan),
            "o": ParamSpec((s.hidden_size, s.num_heads * s.value_dim), MATRIX, normal_init(2.0 * (s.num_heads * s.value_dim) ** -0.5)),
        }
        if s.sink:
            specs["sink"] = ParamSpec((s.num_heads,), VECTOR, normal_init(1.0))
        return specs

    def bind(self, t):
        s = self.spec
        self.in_w = torch.cat([t["q"], t["k"], t["v"]], 0).contiguous()
        self.o_w, self.q_norm, self.k_norm, self.sinks = t["o"], t["q.norm"], t["k.norm"], t.get("sink")
        self.slopes = None
        if s.slope_span != 0.0:
            slopes = [2.0 ** (-s.slope_span * (h + 1) / s.num_heads) for h in range(s.num_heads)]
            self.slopes = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(self.in_w.device)

    def setup(self, rt) -> None:
        pass

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(kv=KVNeed(s.num_kv_heads, s.head_dim, None, s.value_dim))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True) -> torch.Tensor:
        s = self.spec
        k_cache, v_cache, gi = ctx.cache.kv(cache_layer)
        qkv = K.linear(x, self.in_w)
        q = K.normed_prepare(qkv, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, ctx.positions, ctx.slot_mappings[gi],
                             self.q_norm, self.k_norm, s.norm_eps, s.temp_coef, s.temp_every, k_cache, v_cache, writes_cache)
        table = ctx.block_tables[gi]
        extras = {"slopes": self.slopes, "sinks": self.sinks}

        def few_rows(token_list=None, out=None, n=x.shape[0]):
            # decoded tokens and short portions: key ranges side by side where the sizes allow, else a warp per (token, head)
            args = (q, k_cache, v_cache, None, None, table, None, ctx.token_req, ctx.positions, None, s.softmax_scale, NO_WINDOW, 0)
            if K.pooled_attention_split_ok(q, v_cache):
                return K.pooled_attention_split(*args, K.pooled_splits(n, s.num_kv_heads, ctx.max_context), token_list=token_list,
                                                out=out, **extras)
            return K.pooled_attention(*args, token_list=token_list, out=out, **extras)

        if ctx.has_long_portions and K.pooled_attention_tile_ok(q, v_cache):
            # long portions on the tensor cores: runs of neighbouring tokens share their keys through shared memory
            tiles, n_tiles = ctx.long_portion_tiles(K.pooled_attention_tile_q())
            short, n_short = ctx.short_portion_tokens()
            o = torch.empty((x.shape[0], s.num_heads * s.value_dim), dtype=q.dtype, device=q.device)
            K.pooled_attention_tile(q, k_cache, v_cache, None, None, table, None, ctx.cu_seqlens, ctx.start_pos, ctx.positions,
                                    tiles, None, s.softmax_scale, NO_WINDOW, 0, o, splits=K.pooled_tile_splits(n_tiles, s.num_heads),
                                    **extras)
            if n_short > 0:
                few_rows(short, o, n_short)
        else:
            o = few_rows()
        return K.linear(o, self.o_w)


@MIXERS.register("mixer_pair")
class MixerPair(Part):
    """Two mixers side by side on the same input h: out_scale_left * left(h) + out_scale_right * right(h).  `forward` hands
    back the two outputs with their scales, as a list of (rows, scale): the kernel that joins the layer's sublayers to the
    stream adds them in 32-bit.  Both use the block's cache layer (at most one of them keeps keys and values; their state
    names must differ).  Tensors: the two mixers' own, under their slots' names."""

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        self.slots = (spec.left, spec.right)
        self.mixers = [MIXERS.get(m.spec.kind)(m.spec, perturb_init=perturb_init, shared=shared) for m in self.slots]
        for m in self.slots:
            if m.in_scale != 1.0:
                raise ValueError("a mixer pair's mixers read the input as it is")

    def children(self):
        return {slot.name: mixer for slot, mixer in zip(self.slots, self.mixers)}

    def setup(self, rt) -> None:
        for m in self.mixers:
            m.setup(rt)

    def cache_needs(self) -> CacheNeeds:
        kv, states = None, []
        for mixer in self.mixers:
            need = mixer.cache_needs()
            if need.more_paged:
                raise ValueError("a mixer pair takes mixers with one paged need at most")
            if need.kv is not None:
                if kv is not None:
                    raise ValueError("a mixer pair holds at most one mixer with a key/value cache")
                kv = need.kv
            states.extend(need.states)
        names = [s.name for s in states]
        if len(set(names)) != len(names):
            raise ValueError(f"state names clash inside a mixer pair: {names}")
        return CacheNeeds(kv=kv, states=tuple(states))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True):
        outs = []
        for slot, mixer in zip(self.slots, self.mixers):
            y = mixer.forward(x, ctx, cache_layer, writes_cache)
            outs += [(t, sc * slot.out_scale) for t, sc in y] if isinstance(y, list) else [(y, slot.out_scale)]
        return outs
