"""Windowed grouped-query attention whose values are its convolved keys, with whole-row query/key norms, a sink and a gate per head."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, KVNeed, StateNeed
from ..ops import kernels as K
from ..registry import MIXERS
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init, ones_init
from .pooled_attention import _position
from .sink_attention import NO_WINDOW


@MIXERS.register("conv_attention")
class ConvAttention(Part):
    """q [heads, head_dim] and k [kv_heads, head_dim] from the input h; there is no value projection.  Both pass a short
    causal convolution per channel (no bias, no activation, zeros before the sequence's start; the last taps - 1 projected
    rows are per-request state).  The values are the keys as they leave the convolution.  Then q and k are each RMS-normed
    over their whole row (all heads at once, a weight per column) and rotated over neighbouring pairs of every head's first
    `position.rotary_dim` columns.  Query head j reads key/value head j // (heads / kv_heads); scores times `softmax_scale`;
    position i sees j with 0 <= i - j < window; exp(sink_j) joins the softmax's denominator with no key and no value; the
    head's output is multiplied by sigmoid((W_g h)_j) before the output projection.

    The four products that read h are one (rows q | k | g).  Keys (normed, rotated) and values are cached in pages that go
    back once the window has passed them.  The attention itself runs on the kernels of the attention over a window and pooled
    blocks, with no blocks and their sink option: prompt portions of a bfloat16 engine on the tensor cores, decoded tokens,
    short portions and float32 engines with key ranges side by side or a warp per (token, head).  Norms, angles, scores,
    weights and the gate are 32-bit.  Tensors: q, q.conv, q.norm, k, k.conv, k.norm, sink, g, o."""
    kernels = ("attention_pooled", "conv", "rope", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        if not 1 <= spec.conv_kernel <= 8:
            raise ValueError("the short convolution takes 1 .. 8 taps")
        self.spec = spec
        self._jitter = 0.1 if perturb_init else 0.0
        self.position = _position(spec.position, shared)
        self.in_w = self.conv_w = self.q_norm = self.k_norm = self.sinks = self.o_w = None

    def param_specs(self):
        s = self.spec
        nq, nk = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        fan = normal_init(s.hidden_size ** -0.5)          # random weights: products of unit-size rows stay of unit size
        taps = normal_init(0.5)
        specs = {
            "q": ParamSpec((nq, s.hidden_size), MATRIX, fan), "q.conv": ParamSpec((nq, s.conv_kernel), VECTOR, taps),
            "q.norm": ParamSpec((nq,), VECTOR, ones_init(self._jitter)),
            "k": ParamSpec((nk, s.hidden_size), MATRIX, fan), "k.conv": ParamSpec((nk, s.conv_kernel), VECTOR, taps),
            "k.norm": ParamSpec((nk,), VECTOR, ones_init(self._jitter)),
            "o": ParamSpec((s.hidden_size, nq), MATRIX, normal_init(2.0 * nq ** -0.5)),
        }
        if s.sink:
            specs["sink"] = ParamSpec((s.num_heads,), VECTOR, normal_init(1.0))
        if s.head_gate:
            specs["g"] = ParamSpec((s.num_heads, s.hidden_size), MATRIX, fan)
        return specs

    def bind(self, t):
        self.in_w = torch.cat([t["q"], t["k"]] + ([t["g"]] if self.spec.head_gate else []), 0).contiguous()
        self.conv_w = torch.cat([t["q.conv"], t["k.conv"]], 0).contiguous()
        self.q_norm, self.k_norm, self.sinks, self.o_w = t["q.norm"], t["k.norm"], t.get("sink"), t["o"]

    def setup(self, rt) -> None:
        self.position.setup(rt)

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        C = (s.num_heads + s.num_kv_heads) * s.head_dim
        states = (StateNeed("conv", (C, s.conv_kernel - 1), None),) if s.conv_kernel > 1 else ()
        return CacheNeeds(kv=KVNeed(s.num_kv_heads, s.head_dim, s.window, s.head_dim), states=states)

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True) -> torch.Tensor:
        s = self.spec
        H, G, dim = s.num_heads, s.num_kv_heads, s.head_dim
        C = (H + G) * dim
        window = s.window if s.window is not None else NO_WINDOW
        k_cache, v_cache, gi = ctx.cache.kv(cache_layer)
        proj = K.linear(x, self.in_w)                                     # q | k | gate logits
        state = ctx.cache.states[cache_layer]["conv"] if s.conv_kernel > 1 else None
        qk = K.causal_conv1d(proj[:, :C], self.conv_w, None, state, ctx.cu_seqlens, ctx.start_pos, ctx.slots, ctx.num_requests,
                             ctx.max_len, (C, C), (1.0, 1.0, 1.0), activation="none")
        q = K.rownorm_prepare(qk, H, G, dim, ctx.positions, ctx.slot_mappings[gi], self.position.table, self.q_norm, self.k_norm,
                              s.norm_eps, k_cache, v_cache, writes_cache)
        table = ctx.block_tables[gi]
        extras = {"slopes": None, "sinks": self.sinks}
        most_keys = min(window, ctx.max_context)

        def few_rows(token_list=None, out=None, n=x.shape[0]):
            # decoded tokens and short portions: key ranges side by side where the sizes allow, else a warp per (token, head)
            args = (q, k_cache, v_cache, None, None, table, None, ctx.token_req, ctx.positions, None, s.softmax_scale, window, 0)
            if K.pooled_attention_split_ok(q, v_cache):
                return K.pooled_attention_split(*args, K.pooled_splits(n, G, most_keys), token_list=token_list, out=out, **extras)
            return K.pooled_attention(*args, token_list=token_list, out=out, **extras)

        if ctx.has_long_portions and K.pooled_attention_tile_ok(q, v_cache):
            # long portions on the tensor cores: runs of neighbouring tokens share their keys through shared memory
            tiles, n_tiles = ctx.long_portion_tiles(K.pooled_attention_tile_q())
            short, n_short = ctx.short_portion_tokens()
            o = torch.empty((x.shape[0], H * dim), dtype=q.dtype, device=q.device)
            K.pooled_attention_tile(q, k_cache, v_cache, None, None, table, None, ctx.cu_seqlens, ctx.start_pos, ctx.positions,
                                    tiles, None, s.softmax_scale, window, 0, o, splits=K.pooled_tile_splits(n_tiles, H), **extras)
            if n_short > 0:
                few_rows(short, o, n_short)
        else:
            o = few_rows()
        if s.head_gate:
            K.head_gate(o, proj[:, C:], H)
        return K.linear(o, self.o_w)
