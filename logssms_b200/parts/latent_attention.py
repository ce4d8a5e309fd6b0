"""Attention over a paged cache of latents: one compressed row and one rotated key part per token."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, PagedNeed, PagedTensor
from ..ops import kernels as K
from ..registry import MIXERS, POSITION_ENCODINGS
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init, ones_init
from .rope import NoPositionEncoding


@MIXERS.register("latent_attention")
class LatentAttention(Part):
    """q = W_q h, per head [nope_dim | rot_dim]; W_dkv h = [latent (kv_rank) | rotated key part (rot_dim)].  The
    latent is RMS-normed (c), the key part and every head's rot_dim query part are rotated; only c and the key part
    are cached, per token, in pages.  A head's key is [W_uk,h c | key part], its value W_uv,h c; scores are scaled by
    `softmax_scale`, position i sees j with 0 <= i - j < window.

    The attention runs in the latent space: the query's unrotated part is folded through W_uk,h once per token, the
    softmax-weighted sum of the cached c rows is expanded through W_uv,h afterwards, so no key or value is ever
    expanded and a token costs (kv_rank + rot_dim) numbers of cache.  Tensors: q, dkv, dkv.norm, uk, uv, o.

    Options of the spec: `pairing` "neighbours" rotates columns (2i, 2i + 1) instead of (i, i + n/2); `sink`: exp(sink_h), a
    stored number per head, joins the softmax's denominator with no key and no value (tensor sink); `head_gate`: a head's
    output is multiplied by sigmoid((W_g h)_h) (tensor g, its rows ride in the input product); `own_latents` False: the layer
    has no dkv and no dkv.norm, and reads the latents and rotated key parts that another layer stored in the cache layer the
    schedule gives it (with `writes_cache=False`)."""
    kernels = ("attention_latent", "attention_pooled", "rope", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        self._jitter = 0.1 if perturb_init else 0.0
        if spec.position is None:
            self.position = NoPositionEncoding()
        else:
            key = ("position", spec.position)
            if shared is not None and key in shared:
                self.position = shared[key]
            else:
                self.position = POSITION_ENCODINGS.get(spec.position.kind)(spec.position)
                if shared is not None:
                    shared[key] = self.position
        if spec.pairing not in ("halves", "neighbours"):
            raise ValueError("the rotation pairs halves or neighbours")
        self.in_w = self.norm_w = self.uk = self.uv_t = self.o_w = self.sinks = None

    def param_specs(self):
        s = self.spec
        fan = normal_init(s.hidden_size ** -0.5)          # random weights: products of unit-size rows stay of unit size
        up = normal_init(s.kv_rank ** -0.5)
        specs = {
            "q": ParamSpec((s.num_heads * (s.nope_dim + s.rot_dim), s.hidden_size), MATRIX, fan),
            "uk": ParamSpec((s.num_heads * s.nope_dim, s.kv_rank), MATRIX, up),
            "uv": ParamSpec((s.num_heads * s.value_dim, s.kv_rank), MATRIX, up),
            "o": ParamSpec((s.hidden_size, s.num_heads * s.value_dim), MATRIX, normal_init(2.0 * (s.num_heads * s.value_dim) ** -0.5)),
        }
        if s.own_latents:
            specs["dkv"] = ParamSpec((s.kv_rank + s.rot_dim, s.hidden_size), MATRIX, fan)
            specs["dkv.norm"] = ParamSpec((s.kv_rank,), VECTOR, ones_init(self._jitter))
        if s.sink:
            specs["sink"] = ParamSpec((s.num_heads,), VECTOR, normal_init(1.0))
        if s.head_gate:
            specs["g"] = ParamSpec((s.num_heads, s.hidden_size), MATRIX, fan)
        return specs

    def bind(self, t):
        s = self.spec
        # rows of the one input product: queries | down-projection (a layer with latents of its own) | gate logits
        self.in_w = torch.cat([t["q"]] + ([t["dkv"]] if s.own_latents else []) + ([t["g"]] if s.head_gate else []), 0).contiguous()
        self.norm_w, self.o_w, self.sinks = t.get("dkv.norm"), t["o"], t.get("sink")
        self.uk = t["uk"].view(s.num_heads, s.nope_dim, s.kv_rank).contiguous()                       # [H, K = nope, N = rank]
        self.uv_t = t["uv"].view(s.num_heads, s.value_dim, s.kv_rank).transpose(1, 2).contiguous()     # [H, K = rank, N = value]

    def setup(self, rt) -> None:
        self.position.setup(rt)

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(kv=PagedNeed((PagedTensor("c", (s.kv_rank,)), PagedTensor("kr", (s.rot_dim,))), s.window))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True) -> torch.Tensor:
        s = self.spec
        T, H = x.shape[0], s.num_heads
        gi = ctx.cache.group_of_layer[cache_layer]
        group = ctx.cache.groups[gi]
        c_cache, kr_cache = group.tensor("c", cache_layer), group.tensor("kr", cache_layer)
        if writes_cache and not s.own_latents:
            raise ValueError("a latent-attention layer without latents of its own reads another layer's cache (writes_cache=False)")
        writes_cache = writes_cache and s.own_latents
        proj = K.linear(x, self.in_w)                                      # queries | latent | rotated key part | gate logits
        q_cols = H * (s.nope_dim + s.rot_dim)
        own = q_cols + (s.kv_rank + s.rot_dim if s.own_latents else 0)
        K.latent_prepare(proj[:, :own], H, s.nope_dim, s.rot_dim, s.kv_rank, ctx.positions, ctx.slot_mappings[gi],
                         self.position.table, self.norm_w, s.norm_eps, c_cache, kr_cache, writes_cache,
                         neighbours=s.pairing == "neighbours")
        q = proj[:, :H * (s.nope_dim + s.rot_dim)].view(T, H, s.nope_dim + s.rot_dim)
        qa = K.heads_matmul(q[:, :, :s.nope_dim], self.uk)                 # [T, H, rank]
        if ctx.has_long_portions and T * H >= 2048 and K.latent_attention_mma_ok(qa, s.rot_dim):
            # prompt portions on the tensor cores: up to 64 (token, head) rows of neighbouring tokens share a key tile
            rows = K.latent_wide_rows(T, H, s.kv_rank)
            blocks, _ = ctx.token_blocks(K.latent_wide_tokens(H, rows))
            lat = K.latent_attention_wide(qa, q[:, :, s.nope_dim:], c_cache, kr_cache, ctx.block_tables[gi], ctx.token_req,
                                          ctx.positions, blocks, s.softmax_scale, s.window or 0, rows=rows, sinks=self.sinks)
        elif ctx.host_lens is not None and K.latent_attention_mma_ok(qa, s.rot_dim):
            # the tensor-core form for few rows: tiles of 16 (token, head) rows that share their keys
            # (a step of single tokens needs no work list: every token is a block of its own)
            per_block = 1 if ctx.max_len == 1 else max(1, 16 // H)
            blocks, n_blocks = (None, T) if per_block == 1 else ctx.token_blocks(per_block)
            keys = min(ctx.max_context, (s.window or ctx.max_context) + per_block)
            lat = K.latent_attention_mma(qa, q[:, :, s.nope_dim:], c_cache, kr_cache, ctx.block_tables[gi], ctx.token_req,
                                         ctx.positions, blocks, s.softmax_scale, s.window or 0,
                                         splits=K.latent_splits(n_blocks, H, keys), sinks=self.sinks)
        else:
            qa = qa if qa.is_contiguous() else qa.contiguous()
            lat = K.latent_attention(qa, q[:, :, s.nope_dim:], c_cache, kr_cache, ctx.block_tables[gi], ctx.token_req,
                                     ctx.positions, s.softmax_scale, s.window or 0, sinks=self.sinks)
        o = K.heads_matmul(lat, self.uv_t)                                 # [T, H, value]
        o = o.reshape(T, H * s.value_dim)
        if s.head_gate:
            K.head_gate(o, proj[:, own:], H)
        return K.linear(o, self.o_w)
