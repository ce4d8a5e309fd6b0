"""Linear attention with one fixed decay per head."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, StateNeed
from ..ops import kernels as K
from ..registry import MIXERS
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init, ones_init


@MIXERS.register("lightning_attention")
class LightningAttention(Part):
    """q, k [heads, key_dim], v [heads, value_dim] = silu of their projections of the input h.  Per head
    S <- decay_h S + k v^T, o = S^T q, with one fixed decay per head and no other scale.  The heads' outputs are RMS-normed
    together (one weight over all of them), times sigmoid(W_g h), then the output projection.

    Per-request state: S [heads, key_dim, value_dim] in float32.  It is the gated-linear-attention recurrence with a decay
    that all key channels and tokens of a head share, and runs on that mixer's kernels: prompt portions of a bfloat16
    engine in chunks of 16 tokens on the tensor cores (`K.gla_chunked`), everything else token by token (`K.gla_scan`).
    The four input products are one (rows q | k | v | g, merged at bind time).  Tensors: q, k, v, g, norm, o."""
    kernels = ("gla", "moe", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if len(spec.decay) != spec.num_heads:
            raise ValueError("lightning attention takes one decay per head")
        self.spec = spec
        self._jitter = 0.1 if perturb_init else 0.0
        self.in_w = self.norm_w = self.o_w = self.decay = None

    def param_specs(self):
        s = self.spec
        qk, vv = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        fan = normal_init(s.hidden_size ** -0.5)          # random weights: products of unit-size rows stay of unit size
        return {
            "q": ParamSpec((qk, s.hidden_size), MATRIX, fan), "k": ParamSpec((qk, s.hidden_size), MATRIX, fan),
            "v": ParamSpec((vv, s.hidden_size), MATRIX, fan), "g": ParamSpec((vv, s.hidden_size), MATRIX, fan),
            "norm": ParamSpec((vv,), VECTOR, ones_init(self._jitter)),
            "o": ParamSpec((s.hidden_size, vv), MATRIX, normal_init(2.0 * vv ** -0.5)),
        }

    def bind(self, t):
        self.in_w = torch.cat([t["q"], t["k"], t["v"], t["g"]], 0).contiguous()
        self.norm_w, self.o_w = t["norm"], t["o"]
        self.decay = torch.tensor(self.spec.decay, dtype=torch.float32, device=self.in_w.device)

    def setup(self, rt) -> None:
        pass

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(states=(StateNeed("lightning", (s.num_heads, s.key_dim, s.value_dim), torch.float32),))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True) -> torch.Tensor:
        s = self.spec
        H, dk, dv = s.num_heads, s.key_dim, s.value_dim
        qk, vv = H * dk, H * dv
        proj = K.silu_columns(K.linear(x, self.in_w), 2 * qk + vv)        # silu(q | k | v) | gate
        state = ctx.cache.states[cache_layer]["lightning"]
        sizes = (H, dk, dv, 1.0, 1.0)
        if ctx.has_long_portions and K.gla_chunked_ok(proj, dk):
            # long portions in chunks on the tensor cores; decoded tokens and short portions token by token
            chunks, n_chunks, per_request, n_long = ctx.long_portion_chunks(K.GLA_CHUNK)
            _, _, short_list, n_short = ctx.requests_by_portion()
            o = torch.empty((x.shape[0], vv), dtype=torch.float32, device=x.device)
            seg = {}
            if K.gla_segmented_pays(ctx.num_tokens, n_long, H, dv):
                segments, _, seg_requests, _ = ctx.long_portion_segments(K.GLA_CHUNK, K.GLA_SEGMENT)
                seg = {"segments": segments, "segment_requests": seg_requests}
            K.gla_chunked(proj, None, state, ctx.cu_seqlens, ctx.start_pos, ctx.slots, chunks, n_chunks, per_request, n_long,
                          *sizes, out=o, head_decay=self.decay, **seg)
            if n_short > 0:
                K.gla_scan(proj, None, state, ctx.cu_seqlens, ctx.start_pos, ctx.slots, ctx.num_requests, *sizes,
                           request_list=short_list, out=o, head_decay=self.decay)
        else:
            o = K.gla_scan(proj, None, state, ctx.cu_seqlens, ctx.start_pos, ctx.slots, ctx.num_requests, *sizes,
                           head_decay=self.decay)
        y = K.gla_norm_gate(o, proj[:, 2 * qk + vv:], self.norm_w, s.norm_eps, 1, sigmoid_gate=True)
        return K.linear(y, self.o_w)
