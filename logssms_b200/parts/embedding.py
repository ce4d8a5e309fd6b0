"""Token embedding and output head."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..registry import EMBEDDINGS, HEADS, NORMS
from .base import MATRIX, ParamSpec, Part, normal_init


@EMBEDDINGS.register("embedding")
class Embedding(Part):
    """out = round(table[id] * multiplier), one kernel (python/logssms/models/falcon_h1.py:213)."""
    kernels = ("embed",)

    def __init__(self, vocab_size: int, hidden_size: int, multiplier: float = 1.0):
        self.vocab_size, self.hidden_size, self.multiplier = vocab_size, hidden_size, multiplier
        self.weight: torch.Tensor | None = None
        self.bad_ids: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size), MATRIX)}

    def bind(self, t):
        self.weight = t["weight"]
        self.bad_ids = torch.zeros(1, dtype=torch.int32, device=self.weight.device)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return K.embed_gather(self.weight, ids, self.multiplier, self.bad_ids)


@EMBEDDINGS.register("pair_embedding")
class PairEmbedding(Part):
    """Token embedding times a multiplier plus a hashed embedding of the (previous token, token) pair:
    row (previous * mul_prev + token * mul_cur) mod buckets of a second table, whose last row (number `buckets`)
    serves a sequence's first token.  The sum is made in 32-bit and starts a 32-bit stream (`K.StreamRows`).  The
    previous token is per-request state (one int32 per slot), so that prompts may be cut anywhere and decoded ids
    that never visit the host are still seen.  Tensors: `embed`, `bigram`."""
    kernels = ("embed",)
    needs_context = True      # forward(ids, ctx, cache_layer): the model gives it a cache layer for its state

    def __init__(self, vocab_size: int, hidden_size: int, multiplier: float = 1.0, *, buckets: int, mul_prev: int,
                 mul_cur: int):
        self.vocab_size, self.hidden_size, self.multiplier = vocab_size, hidden_size, multiplier
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.weight = self.pairs = self.bad_ids = None

    def param_specs(self):
        # random weights: both tables of a size that matters in the sum
        return {"embed": ParamSpec((self.vocab_size, self.hidden_size), MATRIX, normal_init(1.0 / max(abs(self.multiplier), 1e-3))),
                "bigram": ParamSpec((self.buckets + 1, self.hidden_size), MATRIX, normal_init(0.7))}

    def bind(self, t):
        self.weight, self.pairs = t["embed"], t["bigram"]
        self.bad_ids = torch.zeros(1, dtype=torch.int32, device=self.weight.device)

    def cache_needs(self):
        from ..cache import CacheNeeds, StateNeed
        return CacheNeeds(states=(StateNeed("previous_token", (1,), torch.int32),))

    def forward(self, ids: torch.Tensor, ctx=None, cache_layer: int | None = None):
        state = ctx.cache.states[cache_layer]["previous_token"]
        return K.embed_pair(self.weight, self.pairs, ids, ctx.token_req, ctx.cu_seqlens, ctx.start_pos, ctx.slots, state,
                            self.multiplier, self.buckets, self.mul_prev, self.mul_cur, self.bad_ids)


@EMBEDDINGS.register("stream_embedding")
class StreamEmbedding(Part):
    """The token's row of the table as the first value of a 32-bit stream (`K.StreamRows`); the rows themselves, in the
    activation dtype, stay at hand as the stream's `act` (a model whose layers mix them in again reads them there).
    Tensor: `embed`."""
    kernels = ("embed", "norm")

    def __init__(self, vocab_size: int, hidden_size: int, multiplier: float = 1.0):
        if multiplier != 1.0:
            raise ValueError("a stream embedding has no multiplier")
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.weight = self.bad_ids = None

    def param_specs(self):
        return {"embed": ParamSpec((self.vocab_size, self.hidden_size), MATRIX, normal_init(1.0))}

    def bind(self, t):
        self.weight = t["embed"]
        self.bad_ids = torch.zeros(1, dtype=torch.int32, device=self.weight.device)

    def forward(self, ids: torch.Tensor):
        rows = K.embed_gather(self.weight, ids, 1.0, self.bad_ids)
        return K.StreamRows(K.scale(rows, 1.0, to_f32=True), rows)


@EMBEDDINGS.register("normed_embedding")
class NormedEmbedding(Part):
    """The token's row of the table, normed (the norm of `norm`, a `NormSpec`, with its own weight): the first value of a
    32-bit stream (`K.StreamRows`).  Tensors: `embed` and the norm's weight."""
    kernels = ("embed", "stream_layer")

    def __init__(self, vocab_size: int, hidden_size: int, multiplier: float = 1.0, *, norm):
        if multiplier != 1.0:
            raise ValueError("a normed embedding has no multiplier (the norm would undo it)")
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.norm = NORMS.get(norm.kind)(norm)
        if not hasattr(self.norm, "norm_kind"):
            raise ValueError(f"norm {norm.kind!r} has no form on a 32-bit stream")
        self.weight = self.bad_ids = None

    def param_specs(self):
        return {"embed": ParamSpec((self.vocab_size, self.hidden_size), MATRIX, normal_init(1.0))}

    def children(self):
        return {"": self.norm}

    def bind(self, t):
        self.weight = t["embed"]
        self.bad_ids = torch.zeros(1, dtype=torch.int32, device=self.weight.device)

    def forward(self, ids: torch.Tensor):
        x = K.embed_norm(self.weight, ids, self.norm.weight, self.norm.eps, self.norm.norm_kind, self.bad_ids)
        return K.StreamRows(x, x.new_empty((0, self.hidden_size), dtype=self.weight.dtype))


@HEADS.register("lm_head")
class LMHead(Part):
    """logits = float32((h W^T) * multiplier); W is the embedding table when the model ties them
    (python/logssms/layers/embedding.py:94-106, python/logssms/models/falcon_h1.py:237)."""
    kernels = ("norm", "linear_skinny", "gemm_tcgen05")
    param_name = "weight"         # checkpoint name of the matrix relative to the head's prefix

    def __init__(self, vocab_size: int, hidden_size: int, multiplier: float, tied_to: Embedding | None):
        self.vocab_size, self.hidden_size, self.multiplier, self.tied_to = vocab_size, hidden_size, multiplier, tied_to
        self._weight = None

    def param_specs(self):
        if self.tied_to is not None:
            return {}
        return {self.param_name: ParamSpec((self.vocab_size, self.hidden_size), MATRIX)}

    def bind(self, t):
        self._weight = t.get(self.param_name)

    @property
    def weight(self) -> torch.Tensor:
        return self.tied_to.weight if self.tied_to is not None else self._weight

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return K.linear(h, self.weight, out_scale=self.multiplier, out_f32=True)


@HEADS.register("lm_head_bare")
class BareLMHead(LMHead):
    """The same head whose matrix is stored under the head's prefix itself (`head`, not `head.weight`)."""
    param_name = ""
