"""Plain data that describes a model as parts, layer by layer.

An architecture's typed config (e.g. `FalconH1Config`) turns its config.json
keys into one `ModelSpec`.  Everything below the architecture file works from
these specs only, so no part knows which model it is in, and every size and
constant a part needs arrives as a field.

`kind` names an entry of the matching registry in `logssms_b200.registry`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding (neox / half-split pairing).

    Mirrors the reference's `RotaryConfig` (python/logssms/models/config.py:33-37).
    `scaling` is the config.json `rope_scaling` mapping as sorted items, or None.
    """
    head_dim: int
    rotary_dim: int
    theta: float
    max_position: int
    scaling: tuple[tuple[str, Any], ...] | None = None
    kind: str = "rope"


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    kind: str = "rmsnorm"
    param_name: str = "weight"     # checkpoint name of the weight relative to the norm's prefix ("" : the prefix itself)
    offset: float = 0.0            # the norm multiplies by offset + stored weight (1.0: a weight stored around zero)


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged key/value cache."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: RopeSpec | None
    key_scale: float = 1.0
    softmax_scale: float | None = None      # None -> head_dim ** -0.5
    window: int | None = None               # None -> all earlier keys
    kind: str = "attention"


@dataclass(frozen=True)
class Mamba2Spec:
    """Mamba2 (SSD) mixer with a depthwise causal conv in front."""
    hidden_size: int
    num_heads: int
    head_dim: int
    state_dim: int
    num_groups: int
    conv_kernel: int
    conv_bias: bool
    proj_bias: bool
    out_bias: bool
    gated_norm: bool
    norm_before_gate: bool
    norm_eps: float
    multipliers: tuple[float, float, float, float, float]   # gate z, x, B, C, dt
    chunk_size: int
    kind: str = "mamba2"

    @property
    def inner_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def conv_dim(self) -> int:
        return self.inner_size + 2 * self.num_groups * self.state_dim

    @property
    def proj_size(self) -> int:
        return self.inner_size + self.conv_dim + self.num_heads


@dataclass(frozen=True)
class GatedMLPSpec:
    hidden_size: int
    intermediate_size: int
    activation_scale: float = 1.0
    output_scale: float = 1.0
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class GLASpec:
    """Gated linear attention: a matrix state per head with a decay per key channel,
    decay = sigmoid(low-rank projection + bias) ** (1 / tau); per-head RMSNorm of the output, SiLU output gate."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    tau: float
    norm_eps: float
    decay_rank: int | None = None      # None: whatever the checkpoint's low-rank decay projection has
    kind: str = "gla"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values are expanded from one cached latent per token; every head's key has an
    unrotated part of `nope_dim` (from the latent) and a rotated part of `rot_dim` that all heads share."""
    hidden_size: int
    num_heads: int
    nope_dim: int
    rot_dim: int
    value_dim: int
    kv_rank: int
    softmax_scale: float
    window: int | None              # None -> all earlier keys
    position: RopeSpec | None       # rotation of the first `position.rotary_dim` dims of the rotated part
    norm_eps: float
    kind: str = "latent_attention"
    pairing: str = "halves"         # the rotation pairs column i with i + n/2 ("halves") or 2i with 2i + 1 ("neighbours")
    sink: bool = False              # a stored number per head joins the softmax's denominator as exp(sink_h)
    head_gate: bool = False         # a head's output is multiplied by sigmoid of a projection of the input, one number per head
    own_latents: bool = True        # False: no down-projection; the layer reads the latents another layer cached
                                    # (the schedule gives it that layer's cache, `writes_cache=False`)


@dataclass(frozen=True)
class DenseMLPSpec:
    """down(act(up(x))), no gate."""
    hidden_size: int
    intermediate_size: int
    activation: str = "gelu_tanh"
    kind: str = "dense_mlp"


@dataclass(frozen=True)
class RoutedMLPSpec:
    """Mixture of gated experts behind a router, with a choice correction, expert groups and identity experts.

    `score`: "softmax" over all router outputs, or "sigmoid" of each.  `expert`: "clamped" (g~ sigmoid(act_alpha g~)
    (u~ + 1) with gate and up clamped at `limit`) or "silu" (silu(g) u).  `weigh`: the chosen expert's weight multiplies
    its "output" or its "input".  `correction`: whether the checkpoint holds a correction of the choice.  `score` "softmax_chosen": the
    router's outputs themselves are ranked and the chosen experts' weights are the softmax over the chosen outputs alone; with it
    go `expert` "silu" weighted at the "output".  `router_bias`: the router's outputs get a stored bias.  `shared_size` > 0: one
    more expert of that size (of the routed experts' form) runs for every token with weight 1."""
    hidden_size: int
    expert_size: int
    num_experts: int
    num_identity: int
    top: int
    num_groups: int
    keep_groups: int
    route_scale: float
    limit: float
    act_alpha: float = 1.702
    score: str = "softmax"
    expert: str = "clamped"
    weigh: str = "output"
    correction: bool = True
    router_bias: bool = False
    shared_size: int = 0
    kind: str = "routed_mlp"


@dataclass(frozen=True)
class ClampedGLUSpec:
    """Dense gated feed-forward with clamped branches: down(g~ sigmoid(act_alpha g~) (u~ + 1)), g~ = min(gate, limit),
    u~ = clamp(up, -limit, limit)."""
    hidden_size: int
    intermediate_size: int
    limit: float
    act_alpha: float = 1.702
    kind: str = "clamped_glu"


@dataclass(frozen=True)
class GLUSpec:
    """Dense gated feed-forward down(act(gate(x)) * up(x)), act "gelu_tanh" or "silu"."""
    hidden_size: int
    intermediate_size: int
    activation: str = "gelu_tanh"
    kind: str = "glu"


@dataclass(frozen=True)
class DeltaRuleSpec:
    """Gated delta rule with a decay per key channel: q, k (`num_key_heads` heads of `key_dim`) and v (`num_heads` heads of
    `value_dim`) pass a short causal convolution of `conv_kernel` taps and silu; q and k become unit vectors per head
    (x / sqrt(|x|^2 + unit_eps), q also times key_dim^-1/2); per head S <- diag(g) S, u = b (v - S^T k), S <- S + k u^T,
    o = S^T q with g = exp(-exp(A_log) softplus(low-rank projection + dt_bias)) per key channel and b = sigmoid(.) per
    head; o is RMS-normed per head, times sigmoid of a low-rank gate, then the output projection."""
    hidden_size: int
    num_heads: int
    num_key_heads: int
    key_dim: int
    value_dim: int
    conv_kernel: int
    norm_eps: float
    unit_eps: float = 1e-6
    decay_rank: int | None = None      # None: whatever the checkpoint's low-rank decay projection has
    gate_rank: int | None = None       # the same for the low-rank output gate
    kind: str = "channel_delta"


@dataclass(frozen=True)
class SinkAttentionSpec:
    """Causal grouped-query attention without rotation: queries and keys RMS-normed per head (a weight each, shared by the
    heads), the query times 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) at position p (temp_every 0: no such
    factor); score = softmax_scale * (q . k) - slope_h * (i - j) with slope_h = 2^(-slope_span * (h + 1) / heads)
    (slope_span 0: no bias); with `sink` a stored number per head joins the softmax's denominator as exp(sink_h)."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    softmax_scale: float
    norm_eps: float
    temp_coef: float = 0.0
    temp_every: int = 0
    slope_span: float = 8.0
    sink: bool = True
    kind: str = "sink_attention"


@dataclass(frozen=True)
class ConvAttentionSpec:
    """Grouped-query attention over a sliding window whose values are its keys: q and k pass a short causal convolution per
    channel (`conv_kernel` taps, no activation); v is k as it leaves the convolution; q and k are then each RMS-normed over
    their whole row (all heads at once, a weight per column), rotated over neighbouring pairs of every head's first
    `position.rotary_dim` columns; scores times `softmax_scale`, position i sees j with 0 <= i - j < window (None: every
    j <= i); with `sink` a stored number per head joins the softmax's denominator; with `head_gate` a head's output is
    multiplied by sigmoid of a projection of the input."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    conv_kernel: int
    softmax_scale: float
    window: int | None
    position: RopeSpec | None
    norm_eps: float
    sink: bool = True
    head_gate: bool = True
    kind: str = "conv_attention"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """Gated delta rule with one decay per head: q, k (`num_key_heads` heads of `key_dim`) and v (`num_heads` heads of
    `value_dim`) pass a short causal convolution of `conv_kernel` taps and silu; q and k become unit vectors per head
    (x / sqrt(|x|^2 + unit_eps), q also times key_dim^-1/2); per head S <- g S, u = b (v - S^T k), S <- S + k u^T, o = S^T q
    with g = exp(-exp(A_log) softplus(projection + dt_bias)) and b = sigmoid(projection), one number per head each; o is
    RMS-normed per head (one weight for all heads), times silu of a gate projection, then the output projection."""
    hidden_size: int
    num_heads: int
    num_key_heads: int
    key_dim: int
    value_dim: int
    conv_kernel: int
    norm_eps: float
    unit_eps: float = 1e-6
    kind: str = "gated_delta"


@dataclass(frozen=True)
class LightningAttentionSpec:
    """Linear attention with one fixed decay per head: q, k, v = silu(projection); S <- decay_h S + k v^T, o = S^T q; the
    heads' outputs are RMS-normed together, times sigmoid(gate projection), then the output projection."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay: tuple[float, ...]
    norm_eps: float
    kind: str = "lightning_attention"


@dataclass(frozen=True)
class MixerPairSpec:
    """Two mixers side by side on the same input; the result is the sum of their outputs, each times its slot's
    `out_scale`.  At most one of them keeps keys and values."""
    left: Any          # MixerSlot
    right: Any         # MixerSlot
    kind: str = "mixer_pair"


@dataclass(frozen=True)
class MinGRUSpec:
    """A gated recurrence per channel whose gates read the current token only: S <- (1 - z) S + z c with z = sigmoid(.),
    c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0); output product over S * silu(gate)."""
    hidden_size: int
    width: int
    kind: str = "mingru"


@dataclass(frozen=True)
class PooledWindowAttentionSpec:
    """Grouped-query attention over a sliding window of tokens plus one pooled key/value (the mean) for every block of
    `pool` tokens that lies wholly behind the window; keys and values of different head sizes; queries and keys rotated
    over neighbouring pairs of their first `position.rotary_dim` dims, values rotated over all of theirs
    (`value_position`) and the summed values turned back by the query's position."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    softmax_scale: float
    window: int
    pool: int
    position: RopeSpec | None            # rotation of queries and keys
    value_position: RopeSpec | None      # rotation of the values (None: values are cached as they are)
    kind: str = "pooled_window_attention"


@dataclass(frozen=True)
class TokenSideSpec:
    """A per-layer input from the token itself: x <- x + RMSNorm(proj(gelu_tanh(gate x) * e)) with e the columns
    [offset, offset + dim) of the token's row of a second embedding table that all layers share."""
    hidden_size: int
    dim: int
    offset: int
    table_width: int
    vocab_size: int
    eps: float
    table_name: str = "side.embed"       # checkpoint name of the shared table, relative to the model


@dataclass(frozen=True)
class MixerSlot:
    """One mixer of a block: its spec, the checkpoint prefix of its tensors
    (relative to the block's prefix), and the scales applied to the normed
    input it reads and to the output it adds to the residual stream."""
    spec: Any
    name: str
    in_scale: float = 1.0
    out_scale: float = 1.0


@dataclass(frozen=True)
class BlockSpec:
    """Pre-norm block: norm -> mixers side by side on the same normed input ->
    their scaled sum joins the residual -> norm -> feed-forward."""
    prefix: str
    mixers: tuple[MixerSlot, ...]
    mixer_norm: NormSpec
    mixer_norm_name: str
    feed_forward: Any
    feed_forward_name: str
    feed_forward_norm: NormSpec
    feed_forward_norm_name: str
    kind: str = "prenorm_parallel"


@dataclass(frozen=True)
class PostNormBlockSpec:
    """Post-norm block on a 32-bit stream: x <- norm(skip_scale * x + mixer(x)), then, when it has a feed-forward,
    x <- norm(skip_scale * x + feed_forward(x))."""
    prefix: str
    mixer: MixerSlot
    mixer_norm: NormSpec
    mixer_norm_name: str
    feed_forward: Any                 # None: no feed-forward sublayer (and no second norm)
    feed_forward_name: str
    feed_forward_norm: NormSpec | None
    feed_forward_norm_name: str
    skip_scale: float = 1.0
    kind: str = "postnorm"


@dataclass(frozen=True)
class OutNormBlockSpec:
    """Block on a 32-bit stream whose norms sit on the sublayers' outputs alone: x <- x + norm1(mixer(x)), then, when it has a
    feed-forward, x <- x + norm2(feed_forward(x)).  The sublayers read the stream itself."""
    prefix: str
    mixer: MixerSlot
    mixer_norm: NormSpec
    mixer_norm_name: str
    feed_forward: Any                 # None: no feed-forward sublayer (and no second norm)
    feed_forward_name: str
    feed_forward_norm: NormSpec | None
    feed_forward_norm_name: str
    kind: str = "outnorm_stream"


@dataclass(frozen=True)
class StreamBlockSpec:
    """Pre-norm block on a 32-bit stream: x <- x + s1 * mixer(norm(x)); with a feed-forward x <- x + s2 * ff(norm(x))
    (s1, s2: a stored scale per channel, when `layer_scale`); then, with `side`, the token's side input."""
    prefix: str
    mixer: MixerSlot
    mixer_norm: NormSpec
    mixer_norm_name: str
    feed_forward: Any                 # None: no feed-forward sublayer (and no second norm or scale)
    feed_forward_name: str
    feed_forward_norm: NormSpec | None
    feed_forward_norm_name: str
    layer_scale: bool = False
    layer_scale_names: tuple[str, str] = ("ls1", "ls2")
    side: TokenSideSpec | None = None
    side_name: str = "side."
    kind: str = "prenorm_stream"


@dataclass(frozen=True)
class ParallelStreamBlockSpec:
    """Block on a 32-bit stream whose sublayers all read ONE norm's output: h = norm(x); x <- x + mixer(h) + feed_forward(h)
    (a block without a feed-forward adds the mixer alone)."""
    prefix: str
    mixer: MixerSlot
    norm: NormSpec
    norm_name: str
    feed_forward: Any                 # None: no feed-forward sublayer
    feed_forward_name: str
    kind: str = "parallel_stream"


@dataclass(frozen=True)
class StreamInputSpec:
    """x <- W [x ; x0] on a 32-bit stream, x0 the rows the stream began as (the embedding's output); W [width, 2 * width]
    is stored at the model's root under `name`."""
    hidden_size: int
    name: str


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  `layer` indexes `ModelSpec.layers` (a layer
    may appear in several entries: its weights then run more than once).
    `cache` names the cache layer this execution uses; by default every entry
    owns one.  An entry whose `cache` equals an earlier entry's and which has
    `writes_cache=False` reads that entry's keys/values instead of storing its own."""
    layer: int
    cache: int
    writes_cache: bool = True
    opens: int | None = None      # index into `ModelSpec.stream_inputs`: that input is applied right before this execution


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    embedding_name: str
    embedding_multiplier: float
    lm_head_name: str
    lm_head_multiplier: float
    tie_word_embeddings: bool
    final_norm: NormSpec
    final_norm_name: str
    layers: tuple[BlockSpec, ...]
    schedule: tuple[ScheduleEntry, ...] = field(default=())
    embedding_kind: str = "embedding"       # registry.EMBEDDINGS: built as cls(vocab_size, hidden_size, multiplier)
    lm_head_kind: str = "lm_head"           # registry.HEADS: built as cls(vocab_size, hidden_size, multiplier, tied_to)
    embedding_options: tuple[tuple[str, Any], ...] = ()    # further keyword arguments of the embedding's constructor
    stream_inputs: tuple[StreamInputSpec, ...] = ()         # see `ScheduleEntry.opens`

    def resolved_schedule(self) -> tuple[ScheduleEntry, ...]:
        if self.schedule:
            return self.schedule
        return tuple(ScheduleEntry(i, i) for i in range(len(self.layers)))
