"""Typed configuration of the Pupopel decoder: layers on a 32-bit stream whose mixer and feed-forward both read the one
norm of the layer (its weight stored around zero) and join the stream together; a layer's mixer is a gated delta rule with
a decay per key channel, or a pair of mixers side by side (softmax attention with a bias by distance and a sink, and
linear attention with a fixed decay per head); feed-forwards are dense gated layers or mixtures of experts with a shared
expert; a run of layers may be looped with the same weights, each pass opening with a product over the stream and the
embedding's output.

config.json is nested: `vocab`, `width`, `norm.eps`, `loop` (start, stop, times) and `layers`, a list whose entries give
`type` (the mixer), `mixer` (its sizes and constants) and `mlp` (the feed-forward, or null).  Every size and constant is
read from there; the ranks of the delta rule's two low-rank projections are the checkpoint's (the optional keys
`decay_rank` and `gate_rank` of its `mixer` only tell the random-weights writer what to draw).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, require
from .specs import (DeltaRuleSpec, GLUSpec, LightningAttentionSpec, MixerPairSpec, MixerSlot, ModelSpec, NormSpec,
                    ParallelStreamBlockSpec, RoutedMLPSpec, ScheduleEntry, SinkAttentionSpec, StreamInputSpec)

ARCHITECTURE = "Pupopel"
MIXER_TYPES = ("channel_delta", "parallel")
SLOPE_SPAN = 8.0          # the bias slopes of a softmax-attention head: 2^(-SLOPE_SPAN * (h + 1) / heads)
UNIT_EPS = 1e-6           # inside the root of the delta rule's unit vectors


def _sub(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"config.json lacks the mapping {where}{key!r}")
    return value


def _positive(raw: Mapping[str, Any], key: str, where: str) -> int:
    value = require(raw, key, int)
    if value < 1:
        raise ConfigError(f"{where}{key} must be positive")
    return value


def _heads(m: Mapping[str, Any], where: str) -> None:
    heads, kv = _positive(m, "heads", where), _positive(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"{where}heads must be a multiple of kv_heads")
    _positive(m, "dim", where)
    _positive(m, "vdim", where)


@dataclass(frozen=True)
class PupopelConfig:
    raw: tuple                 # the config.json mapping, kept to write it back unchanged
    vocab_size: int
    hidden_size: int
    norm_eps: float
    loop: tuple[int, int, int] | None   # start, stop, times; None: no loop (and no product that opens a pass)
    layers: tuple              # of (type, mixer mapping, mlp mapping or None), validated
    torch_dtype: str = "bfloat16"
    max_position_embeddings: int = 8192
    architectures: tuple[str, ...] = (ARCHITECTURE,)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "PupopelConfig":
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks the list 'layers'")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            kind = require(layer, "type", str)
            mixer = _sub(layer, "mixer", where)
            if kind == "channel_delta":
                _heads(mixer, where + "mixer.")
                if not 1 <= require(mixer, "conv", int) <= 8:
                    raise ConfigError(f"{where}mixer.conv must lie within 1 .. 8 taps")
            elif kind == "parallel":
                left = _sub(mixer, "left", where + "mixer.")
                _heads(left, where + "mixer.left.")
                require(left, "scale", float)
                temp = left.get("q_temp")
                if temp is not None:
                    require(temp, "coef", float)
                    _positive(temp, "every", where + "mixer.left.q_temp.")
                right = _sub(mixer, "right", where + "mixer.")
                heads = _positive(right, "heads", where + "mixer.right.")
                _positive(right, "dim", where + "mixer.right.")
                _positive(right, "vdim", where + "mixer.right.")
                decay = right.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != heads or not all(0.0 < float(d) <= 1.0 for d in decay):
                    raise ConfigError(f"{where}mixer.right.decay must list one decay within (0, 1] per head")
                require(mixer, "left_scale", float)
                require(mixer, "right_scale", float)
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this architecture; known: {MIXER_TYPES}")
            mlp = layer.get("mlp")
            if mlp is not None:
                ff_kind = require(mlp, "kind", str)
                if ff_kind == "dense":
                    _positive(mlp, "ff", where + "mlp.")
                elif ff_kind == "moe":
                    _positive(_sub(mlp, "expert", where + "mlp."), "ff", where + "mlp.expert.")
                    router = _sub(mlp, "router", where + "mlp.")
                    if not 1 <= require(router, "top", int) <= _positive(router, "experts", where + "mlp.router."):
                        raise ConfigError(f"{where}mlp.router.top must lie within 1 .. experts")
                    if mlp.get("shared") is not None:
                        _positive(mlp["shared"], "ff", where + "mlp.shared.")
                else:
                    raise ConfigError(f"{where}mlp.kind {ff_kind!r} is neither 'dense' nor 'moe'")
            checked.append((kind, copy.deepcopy(dict(mixer)), None if mlp is None else copy.deepcopy(dict(mlp))))
        eps = require(_sub(raw, "norm", ""), "eps", float)
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        loop = raw.get("loop")
        bounds = None
        if loop is not None:
            bounds = (require(loop, "start", int), require(loop, "stop", int), require(loop, "times", int))
            if not 0 <= bounds[0] <= bounds[1] <= len(checked) or bounds[2] < 1:
                raise ConfigError("loop must name a range of layers start <= stop and times >= 1")
        return cls(
            raw=tuple(sorted(copy.deepcopy(dict(raw)).items(), key=lambda kv: kv[0])),
            vocab_size=_positive(raw, "vocab", ""), hidden_size=_positive(raw, "width", ""), norm_eps=eps,
            loop=bounds, layers=tuple(checked), torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
            max_position_embeddings=int(raw.get("max_position_embeddings", 8192)),
        )

    def __hash__(self):
        return hash((self.vocab_size, self.hidden_size, len(self.layers)))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        return copy.deepcopy(dict(self.raw))

    # ------------------------------------------------------------------ as parts
    def layer_runs(self) -> list[tuple[int, bool]]:
        """(layer, does a pass of the loop open here) in the order the layers run: the looped range `times` times in a row,
        between what lies before and after."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        inner = [(i, i == start) for i in range(start, stop)]
        return [(i, False) for i in range(start)] + inner * times + [(i, False) for i in range(stop, n)]

    def model_spec(self) -> ModelSpec:
        H, eps = self.hidden_size, self.norm_eps
        norm = NormSpec(H, eps, kind="rmsnorm", param_name="", offset=1.0)
        blocks = []
        for i, (kind, m, mlp) in enumerate(self.layers):
            if kind == "channel_delta":
                mixer = DeltaRuleSpec(hidden_size=H, num_heads=int(m["heads"]), num_key_heads=int(m["kv_heads"]), key_dim=int(m["dim"]),
                                      value_dim=int(m["vdim"]), conv_kernel=int(m["conv"]), norm_eps=eps, unit_eps=UNIT_EPS,
                                      decay_rank=m.get("decay_rank"), gate_rank=m.get("gate_rank"))
                slot = MixerSlot(mixer, "mix.")
            else:
                L, R = m["left"], m["right"]
                temp = L.get("q_temp") or {"coef": 0.0, "every": 0}
                left = SinkAttentionSpec(hidden_size=H, num_heads=int(L["heads"]), num_kv_heads=int(L["kv_heads"]), head_dim=int(L["dim"]),
                                         value_dim=int(L["vdim"]), softmax_scale=float(L["scale"]), norm_eps=eps,
                                         temp_coef=float(temp["coef"]), temp_every=int(temp["every"]), slope_span=SLOPE_SPAN, sink=True)
                right = LightningAttentionSpec(hidden_size=H, num_heads=int(R["heads"]), key_dim=int(R["dim"]), value_dim=int(R["vdim"]),
                                               decay=tuple(float(d) for d in R["decay"]), norm_eps=eps)
                slot = MixerSlot(MixerPairSpec(MixerSlot(left, "left.", out_scale=float(m["left_scale"])),
                                               MixerSlot(right, "right.", out_scale=float(m["right_scale"]))), "mix.")
            ff = None
            if mlp is not None and mlp["kind"] == "dense":
                ff = GLUSpec(H, int(mlp["ff"]), "gelu_tanh")
            elif mlp is not None:
                r = mlp["router"]
                shared = mlp.get("shared")
                ff = RoutedMLPSpec(hidden_size=H, expert_size=int(mlp["expert"]["ff"]), num_experts=int(r["experts"]),
                                   num_identity=0, top=int(r["top"]), num_groups=1, keep_groups=1, route_scale=1.0, limit=0.0,
                                   score="softmax_chosen", expert="silu", weigh="output", correction=False, router_bias=True,
                                   shared_size=0 if shared is None else int(shared["ff"]))
            blocks.append(ParallelStreamBlockSpec(prefix=f"l{i}.", mixer=slot, norm=norm, norm_name="norm1", feed_forward=ff,
                                                  feed_forward_name="mlp."))
        schedule = tuple(ScheduleEntry(layer, run, opens=0 if opens else None) for run, (layer, opens) in enumerate(self.layer_runs()))
        return ModelSpec(
            vocab_size=self.vocab_size, hidden_size=H, embedding_name="", embedding_multiplier=1.0,
            lm_head_name="head", lm_head_multiplier=1.0, tie_word_embeddings=False,
            final_norm=norm, final_norm_name="final.norm", layers=tuple(blocks), schedule=schedule,
            embedding_kind="stream_embedding", lm_head_kind="lm_head_bare",
            stream_inputs=() if self.loop is None else (StreamInputSpec(H, "loop.in"),),
        )
