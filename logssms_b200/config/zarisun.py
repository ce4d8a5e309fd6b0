"""Typed configuration of the Zarisun decoder: layers on a 32-bit stream whose norms sit on the sublayers' outputs
(x <- x + norm(mixer(x)), x <- x + norm(ff(x)); mixer and feed-forward read the stream itself).  A layer's mixer is
windowed attention whose values are its convolved keys (`attention`), a gated delta rule with one decay per head (`delta`),
or attention over cached latents (`latent_attention`), which may read the latents of an earlier layer (`kv_from`).  Both
attentions rotate neighbouring pairs with frequencies stretched by a ramp, have a sink per head and a sigmoid gate per
head.  Feed-forwards are dense gated layers (silu) or absent.  The output head is the embedding table times `logit_scale`.

config.json is nested: `vocab`, `width`, `norm.eps`, `logit_scale` and `layers`, a list whose entries give `type` (the
mixer), `mixer` (its sizes and constants) and `mlp` (the feed-forward, or null).  Every size and constant is read from there.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, require
from .specs import (ConvAttentionSpec, GatedDeltaSpec, GLUSpec, LatentAttentionSpec, MixerSlot, ModelSpec, NormSpec, OutNormBlockSpec,
                    RopeSpec, ScheduleEntry)

ARCHITECTURE = "Zarisun"
MIXER_TYPES = ("attention", "delta", "latent_attention")
UNIT_EPS = 1e-6           # inside the root of the delta rule's unit vectors
MAX_TAPS = 8              # the short convolutions' kernels take up to so many taps


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


def _rotation(m: Mapping[str, Any], where: str, limit: int) -> None:
    """Checks `rot` (None: no rotation): an even number of columns within the rotated part, a base, and a complete
    `scaling` if there is one."""
    rot = m.get("rot")
    if rot is None:
        return
    dims = _positive(rot, "dims", where + "rot.")
    if dims % 2 or dims > limit:
        raise ConfigError(f"{where}rot.dims must be even and at most {limit}")
    if require(rot, "base", float) <= 1.0:
        raise ConfigError(f"{where}rot.base must exceed 1")
    sc = rot.get("scaling")
    if sc is not None:
        for key in ("factor", "original", "fast", "slow"):
            if require(sc, key, float) <= 0:
                raise ConfigError(f"{where}rot.scaling.{key} must be positive")


def _rope(m: Mapping[str, Any], part_dim: int, max_position: int) -> RopeSpec | None:
    rot = m.get("rot")
    if rot is None:
        return None
    sc = rot.get("scaling")
    scaling = None if sc is None else tuple(sorted((k, float(sc[k])) for k in ("factor", "original", "fast", "slow")))
    return RopeSpec(head_dim=part_dim, rotary_dim=int(rot["dims"]), theta=float(rot["base"]), max_position=max_position,
                    scaling=scaling, kind="rope_ramp")


@dataclass(frozen=True)
class ZarisunConfig:
    raw: tuple                 # the config.json mapping, kept to write it back unchanged
    vocab_size: int
    hidden_size: int
    norm_eps: float
    logit_scale: float
    layers: tuple              # of (type, mixer mapping, mlp mapping or None), validated
    torch_dtype: str = "bfloat16"
    max_position_embeddings: int = 8192
    architectures: tuple[str, ...] = (ARCHITECTURE,)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZarisunConfig":
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks the list 'layers'")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            kind = require(layer, "type", str)
            mixer = _sub(layer, "mixer", where)
            mw = where + "mixer."
            if kind in ("attention", "delta"):
                heads, kv = _positive(mixer, "heads", mw), _positive(mixer, "kv_heads", mw)
                if heads % kv:
                    raise ConfigError(f"{mw}heads must be a multiple of kv_heads")
                dim, vdim = _positive(mixer, "dim", mw), _positive(mixer, "vdim", mw)
                if not 1 <= require(mixer, "conv", int) <= MAX_TAPS:
                    raise ConfigError(f"{mw}conv must lie within 1 .. {MAX_TAPS} taps")
                if kind == "attention":
                    if vdim != dim:
                        raise ConfigError(f"{mw}vdim must equal dim: the values of this attention are its keys")
                    require(mixer, "scale", float)
                    mask = mixer.get("mask")
                    if mask is not None:
                        _positive(mask, "size", mw + "mask.")
                    _rotation(mixer, mw, dim)
            elif kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "kv_rank"):
                    _positive(mixer, key, mw)
                rot_dim = require(mixer, "rot_dim", int)
                if rot_dim < 0 or rot_dim % 2:
                    raise ConfigError(f"{mw}rot_dim must be even and not negative")
                require(mixer, "scale", float)
                _rotation(mixer, mw, rot_dim)
                src = mixer.get("kv_from")
                if src is not None:
                    src = int(src)
                    if not 0 <= src < i or checked[src][0] != "latent_attention" or checked[src][1].get("kv_from") is not None:
                        raise ConfigError(f"{mw}kv_from must name an earlier latent_attention layer with latents of its own")
                    theirs = checked[src][1]
                    if (int(theirs["kv_rank"]), int(theirs["rot_dim"]), theirs.get("rot")) != (int(mixer["kv_rank"]), rot_dim, mixer.get("rot")):
                        raise ConfigError(f"{mw}kv_rank, rot_dim and rot must equal those of layer {src}, whose latents it reads")
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this architecture; known: {MIXER_TYPES}")
            mlp = layer.get("mlp")
            if mlp is not None:
                ff_kind = require(mlp, "kind", str)
                if ff_kind != "dense":
                    raise ConfigError(f"{where}mlp.kind {ff_kind!r} is not 'dense'")
                _positive(mlp, "ff", where + "mlp.")
            checked.append((kind, copy.deepcopy(dict(mixer)), None if mlp is None else copy.deepcopy(dict(mlp))))
        eps = require(_sub(raw, "norm", ""), "eps", float)
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        return cls(
            raw=tuple(sorted(copy.deepcopy(dict(raw)).items(), key=lambda kv: kv[0])),
            vocab_size=_positive(raw, "vocab", ""), hidden_size=_positive(raw, "width", ""), norm_eps=eps,
            logit_scale=float(raw.get("logit_scale", 1.0)), layers=tuple(checked),
            torch_dtype=str(raw.get("torch_dtype", "bfloat16")),
            max_position_embeddings=int(raw.get("max_position_embeddings", 8192)),
        )

    def __hash__(self):
        return hash((self.vocab_size, self.hidden_size, len(self.layers)))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        return copy.deepcopy(dict(self.raw))

    # ------------------------------------------------------------------ as parts
    def cache_layers(self) -> list[int]:
        """The cache layer of every layer: one of its own, but for a latent-attention layer with `kv_from`, which uses (and
        does not write) the cache layer of the layer it names."""
        own, nxt = [], 0
        for kind, m, _ in self.layers:
            if kind == "latent_attention" and m.get("kv_from") is not None:
                own.append(own[int(m["kv_from"])])
            else:
                own.append(nxt)
                nxt += 1
        return own

    def model_spec(self) -> ModelSpec:
        H, eps, far = self.hidden_size, self.norm_eps, self.max_position_embeddings
        blocks = []
        for i, (kind, m, mlp) in enumerate(self.layers):
            if kind == "attention":
                mask = m.get("mask")
                mixer = ConvAttentionSpec(hidden_size=H, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
                                          conv_kernel=int(m["conv"]), softmax_scale=float(m["scale"]),
                                          window=None if mask is None else int(mask["size"]), position=_rope(m, int(m["dim"]), far),
                                          norm_eps=eps, sink=True, head_gate=True)
            elif kind == "delta":
                mixer = GatedDeltaSpec(hidden_size=H, num_heads=int(m["heads"]), num_key_heads=int(m["kv_heads"]), key_dim=int(m["dim"]),
                                       value_dim=int(m["vdim"]), conv_kernel=int(m["conv"]), norm_eps=eps, unit_eps=UNIT_EPS)
            else:
                mixer = LatentAttentionSpec(hidden_size=H, num_heads=int(m["heads"]), nope_dim=int(m["dim"]), rot_dim=int(m["rot_dim"]),
                                            value_dim=int(m["vdim"]), kv_rank=int(m["kv_rank"]), softmax_scale=float(m["scale"]),
                                            window=None, position=_rope(m, int(m["rot_dim"]), far), norm_eps=eps, pairing="neighbours",
                                            sink=True, head_gate=True, own_latents=m.get("kv_from") is None)
            ff = None if mlp is None else GLUSpec(H, int(mlp["ff"]), "silu")
            norm = NormSpec(H, eps, kind="rmsnorm", param_name="")
            blocks.append(OutNormBlockSpec(prefix=f"l{i}.", mixer=MixerSlot(mixer, "mix."), mixer_norm=norm, mixer_norm_name="norm1",
                                           feed_forward=ff, feed_forward_name="mlp.", feed_forward_norm=None if ff is None else norm,
                                           feed_forward_norm_name="norm2"))
        caches = self.cache_layers()
        schedule = tuple(ScheduleEntry(i, c, writes_cache=caches.index(c) == i) for i, c in enumerate(caches))
        return ModelSpec(
            vocab_size=self.vocab_size, hidden_size=H, embedding_name="", embedding_multiplier=1.0,
            lm_head_name="head.", lm_head_multiplier=self.logit_scale, tie_word_embeddings=True,
            final_norm=NormSpec(H, eps, kind="rmsnorm", param_name=""), final_norm_name="final.norm", layers=tuple(blocks),
            schedule=schedule, embedding_kind="stream_embedding", lm_head_kind="lm_head",
        )
