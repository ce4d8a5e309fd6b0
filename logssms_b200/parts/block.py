"""How a layer's parts are arranged."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..ops.profiler import PROFILER, nvtx_range
from ..registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from .base import Part


@BLOCKS.register("prenorm_parallel")
class PreNormParallelBlock(Part):
    """norm -> one or two mixers side by side on the same normed input (each with its own input
    scale) -> their scaled sum joins the residual inside the next norm -> feed-forward.  The
    feed-forward's output joins the residual inside the NEXT block's first norm (or the final
    norm), so a block returns (x, residual) with x not yet added.

    With two mixers this is Falcon-H1's layer (python/logssms/models/falcon_h1.py:152-185);
    with one mixer and unit scales it is the plain sequential pre-norm decoder layer."""

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if not 1 <= len(spec.mixers) <= 2:
            raise ValueError("prenorm_parallel blocks take one or two mixers")
        self.spec = spec
        self.mixers = [MIXERS.get(m.spec.kind)(m.spec, perturb_init=perturb_init, shared=shared) for m in spec.mixers]
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, perturb_init)
        self.ff_norm = NORMS.get(spec.feed_forward_norm.kind)(spec.feed_forward_norm, perturb_init)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, perturb_init=perturb_init,
                                                                      shared=shared)

    @property
    def input_norm(self):
        """The norm that reads this block's input: the block before may hand it rows in the form it takes
        (`takes_summed_rows`, `takes_scaled_rows`).  A block kind that names none is handed plain tensors."""
        return self.mixer_norm

    def children(self):
        s = self.spec
        kids = {s.mixer_norm_name: self.mixer_norm, s.feed_forward_norm_name: self.ff_norm,
                s.feed_forward_name: self.feed_forward}
        for slot, mixer in zip(s.mixers, self.mixers):
            kids[slot.name] = mixer
        return kids

    def cache_needs(self):
        """Needs of all mixers of this block, merged into one cache layer."""
        from ..cache import CacheNeeds
        kv, states = None, []
        for mixer in self.mixers:
            need = mixer.cache_needs()
            if need.kv is not None:
                if kv is not None:
                    raise ValueError("a block holds at most one mixer with a key/value cache")
                kv = need.kv
            states.extend(need.states)
        names = [s.name for s in states]
        if len(set(names)) != len(names):
            raise ValueError(f"state names clash inside one block: {names}")
        return CacheNeeds(kv=kv, states=tuple(states))

    def setup(self, rt) -> None:
        for part in (*self.mixers, self.feed_forward):
            part.setup(rt)

    def forward(self, x: torch.Tensor, residual, ctx, cache_layer: int, writes_cache: bool = True):
        if PROFILER.nvtx and not getattr(self, "_ranged", False):
            # named ranges around the parts, put on once (only when ranges are switched on)
            self._ranged = True
            for part, label in [*((m, s.spec.kind) for m, s in zip(self.mixers, self.spec.mixers)),
                                (self.feed_forward, self.spec.feed_forward.kind),
                                (self.mixer_norm, "mixer norm"), (self.ff_norm, "feed-forward norm")]:
                inner = part.forward

                def ranged(*args, _inner=inner, _label=label, **kwargs):
                    with nvtx_range(_label):
                        return _inner(*args, **kwargs)
                part.forward = ranged
        slots = self.spec.mixers
        # parts whose first step is a product say so (`takes_normed_rows`): the norm in front of them can then
        # ride in that product's prologue (decode steps: fewer dependent launches)
        defer_mix = {"defer": True} if (getattr(self.mixer_norm, "can_defer", False)
                                         and all(getattr(m, "takes_normed_rows", False) for m in self.mixers)) else {}
        defer_ff = {"defer": True} if (getattr(self.ff_norm, "can_defer", False)
                                       and getattr(self.feed_forward, "takes_normed_rows", False)) else {}
        ins, residual = self.mixer_norm.forward(x, residual, out_scales=tuple(m.in_scale for m in slots), **defer_mix)
        # Where the norm in front of the feed-forward is deferred anyway, the first mixer's last product may join the
        # residual stream in its epilogue (`joins_residual`): it then returns `SummedRows`, the norm has nothing left to
        # read but those, and the feed-forward's product norms its own columns without a pass over whole rows.
        join_mix = bool(defer_ff) and getattr(self.mixers[0], "joins_residual", False) \
            and getattr(self.ff_norm, "takes_summed_rows", False) and isinstance(ins[0], K.NormedRows) \
            and (len(slots) == 2 or slots[0].out_scale == 1.0)
        in_scales = (slots[0].out_scale, slots[1].out_scale) if len(slots) == 2 else (slots[0].out_scale, 1.0)
        side = ctx.extras.get("side_stream") if len(self.mixers) == 2 else None
        if side is None:
            if join_mix:
                rest = [mixer.forward(inp, ctx, cache_layer, writes_cache) for mixer, inp in zip(self.mixers[1:], ins[1:])]
                first = self.mixers[0].forward(ins[0], ctx, cache_layer, writes_cache,
                                               join=K.ResidualJoin(residual, rest[0] if rest else None, in_scales))
                outs = [first, *rest]
            else:
                outs = [mixer.forward(inp, ctx, cache_layer, writes_cache) for mixer, inp in zip(self.mixers, ins)]
        else:
            # Inside a graph capture the two mixers go to two streams, so that the graph may run their
            # kernels side by side (each alone leaves most of the 148 SMs idle at small batch).
            main = torch.cuda.current_stream()
            fork = torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                second = self.mixers[1].forward(ins[1], ctx, cache_layer, writes_cache)
                join = torch.cuda.Event()
                join.record(side)
            if join_mix:
                def other_branch():
                    main.wait_event(join)                     # called by the first mixer right before its last product
                    return second
                first = self.mixers[0].forward(ins[0], ctx, cache_layer, writes_cache,
                                               join=K.ResidualJoin(residual, other_branch, in_scales))
                if not isinstance(first, K.SummedRows):
                    main.wait_event(join)
            else:
                first = self.mixers[0].forward(ins[0], ctx, cache_layer, writes_cache)
                main.wait_event(join)
            outs = [first, second]
        next_join = bool(ctx.extras.get("next_norm_takes_summed")) and getattr(self.feed_forward, "joins_residual", False)
        if isinstance(outs[0], K.SummedRows):
            (h,), residual = self.ff_norm.forward(outs[0], None, **defer_ff)
        elif len(outs) == 2:
            (h,), residual = self.ff_norm.forward(outs[0], residual, other=outs[1],
                                                  in_scales=(slots[0].out_scale, slots[1].out_scale), **defer_ff)
        else:
            if slots[0].out_scale != 1.0:
                outs[0] = K.scale(outs[0], slots[0].out_scale)
            (h,), residual = self.ff_norm.forward(outs[0], residual, **defer_ff)
        if next_join and isinstance(h, K.NormedRows):
            # the same at the feed-forward's last product, for the norm of the next layer
            out = self.feed_forward.forward(h, join=K.ResidualJoin(residual))
            return (out, None) if isinstance(out, K.SummedRows) else (out, residual)
        if ctx.extras.get("next_norm_takes_scaled") and getattr(self.feed_forward, "can_lazy_scale", False):
            # the norm that reads the output next applies the feed-forward's output multiplier while it loads it
            return self.feed_forward.forward(h, lazy_scale=True), residual
        return self.feed_forward.forward(h), residual


@BLOCKS.register("postnorm")
class PostNormBlock(Part):
    """x <- norm1(skip_scale * x + mixer(x)); then, with a feed-forward, x <- norm2(skip_scale * x + ff(x)).

    The stream x is 32-bit whatever the activation dtype (`K.StreamRows`): the sum and the norm are made in 32-bit by
    one kernel, which also leaves the copy rounded to the activation dtype that the next sublayer's products read.  A
    block returns (stream, None): nothing is left to be added."""
    input_norm = None            # no norm reads this block's input: it is handed the stream as it is

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        m = spec.mixer
        if m.in_scale != 1.0 or m.out_scale != 1.0:
            raise ValueError("postnorm blocks take a mixer without input or output scales")
        self.mixer = MIXERS.get(m.spec.kind)(m.spec, perturb_init=perturb_init, shared=shared)
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, perturb_init)
        self.feed_forward = self.ff_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, perturb_init=perturb_init,
                                                                          shared=shared)
            self.ff_norm = NORMS.get(spec.feed_forward_norm.kind)(spec.feed_forward_norm, perturb_init)
        for norm in (self.mixer_norm, self.ff_norm):
            if norm is not None and not hasattr(norm, "post"):
                raise ValueError("postnorm blocks need norms with a post-norm form (`post`)")

    def children(self):
        s = self.spec
        kids = {s.mixer_norm_name: self.mixer_norm, s.mixer.name: self.mixer}
        if self.feed_forward is not None:
            kids[s.feed_forward_norm_name] = self.ff_norm
            kids[s.feed_forward_name] = self.feed_forward
        return kids

    def cache_needs(self):
        return self.mixer.cache_needs()

    def setup(self, rt) -> None:
        self.mixer.setup(rt)
        if self.feed_forward is not None:
            self.feed_forward.setup(rt)

    def forward(self, x, residual, ctx, cache_layer: int, writes_cache: bool = True):
        if not isinstance(x, K.StreamRows) or residual is not None:
            raise ValueError("a postnorm block takes a 32-bit stream (`StreamRows`), as its embedding or the block before leaves it")
        skip = self.spec.skip_scale
        with nvtx_range(self.spec.mixer.spec.kind):
            y = self.mixer.forward(x.act, ctx, cache_layer, writes_cache)
        x = self.mixer_norm.post(x, y, skip)
        if self.feed_forward is not None:
            with nvtx_range(self.spec.feed_forward.kind):
                y = self.feed_forward.forward(x.act)
            if isinstance(y, tuple):          # (rows, rows to add with a weight per row): the norm's kernel adds them
                y, extra, row_scale = y
                x = self.ff_norm.post(x, y, skip, extra=extra, row_scale=row_scale)
            else:
                x = self.ff_norm.post(x, y, skip)
        return x, None


@BLOCKS.register("outnorm_stream")
class OutNormStreamBlock(Part):
    """x <- x + norm1(mixer(x)); then, with a feed-forward, x <- x + norm2(ff(x)): the norms sit on the sublayers' outputs
    alone, and the sublayers read the stream itself.

    The stream x is 32-bit whatever the activation dtype (`K.StreamRows`); the sublayers read its copy rounded to the
    activation dtype.  One kernel besides the sublayers' own per sublayer: the output's root mean square, the norm's weight, the
    sum into the stream (all 32-bit) and the rounded copy that the next sublayer reads (`K.stream_add_norm` with `unit_eps`)."""
    input_norm = None            # no norm reads this block's input: it is handed the stream as it is
    kernels = ("stream_layer",)

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        m = spec.mixer
        if m.in_scale != 1.0 or m.out_scale != 1.0:
            raise ValueError("outnorm_stream blocks take a mixer without input or output scales")
        self.mixer = MIXERS.get(m.spec.kind)(m.spec, perturb_init=perturb_init, shared=shared)
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, perturb_init)
        self.feed_forward = self.ff_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, perturb_init=perturb_init,
                                                                          shared=shared)
            self.ff_norm = NORMS.get(spec.feed_forward_norm.kind)(spec.feed_forward_norm, perturb_init)
        for norm in (self.mixer_norm, self.ff_norm):
            if norm is not None and getattr(norm, "norm_kind", None) != "rmsnorm":
                raise ValueError("outnorm_stream blocks norm their sublayers' outputs by root mean square (`rmsnorm`)")

    def children(self):
        s = self.spec
        kids = {s.mixer_norm_name: self.mixer_norm, s.mixer.name: self.mixer}
        if self.feed_forward is not None:
            kids[s.feed_forward_norm_name] = self.ff_norm
            kids[s.feed_forward_name] = self.feed_forward
        return kids

    def cache_needs(self):
        return self.mixer.cache_needs()

    def setup(self, rt) -> None:
        self.mixer.setup(rt)
        if self.feed_forward is not None:
            self.feed_forward.setup(rt)

    def forward(self, x, residual, ctx, cache_layer: int, writes_cache: bool = True):
        if not isinstance(x, K.StreamRows) or residual is not None:
            raise ValueError("an outnorm_stream block takes a 32-bit stream (`StreamRows`), as its embedding or the block before leaves it")
        act = x.act.dtype
        stream, h = x.f32, x.act
        if h.shape != stream.shape:                    # the block before left no rounded copy
            _, h = K.stream_add_norm(stream, None, None, None, 0.0, "none", act)
        with nvtx_range(self.spec.mixer.spec.kind):
            y = self.mixer.forward(h, ctx, cache_layer, writes_cache)
        n = self.mixer_norm
        _, h = K.stream_add_norm(stream, y, n.weight, None, 0.0, "none", act, unit_eps=n.eps)
        if self.feed_forward is not None:
            with nvtx_range(self.spec.feed_forward.kind):
                y = self.feed_forward.forward(h)
            n = self.ff_norm
            _, h = K.stream_add_norm(stream, y, n.weight, None, 0.0, "none", act, unit_eps=n.eps)
        return K.StreamRows(stream, h), None


class SharedTable(Part):
    """A table stored once at the model's root that several layers read (each a slice of every row)."""

    def __init__(self, name: str, shape: tuple[int, int], std: float = 1.0):
        self.name, self.shape, self.std = name, tuple(shape), std
        self.table: torch.Tensor | None = None

    def param_specs(self):
        from .base import MATRIX, ParamSpec, normal_init
        return {self.name: ParamSpec(self.shape, MATRIX, normal_init(self.std))}

    def bind(self, t):
        self.table = t[self.name]


class TokenSideInput(Part):
    """A layer's input from the token itself: x <- x + RMSNorm(proj (gelu_tanh(gate x) * e)) * norm, where e are this
    layer's `dim` columns of the token's row of a side table that all layers share (one tensor at the model's root).
    It runs inside the kernel that closes the layer (`K.stream_side`); in steps of many tokens of a bfloat16 engine the two
    small products go to the library between three light kernels.  Tensors: gate [dim, width], proj [width, dim],
    norm [width]; the table under `spec.table_name`."""
    kernels = ("stream_layer", "linear_skinny", "gemm_tcgen05")
    FUSED_MAX_ROWS = 128      # up to so many tokens one kernel does it all; beyond, the products go to the library

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        from .base import MATRIX, VECTOR, ParamSpec, normal_init, ones_init
        self.spec = spec
        self._specs = {"gate": ParamSpec((spec.dim, spec.hidden_size), MATRIX, normal_init(spec.hidden_size ** -0.5)),
                       "proj": ParamSpec((spec.hidden_size, spec.dim), MATRIX, normal_init(spec.dim ** -0.5)),
                       "norm": ParamSpec((spec.hidden_size,), VECTOR, ones_init(0.1 if perturb_init else 0.0))}
        prefix, _, name = spec.table_name.rpartition(".")
        prefix = prefix + "." if prefix else ""
        parts = shared.setdefault("model_parts", {}) if shared is not None else {}
        table = parts.get(prefix)
        if table is None:
            table = parts[prefix] = SharedTable(name, (spec.vocab_size, spec.table_width))
        elif not isinstance(table, SharedTable) or table.name != name or table.shape != (spec.vocab_size, spec.table_width):
            raise ValueError(f"the layers disagree on the side table {spec.table_name!r}")
        self.shared_table = table
        self.gate = self.proj = self.proj_t = self.norm = None

    def param_specs(self):
        return dict(self._specs)

    def bind(self, t):
        self.gate, self.proj, self.proj_t, self.norm = t["gate"], t["proj"], t["proj"].t().contiguous(), t["norm"]

    def close(self, x_f32, y, channel_scale, ids, next_norm, act_dtype):
        """x += channel_scale * y (y may be None), the side input, and the norm that follows; (x, normed or None)."""
        s = self.spec
        nw, neps, nkind = (None, 0.0, "layernorm") if next_norm is None else (next_norm.weight, next_norm.eps, next_norm.norm_kind)
        if x_f32.shape[0] > self.FUSED_MAX_ROWS and act_dtype == torch.bfloat16:
            # many tokens: the two small products on the tensor cores (the library), three light kernels around them
            _, rounded = K.stream_add_norm(x_f32, y, channel_scale, None, 0.0, "none", act_dtype)
            a = K.side_gate(K.linear(rounded, self.gate), ids, self.shared_table.table, s.offset)
            return K.stream_add_norm(x_f32, K.linear(a, self.proj), self.norm, nw, neps, nkind, act_dtype, unit_eps=s.eps)
        return K.stream_side(x_f32, y, channel_scale, ids, self.shared_table.table, s.offset, self.gate, self.proj_t, self.norm,
                             s.eps, nw, neps, nkind, act_dtype)


@BLOCKS.register("prenorm_stream")
class PreNormStreamBlock(Part):
    """Pre-norm block on a 32-bit stream (`K.StreamRows`): x <- x + s1 * mixer(norm1(x)); with a feed-forward
    x <- x + s2 * ff(norm2(x)); with a side input x <- x + side(x, token).  s1, s2 are stored scales per channel
    (`layer_scale`).  Every sum and norm is 32-bit; the sublayers read the normed rows in the activation dtype.

    Three kernels besides the sublayers' own: the mixer's output joins the stream and norm2 reads it in one
    (`K.stream_add_norm`); the feed-forward's output joins, the side input is added and the NEXT block's first norm
    reads the result in one (`K.stream_side`); norm1 runs alone only where the block before could not do it."""

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        m = spec.mixer
        if m.in_scale != 1.0 or m.out_scale != 1.0:
            raise ValueError("prenorm_stream blocks take a mixer without input or output multipliers")
        self.mixer = MIXERS.get(m.spec.kind)(m.spec, perturb_init=perturb_init, shared=shared)
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, perturb_init)
        self.feed_forward = self.ff_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, perturb_init=perturb_init,
                                                                          shared=shared)
            self.ff_norm = NORMS.get(spec.feed_forward_norm.kind)(spec.feed_forward_norm, perturb_init)
        for norm in (self.mixer_norm, self.ff_norm):
            if norm is not None and not hasattr(norm, "norm_kind"):
                raise ValueError("prenorm_stream blocks need norms with a form on a 32-bit stream (`norm_kind`)")
        self.side = None if spec.side is None else TokenSideInput(spec.side, perturb_init, shared)
        self._jitter = 0.3 if perturb_init else 0.0
        self.scale_mixer = self.scale_ff = None

    @property
    def input_norm(self):
        return self.mixer_norm

    def param_specs(self):
        from .base import VECTOR, ParamSpec, ones_init
        if not self.spec.layer_scale:
            return {}
        H = self.spec.mixer_norm.size
        names = self.spec.layer_scale_names[:2 if self.feed_forward is not None else 1]
        return {n: ParamSpec((H,), VECTOR, ones_init(self._jitter)) for n in names}

    def bind(self, t):
        names = self.spec.layer_scale_names
        self.scale_mixer, self.scale_ff = t.get(names[0]), t.get(names[1])

    def children(self):
        s = self.spec
        kids = {s.mixer_norm_name: self.mixer_norm, s.mixer.name: self.mixer}
        if self.feed_forward is not None:
            kids[s.feed_forward_norm_name] = self.ff_norm
            kids[s.feed_forward_name] = self.feed_forward
        if self.side is not None:
            kids[s.side_name] = self.side
        return kids

    def cache_needs(self):
        return self.mixer.cache_needs()

    def setup(self, rt) -> None:
        self.mixer.setup(rt)
        if self.feed_forward is not None:
            self.feed_forward.setup(rt)

    def forward(self, x, residual, ctx, cache_layer: int, writes_cache: bool = True):
        if not isinstance(x, K.StreamRows) or residual is not None:
            raise ValueError("a prenorm_stream block takes a 32-bit stream (`StreamRows`), as its embedding or the block before leaves it")
        act = x.act.dtype
        stream = x.f32
        if x.normed_by is self.mixer_norm:
            h = x.act
        else:
            _, h = K.stream_add_norm(stream, None, None, self.mixer_norm.weight, self.mixer_norm.eps, self.mixer_norm.norm_kind, act)
        with nvtx_range(self.spec.mixer.spec.kind):
            y = self.mixer.forward(h, ctx, cache_layer, writes_cache)
        scale = self.scale_mixer
        if self.feed_forward is not None:
            _, h = K.stream_add_norm(stream, y, scale, self.ff_norm.weight, self.ff_norm.eps, self.ff_norm.norm_kind, act)
            with nvtx_range(self.spec.feed_forward.kind):
                y = self.feed_forward.forward(h)
            scale = self.scale_ff
        # what is left to join the stream (y with its scale) joins in the kernel that closes the block
        nxt = ctx.extras.get("next_input_norm")
        nxt = nxt if hasattr(nxt, "norm_kind") else None
        if self.side is not None:
            _, h = self.side.close(stream, y, scale, ctx.token_ids, nxt, act)
        elif nxt is not None:
            _, h = K.stream_add_norm(stream, y, scale, nxt.weight, nxt.eps, nxt.norm_kind, act)
        else:
            K.stream_add_norm(stream, y, scale, None, 0.0, "layernorm", act)
            h = None
        if h is None:
            return K.StreamRows(stream, x.act[:0]), None
        return K.StreamRows(stream, h, normed_by=nxt), None


class StreamInput(Part):
    """x <- W [x ; x0] on a 32-bit stream: x0 are the rows the stream began as (the embedding's output, in the activation
    dtype), W [width, 2 * width] is stored at the model's root.  The product reads the stream rounded to the activation
    dtype beside x0 (one small kernel lays them side by side) and its sums are the new stream, unrounded."""
    kernels = ("stream_layer", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False):
        self.spec = spec
        self.weight = None

    def param_specs(self):
        from .base import MATRIX, ParamSpec, normal_init
        H = self.spec.hidden_size
        return {"": ParamSpec((H, 2 * H), MATRIX, normal_init((2 * H) ** -0.5 * 1.4))}

    def bind(self, t):
        self.weight = t[""]

    def forward(self, x, x0: torch.Tensor):
        if not isinstance(x, K.StreamRows):
            raise ValueError("a stream input mixes a 32-bit stream (`StreamRows`) with the rows it began as")
        y = K.linear(K.stream_pair_rows(x.f32, x0), self.weight, out_f32=True)
        return K.StreamRows(y, x0[:0])


def _addends(y, scale: float = 1.0) -> list:
    """What a sublayer handed back, as a list of (rows, scale): a mixer of several branches hands back such a list itself."""
    if isinstance(y, list):
        return [(t, s * scale) for t, s in y]
    return [(y, scale)]


@BLOCKS.register("parallel_stream")
class ParallelStreamBlock(Part):
    """Block on a 32-bit stream (`K.StreamRows`) whose sublayers all read ONE norm: h = norm(x); x <- x + mixer(h) + ff(h).
    The sum and the norm are 32-bit; the sublayers read h in the activation dtype.  One kernel besides the sublayers' own:
    all their outputs (a mixer of several branches hands back several, each with its scale) join the stream and the NEXT
    block's norm reads the result in one (`K.stream_add_many`); the block's own norm runs alone only where the block
    before could not do it (the first layer, and right behind a product over the stream)."""

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        m = spec.mixer
        if m.in_scale != 1.0:
            raise ValueError("parallel_stream blocks take a mixer without an input multiplier")
        self.mixer = MIXERS.get(m.spec.kind)(m.spec, perturb_init=perturb_init, shared=shared)
        self.norm = NORMS.get(spec.norm.kind)(spec.norm, perturb_init)
        if not hasattr(self.norm, "norm_kind"):
            raise ValueError("parallel_stream blocks need a norm with a form on a 32-bit stream (`norm_kind`)")
        self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, perturb_init=perturb_init, shared=shared)

    @property
    def input_norm(self):
        return self.norm

    def children(self):
        s = self.spec
        kids = {s.norm_name: self.norm, s.mixer.name: self.mixer}
        if self.feed_forward is not None:
            kids[s.feed_forward_name] = self.feed_forward
        return kids

    def cache_needs(self):
        return self.mixer.cache_needs()

    def setup(self, rt) -> None:
        self.mixer.setup(rt)
        if self.feed_forward is not None:
            self.feed_forward.setup(rt)

    def forward(self, x, residual, ctx, cache_layer: int, writes_cache: bool = True):
        if not isinstance(x, K.StreamRows) or residual is not None:
            raise ValueError("a parallel_stream block takes a 32-bit stream (`StreamRows`), as its embedding or the block before leaves it")
        act = x.act.dtype
        stream = x.f32
        if x.normed_by is self.norm:
            h = x.act
        else:
            _, h = K.stream_add_many(stream, [], self.norm.weight, self.norm.eps, self.norm.norm_kind, act)
        with nvtx_range(self.spec.mixer.spec.kind):
            joins = _addends(self.mixer.forward(h, ctx, cache_layer, writes_cache), self.spec.mixer.out_scale)
        if self.feed_forward is not None:
            with nvtx_range(self.spec.feed_forward.kind):
                joins += _addends(self.feed_forward.forward(h))
        # all sublayers' outputs join the stream in the kernel that also makes the next block's normed input
        nxt = ctx.extras.get("next_input_norm")
        nxt = nxt if (hasattr(nxt, "norm_kind") and not ctx.extras.get("next_opens")) else None
        h = None
        while joins:
            now, joins = joins[:4], joins[4:]
            last = not joins
            if last and nxt is not None:
                _, h = K.stream_add_many(stream, now, nxt.weight, nxt.eps, nxt.norm_kind, act)
            else:
                K.stream_add_many(stream, now, None, 0.0, "rmsnorm", act)
        if h is None:
            return K.StreamRows(stream, x.act[:0]), None
        return K.StreamRows(stream, h, normed_by=nxt), None
