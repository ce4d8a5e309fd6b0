"""RMSNorm, in the fused residual form the blocks use."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..registry import NORMS
from .base import VECTOR, ParamSpec, Part, normal_init, ones_init


@NORMS.register("rmsnorm")
class RMSNorm(Part):
    """`forward(x, residual, other=..., in_scales=..., out_scales=...)`:
    residual <- (x [scaled, + other scaled]) + residual ; outputs = rmsnorm(residual) * out_scale_k.
    (python/logssms/layers/norm.py:56-97, python/logssms/kernel/norm.py:8-52.)"""
    can_defer = True          # forward() takes `defer=`: see there
    takes_summed_rows = True  # forward() takes `K.SummedRows` as x: the product before has joined the residual already
    takes_scaled_rows = True  # forward() takes `K.ScaledRows` as x: it applies the pending multiplier while it loads x
    takes_stream_rows = True  # forward() takes `K.StreamRows` as x (a 32-bit stream); `post()` is the post-norm form
    norm_kind = "rmsnorm"     # what the kernels of a pre-norm stream call this norm (`K.NORM_KINDS`)
    kernels = ("norm", "linear_skinny", "stream_norm")

    def __init__(self, spec, perturb_init: bool = False):
        self.size, self.eps = spec.size, spec.eps
        self.param_name = getattr(spec, "param_name", "weight")
        # `offset`: the norm multiplies by offset + the stored weight (1.0: a weight that is stored around zero); the sum is
        # made once, in 32-bit, when the weight arrives
        self.offset = float(getattr(spec, "offset", 0.0))
        self._jitter = 0.1 if perturb_init else 0.0
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        if self.offset != 0.0:
            return {self.param_name: ParamSpec((self.size,), VECTOR, normal_init(self._jitter))}
        return {self.param_name: ParamSpec((self.size,), VECTOR, ones_init(self._jitter))}

    def bind(self, t):
        self.weight = t[self.param_name] if self.offset == 0.0 else t[self.param_name] + self.offset

    def post(self, stream, y, skip_scale: float = 1.0, *, extra=None, row_scale=None):
        """Post-norm on a 32-bit stream: norm(skip_scale * stream + y [+ row_scale[t] * extra]) as `K.StreamRows`."""
        return K.skip_rmsnorm(stream, y, skip_scale, self.weight, self.eps, extra=extra, row_scale=row_scale)

    def forward(self, x, residual=None, *, other=None, in_scales=(1.0, 1.0), out_scales=(1.0,), want_residual=True,
                defer=False):
        """With `defer` (the caller's consumers all take `NormedRows`: their first step is a product), and
        few enough rows, nothing is launched here: the outputs are `NormedRows` that the consumers' products
        normalise in their prologue, and the new residual is a fresh tensor that the first of them writes."""
        if isinstance(x, K.StreamRows):
            # a 32-bit stream: normalised in 32-bit, handed on in the activation dtype
            if residual is not None or other is not None:
                raise ValueError("a 32-bit stream carries its residual itself")
            normed = K.skip_rmsnorm(x, None, 1.0, self.weight, self.eps, want_f32=False, act_dtype=x.act.dtype).act
            return tuple(normed if s == 1.0 else K.scale(normed, s) for s in out_scales), None
        if isinstance(x, K.ScaledRows):
            # the multiplier of the product that made x rides in this norm's load of x (as in_scales[0])
            if other is None and in_scales[0] == 1.0:
                x, in_scales = x.rows, (x.scale, in_scales[1])
            else:
                x = x.tensor()
        if isinstance(x, K.SummedRows):
            # x is already the residual sum (float32), with its rounded copy and the rows' sums of squares
            if residual is not None or other is not None:
                raise ValueError("summed rows have joined their residual already")
            if defer and K.deferred_norm_ok(x):
                shared = {"residual_out": None, "written": True}
                return tuple(K.NormedRows(x, None, None, self.weight, self.eps, (1.0, 1.0), s, shared) for s in out_scales), x.residual
            return K.summed_rmsnorm(x, self.weight, self.eps, out_scales), x.residual
        if defer and K.deferred_norm_ok(x):
            shared = {"residual_out": torch.empty_like(x) if want_residual else None, "written": False}
            outs = tuple(K.NormedRows(x, other, residual, self.weight, self.eps, in_scales, s, shared) for s in out_scales)
            return outs, shared["residual_out"]
        return K.add_rmsnorm(x, self.weight, self.eps, residual, other=other, in_scales=in_scales,
                             out_scales=out_scales, want_residual=want_residual)


@NORMS.register("layernorm")
class LayerNorm(Part):
    """(x - mean) / sqrt(variance + eps) * weight, no bias; the variance is the mean of the squared deviations.  It reads a
    32-bit stream (`K.StreamRows`) and hands the normed rows on in the activation dtype; the blocks of a pre-norm stream
    fuse it into the kernel that closes the sublayer before (`K.stream_add_norm`, `K.stream_side`), by `norm_kind`."""
    takes_stream_rows = True
    norm_kind = "layernorm"
    kernels = ("stream_layer",)

    def __init__(self, spec, perturb_init: bool = False):
        self.size, self.eps = spec.size, spec.eps
        self.param_name = getattr(spec, "param_name", "weight")
        self._jitter = 0.1 if perturb_init else 0.0
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {self.param_name: ParamSpec((self.size,), VECTOR, ones_init(self._jitter))}

    def bind(self, t):
        self.weight = t[self.param_name]

    def forward(self, x, residual=None, *, out_scales=(1.0,), want_residual=True, **unused):
        if not isinstance(x, K.StreamRows) or residual is not None:
            raise ValueError("layernorm reads a 32-bit stream (`StreamRows`)")
        _, normed = K.stream_add_norm(x.f32, None, None, self.weight, self.eps, self.norm_kind, x.act.dtype)
        return tuple(normed if s == 1.0 else K.scale(normed, s) for s in out_scales), None
