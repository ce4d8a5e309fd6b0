"""Feed-forwards without a SwiGLU: the dense up/act/down layer and the routed mixture of clamped gated experts."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..registry import FEED_FORWARDS
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init


@FEED_FORWARDS.register("dense_mlp")
class DenseMLP(Part):
    """down(act(up(x))) with the tanh form of GELU.  Tensors: up, down."""
    kernels = ("moe", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if spec.activation != "gelu_tanh":
            raise ValueError(f"dense_mlp knows the activation gelu_tanh, not {spec.activation!r}")
        self.spec = spec
        self.up = self.down = None

    def param_specs(self):
        s = self.spec
        return {"up": ParamSpec((s.intermediate_size, s.hidden_size), MATRIX, normal_init(s.hidden_size ** -0.5)),
                "down": ParamSpec((s.hidden_size, s.intermediate_size), MATRIX, normal_init(2.0 * s.intermediate_size ** -0.5))}

    def bind(self, t):
        self.up, self.down = t["up"], t["down"]

    def setup(self, rt) -> None:
        pass

    def forward(self, x: torch.Tensor):
        return K.linear(K.gelu_tanh(K.linear(x, self.up)), self.down)


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(Part):
    """down(g~ sigmoid(act_alpha g~) (u~ + 1)) with g~ = min(gate(x), limit), u~ = clamp(up(x), -limit, limit): the
    clamped gated expert as a dense layer.  The gate and up products are one (merged at bind time).  Tensors: gate, up, down."""
    kernels = ("moe", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        self.gate_up = self.down = None

    def param_specs(self):
        s = self.spec
        fan = normal_init(s.hidden_size ** -0.5)
        return {"gate": ParamSpec((s.intermediate_size, s.hidden_size), MATRIX, fan),
                "up": ParamSpec((s.intermediate_size, s.hidden_size), MATRIX, fan),
                "down": ParamSpec((s.hidden_size, s.intermediate_size), MATRIX, normal_init(2.0 * s.intermediate_size ** -0.5))}

    def bind(self, t):
        self.gate_up = torch.cat([t["gate"], t["up"]], 0).contiguous()
        self.down = t["down"]

    def setup(self, rt) -> None:
        pass

    def forward(self, x: torch.Tensor):
        s = self.spec
        return K.linear(K.moe_activation(K.linear(x, self.gate_up), None, 1, s.limit, s.act_alpha), self.down)


@FEED_FORWARDS.register("glu")
class GLU(Part):
    """down(act(gate(x)) * up(x)) with act the tanh form of GELU or silu.  The gate and up products are one (merged at bind
    time).  Tensors: gate, up, down."""
    kernels = ("moe", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if spec.activation not in ("gelu_tanh", "silu"):
            raise ValueError(f"glu knows the activations gelu_tanh and silu, not {spec.activation!r}")
        self.spec = spec
        self.gate_up = self.down = None

    def param_specs(self):
        s = self.spec
        fan = normal_init(s.hidden_size ** -0.5)
        return {"gate": ParamSpec((s.intermediate_size, s.hidden_size), MATRIX, fan),
                "up": ParamSpec((s.intermediate_size, s.hidden_size), MATRIX, fan),
                "down": ParamSpec((s.hidden_size, s.intermediate_size), MATRIX, normal_init(2.0 * s.intermediate_size ** -0.5))}

    def bind(self, t):
        self.gate_up = torch.cat([t["gate"], t["up"]], 0).contiguous()
        self.down = t["down"]

    def setup(self, rt) -> None:
        pass

    def forward(self, x: torch.Tensor):
        return K.linear(K.moe_activation(K.linear(x, self.gate_up), None, 1, 0.0, 0.0, mode=self.spec.activation), self.down)


@FEED_FORWARDS.register("routed_mlp")
class RoutedMLP(Part):
    """`num_experts` gated experts and `num_identity` identity experts behind one router (the softmax form is described;
    `spec.score = "sigmoid"` scores every output by itself, `spec.expert = "silu"` with `spec.weigh = "input"` makes the
    expert down(silu(gate(w h)) * up(w h)), computed as silu(w g) * (w u) from the products g, u of the unweighted input).

    Router (32-bit): s = softmax(W_r h) over all outputs; the choice is made on s + correction among the experts of
    the `keep_groups` best of `num_groups` groups of neighbours; the `top` chosen ones weigh in with s * route_scale.
    Expert: g = min(W_gate h, limit), u = clamp(W_up h, +-limit), y = g sigmoid(act_alpha g) (u + 1), output W_down y.
    An identity expert's output is h itself.

    All experts' gate and up matrices are one stacked matrix, and so are their down matrices; the activation kernel
    multiplies every expert's y by the token's weight for that expert (0: not chosen), so the one stacked down product
    is already the weighted sum over the experts.  `forward` returns (rows, h, identity weight per row): the norm that
    follows adds weight * h in 32-bit.  Tensors: router, correction, e<i>.gate, e<i>.up, e<i>.down.

    `spec.score = "softmax_chosen"` ranks the router's outputs themselves (plus the stored bias `router.b` with
    `spec.router_bias`) and weighs the chosen experts by the softmax over the chosen outputs alone; its experts are
    `spec.expert = "silu"` weighted at the "output": w down(silu(gate h) * up h).  With `spec.shared_size` > 0 one more expert
    of that form and size (tensors shared.gate, shared.up, shared.down) runs for every token with weight 1: its gate and up
    rows lie behind the routed experts' in the one stacked product, its activations behind theirs, and its down matrix
    behind theirs, so the one stacked down product adds it too."""
    kernels = ("moe", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        if (spec.score not in ("softmax", "sigmoid", "softmax_chosen") or spec.expert not in ("clamped", "silu")
                or spec.weigh not in ("output", "input")):
            raise ValueError("routed_mlp knows the scores softmax | sigmoid | softmax_chosen, the experts clamped | silu, weights on output | input")
        if spec.score == "softmax_chosen" and (spec.correction or spec.num_identity or spec.num_groups != 1):
            raise ValueError("the softmax over the chosen outputs goes without correction, identity experts and groups")
        if getattr(spec, "shared_size", 0) and spec.num_identity:
            raise ValueError("a shared expert goes without identity experts")
        self.spec = spec
        self.shared_size = int(getattr(spec, "shared_size", 0))
        self.mode = {("clamped", "output"): "clamped", ("silu", "input"): "silu_input", ("silu", "output"): "silu"}.get((spec.expert, spec.weigh))
        if self.mode is None:
            raise ValueError("routed_mlp has kernels for clamped experts weighted at the output and silu experts weighted at either end")
        self.router = self.correction = self.router_bias = self.gate_up = self.down = None

    def param_specs(self):
        s = self.spec
        n = s.num_experts + s.num_identity
        fan = normal_init(s.hidden_size ** -0.5)          # random weights: products of unit-size rows stay of unit size
        specs = {"router": ParamSpec((n, s.hidden_size), VECTOR, normal_init(1.5 * s.hidden_size ** -0.5))}
        if s.correction:
            specs["correction"] = ParamSpec((n,), VECTOR, normal_init(0.05))
        if getattr(s, "router_bias", False):
            specs["router.b"] = ParamSpec((n,), VECTOR, normal_init(0.3))
        if self.shared_size:
            specs["shared.gate"] = ParamSpec((self.shared_size, s.hidden_size), MATRIX, fan)
            specs["shared.up"] = ParamSpec((self.shared_size, s.hidden_size), MATRIX, fan)
            specs["shared.down"] = ParamSpec((s.hidden_size, self.shared_size), MATRIX, normal_init(2.0 * self.shared_size ** -0.5))
        for e in range(s.num_experts):
            specs[f"e{e}.gate"] = ParamSpec((s.expert_size, s.hidden_size), MATRIX, fan)
            specs[f"e{e}.up"] = ParamSpec((s.expert_size, s.hidden_size), MATRIX, fan)
            specs[f"e{e}.down"] = ParamSpec((s.hidden_size, s.expert_size), MATRIX, normal_init(3.0 * s.expert_size ** -0.5))
        return specs

    def bind(self, t):
        s = self.spec
        self.router, self.correction, self.router_bias = t["router"], t.get("correction"), t.get("router.b")
        shared = [t["shared.gate"], t["shared.up"]] if self.shared_size else []
        self.gate_up = torch.cat([t[f"e{e}.{n}"] for e in range(s.num_experts) for n in ("gate", "up")] + shared, 0).contiguous()
        self.down = torch.cat([t[f"e{e}.down"] for e in range(s.num_experts)] + ([t["shared.down"]] if self.shared_size else []), 1).contiguous()

    def setup(self, rt) -> None:
        pass

    def forward(self, x: torch.Tensor):
        s = self.spec
        dense, _, _, id_weight = K.moe_route(x, self.router, self.correction, s.num_experts, s.top, s.num_groups,
                                             s.keep_groups, s.route_scale, sigmoid_scores=s.score == "sigmoid",
                                             bias=self.router_bias, chosen_softmax=s.score == "softmax_chosen")
        if s.num_experts == 0:
            return torch.zeros_like(x), x, id_weight
        gate_up = K.linear(x, self.gate_up)
        if self.shared_size:
            # the routed experts' activations and the shared expert's side by side, as the stacked down matrix wants them
            routed = s.num_experts * s.expert_size
            y = torch.empty((x.shape[0], routed + self.shared_size), dtype=gate_up.dtype, device=gate_up.device)
            K.moe_activation(gate_up[:, :2 * routed], dense, s.num_experts, s.limit, s.act_alpha, mode=self.mode, out=y[:, :routed])
            K.moe_activation(gate_up[:, 2 * routed:], None, 1, s.limit, s.act_alpha, mode=self.mode, out=y[:, routed:])
        else:
            y = K.moe_activation(gate_up, dense, s.num_experts, s.limit, s.act_alpha, mode=self.mode)
        out = K.linear(y, self.down)
        if s.num_identity == 0:
            return out
        return out, x, id_weight
