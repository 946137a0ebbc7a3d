"""Dense feed-forwards, added to the residual stream: act(h @ w_in + b_in) @ w_out + b_out
(reference: kelpie-models/kelpie_models/models/torch/gpt2.py:94-96), and the gated form with clamped
projections."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Runtime, register_feed_forward
from .util import matrix, vector


@register_feed_forward("mlp")
class DenseMLP:
    """params: activation ("gelu_new" | "gelu"). weights: w_in [D, F], b_in, w_out [F, D], b_out,
    both matrices stored [in, out]; the inner width F is the weights' own."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.activation = params["activation"]
        if self.activation not in ops.ACTIVATIONS or self.activation in (None, "none"):
            raise ValueError(f"mlp: unknown activation {self.activation!r}")
        self.w_in = matrix(weights["w_in"], rt)
        self.b_in = vector(weights["b_in"], rt)
        self.w_out = matrix(weights["w_out"], rt)
        self.b_out = vector(weights["b_out"], rt)
        if self.w_in.shape[1] != self.w_out.shape[0] or self.w_in.shape[0] != self.w_out.shape[1]:
            raise ValueError(f"mlp: w_in {tuple(self.w_in.shape)} and w_out {tuple(self.w_out.shape)} do not fit")

    takes_lazy_norm = True  # the input goes straight into ops.linear

    def matrices(self):
        """The weight matrices in the order in which forward() uses them."""
        return [self.w_in, self.w_out]

    def resident_mlp(self) -> dict:
        return {"w_fc": self.w_in, "b_fc": self.b_in, "w_pr": self.w_out, "b_pr": self.b_out, "act": self.activation,
                "width": self.w_in.shape[0], "inner": self.w_in.shape[1]}

    def forward(self, h, residual, ctx):
        return ops.mlp(h, self.w_in, self.b_in, self.activation, self.w_out, self.b_out, residual=residual)


@register_feed_forward("gated_clamped")
class GatedClampedMLP:
    """W_down y with y = g * sigmoid(alpha * g) * (u + up_offset), g = min(W_gate h, limit) and
    u = clamp(W_up h, -limit, limit). params: limit, alpha, up_offset. weights: w_gate [F, D], w_up [F, D],
    w_down [D, F], all stored [out, in], no biases. The two input projections run as one product over the
    stacked matrix [2 F, D]."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.limit, self.alpha, self.up_offset = float(params["limit"]), float(params["alpha"]), float(params["up_offset"])
        gate, up, down = weights["w_gate"], weights["w_up"], weights["w_down"]
        if gate.shape != up.shape or down.shape != (gate.shape[1], gate.shape[0]):
            raise ValueError(f"gated feed-forward: w_gate {tuple(gate.shape)}, w_up {tuple(up.shape)} and w_down {tuple(down.shape)} do not fit")
        self.inner = gate.shape[0]
        self.w_gate_up = matrix(torch.cat([gate, up], dim=0), rt)
        self.w_down = matrix(down, rt)

    def matrices(self):
        return [self.w_gate_up, self.w_down]

    def input_matrix(self):
        """The stacked projections of the input, [gate; up] x D stored [out, in] (see `forward_projected`)."""
        return self.w_gate_up

    def forward(self, h, residual, ctx):
        return self.forward_projected(ops.linear(h, self.w_gate_up, None, w_is_nk=True), residual, ctx)

    def forward_projected(self, gate_up, residual, ctx):
        """`gate_up` [T, 2 F]: the input's gate and up projections."""
        y = ops.gated_act(gate_up, self.limit, self.alpha, self.up_offset)
        return ops.linear(y, self.w_down, None, w_is_nk=True, residual=residual)


@register_feed_forward("act_mlp")
class ActivatedMLP:
    """W_down act(W_up h) without biases. params: activation ("xielu": for z > 0, softplus(p) z^2 + z / 2; for z <= 0,
    (1/2 + softplus(q)) (e^z - 1 - z) + z / 2, with the two learned numbers p, q of `act`). weights: w_up [F, D], w_down [D, F]
    stored [out, in], act [2]."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.activation = params.get("activation", "xielu")
        if self.activation != "xielu":
            raise ValueError(f"feed-forward: unknown activation {self.activation!r}")
        up, down = weights["w_up"], weights["w_down"]
        if down.shape != (up.shape[1], up.shape[0]) or weights["act"].numel() != 2:
            raise ValueError(f"feed-forward: w_up {tuple(up.shape)}, w_down {tuple(down.shape)} and act {tuple(weights['act'].shape)} do not fit")
        self.w_up, self.w_down = matrix(up, rt), matrix(down, rt)
        p, q = (float(v) for v in weights["act"].to(torch.float64).reshape(2))
        self.a_pos, self.a_neg = _softplus(p), 0.5 + _softplus(q)

    def matrices(self):
        return [self.w_up, self.w_down]

    def _inner(self, h):
        return ops.xielu(ops.linear(h, self.w_up, None, w_is_nk=True), self.a_pos, self.a_neg)

    def mix(self, h, ctx):
        """The feed-forward's output [T, D] in float32, without the residual stream."""
        return ops.linear(self._inner(h), self.w_down, None, w_is_nk=True, out_dtype=torch.float32)

    def forward(self, h, residual, ctx):
        return ops.linear(self._inner(h), self.w_down, None, w_is_nk=True, residual=residual)


def _softplus(x: float) -> float:
    import math

    return x if x > 30.0 else math.log1p(math.exp(x))


@register_feed_forward("gated_mlp")
class GatedMLP:
    """W_down (act(W_gate h) * (W_up h)) with act = relu. params: activation ("relu"). weights: w_gate [F, D], w_up
    [F, D], w_down [D, F], stored [out, in], no biases. The two input projections run as one product."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.activation = params.get("activation", "relu")
        if self.activation != "relu":
            raise ValueError(f"gated feed-forward: unknown activation {self.activation!r}")
        gate, up, down = weights["w_gate"], weights["w_up"], weights["w_down"]
        if gate.shape != up.shape or down.shape != (gate.shape[1], gate.shape[0]):
            raise ValueError(f"gated feed-forward: w_gate {tuple(gate.shape)}, w_up {tuple(up.shape)} and w_down {tuple(down.shape)} do not fit")
        self.w_gate_up = matrix(torch.cat([gate, up], dim=0), rt)
        self.w_down = matrix(down, rt)

    def matrices(self):
        return [self.w_gate_up, self.w_down]

    def forward(self, h, residual, ctx):
        y = ops.expert_act(ops.linear(h, self.w_gate_up, None, w_is_nk=True), self.activation)
        return ops.linear(y, self.w_down, None, w_is_nk=True, residual=residual)


@register_feed_forward("routed_experts")
class RoutedExperts:
    """A mixture of small gated feed-forwards, of which each row uses `top`, and optionally one more that every row uses.

        z = W_router h + b_router (float32); the `top` largest logits are chosen (the lower index wins a tie) and their
        weights are the softmax over the chosen logits only
        expert: W_down y, y = g sigmoid(alpha g) (u + up_offset), g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit)
        output = sum over the chosen experts of weight * expert(h) (+ shared(h), same form with shared_limit)

    With `scoring` "sigmoid" the router is another one: s = sigmoid(W_router h); an expert is chosen by s + correction, only
    among the experts of the `keep_groups` best of `n_groups` equal groups of neighbours (a group counts by the sum of its two
    largest s + correction), the `top` largest; weights are the chosen experts' s over their sum (+ 1e-20). With `activation`
    "silu" an expert is W_down (g sigmoid(g) u) without clamps. With `shared.w_sg` [1, D] the expert that every row uses is
    multiplied by sigmoid(w_sg h), one number per row. With `scoring` "softmax" the scores s are the softmax of the logits over
    ALL experts, chosen inside the best groups as with "sigmoid". `group_mark` "best": a group counts by its largest score alone.
    `normalise` false: the weights are the chosen experts' scores times `route_scale` and are not made to sum to one.

    params: n_experts, top, limit, alpha, up_offset, shared_limit (None: no shared expert); scoring ("softmax_top" | "sigmoid" |
    "softmax"), n_groups, keep_groups, group_mark ("two_best" | "best"), normalise, route_scale, activation ("clamped_swish" |
    "silu"), shared (true: a shared expert, for activations without a limit).
    weights: router [E, D], router_b [E] or correction [E], e<i>.w_gate / e<i>.w_up [F, D], e<i>.w_down [D, F] for every expert,
    and optionally shared.w_gate / shared.w_up [Fs, D], shared.w_down [D, Fs], shared.w_sg [1, D].

    All experts' input projections are stacked into one matrix ([gates of every expert; shared gate; ups of every expert;
    shared up]) and their down matrices side by side into another, so that a layer is two dense products: the
    activation between them multiplies an expert's columns by the row's weight for that expert (zero where it was not
    chosen), and the second product's sum over all columns is the weighted sum over experts. Every step reads all
    experts' weights; a form that reads only the chosen ones for a few rows is not built."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.n_experts, self.top = int(params["n_experts"]), int(params["top"])
        self.activation = params.get("activation", "clamped_swish")
        self.scoring = params.get("scoring", "softmax_top")
        if self.activation not in ("clamped_swish", "silu") or self.scoring not in ("softmax_top", "sigmoid", "softmax"):
            raise ValueError(f"routed experts: unknown activation {self.activation!r} or scoring {self.scoring!r}")
        self.n_groups, self.keep_groups = int(params.get("n_groups", 1)), int(params.get("keep_groups", 1))
        self.group_mark, self.normalise = params.get("group_mark", "two_best"), bool(params.get("normalise", True))
        self.route_scale = float(params.get("route_scale", 1.0))
        clamped = self.activation == "clamped_swish"
        self.limit, self.alpha, self.up_offset = (float(params[k]) if clamped else 0.0 for k in ("limit", "alpha", "up_offset"))
        self.shared = params.get("shared_limit") is not None or bool(params.get("shared", False))
        self.shared_limit = float(params["shared_limit"]) if params.get("shared_limit") is not None else self.limit
        gates = [weights[f"e{i}.w_gate"] for i in range(self.n_experts)]
        ups = [weights[f"e{i}.w_up"] for i in range(self.n_experts)]
        downs = [weights[f"e{i}.w_down"] for i in range(self.n_experts)]
        self.expert_width = gates[0].shape[0]
        if any(g.shape != gates[0].shape or u.shape != gates[0].shape or d.shape != (g.shape[1], g.shape[0]) for g, u, d in zip(gates, ups, downs)):
            raise ValueError("routed experts: the experts' matrices differ in shape or do not fit each other")
        if self.shared:
            gates.append(weights["shared.w_gate"]); ups.append(weights["shared.w_up"]); downs.append(weights["shared.w_down"])
        self.w_gate_up = matrix(torch.cat(gates + ups, dim=0), rt)
        self.w_down = matrix(torch.cat(downs, dim=1), rt)
        router = weights["router"]
        if router.shape[0] != self.n_experts or not 1 <= self.top <= self.n_experts:
            raise ValueError(f"routed experts: router {tuple(router.shape)}, top {self.top}, {self.n_experts} experts")
        # a gate on the shared expert is one more row of the router's matrix: its logit comes out of the router's launch
        self.shared_gate = self.shared and weights.get("shared.w_sg") is not None
        if self.shared_gate:
            if self.scoring == "softmax_top" or weights["shared.w_sg"].numel() != router.shape[1]:
                raise ValueError("routed experts: a gate on the shared expert needs the sigmoid router and one row of the model's width")
            router = torch.cat([router, weights["shared.w_sg"].reshape(1, -1)], dim=0)
        self.router = vector(router, rt)      # float32: the router is computed in 32-bit
        self.router_b = vector(weights["router_b"], rt) if weights.get("router_b") is not None else None
        self.correction = vector(weights["correction"], rt) if weights.get("correction") is not None else None

    def matrices(self):
        return [self.w_gate_up, self.w_down]

    def _inner(self, h):
        gate = None
        if self.scoring != "softmax_top":
            route, _, _, gate = ops.route_scored(h, self.router, self.correction, self.top, self.n_groups, self.keep_groups,
                                                 n_extra=int(self.shared_gate), scoring=self.scoring, group_mark=self.group_mark,
                                                 normalise=self.normalise, weight_scale=self.route_scale)
        else:
            route, _, _ = ops.route_top_k(h, self.router, self.router_b, self.top)
        return ops.expert_act(ops.linear(h, self.w_gate_up, None, w_is_nk=True), self.activation, self.limit, self.alpha,
                              self.up_offset, route=route, n_experts=self.n_experts, expert_width=self.expert_width,
                              tail_limit=self.shared_limit, tail_gate=gate)

    def mix(self, h, ctx):
        """The feed-forward's output [T, D] in float32, without the residual stream."""
        return ops.linear(self._inner(h), self.w_down, None, w_is_nk=True, out_dtype=torch.float32)

    def forward(self, h, residual, ctx):
        return ops.linear(self._inner(h), self.w_down, None, w_is_nk=True, residual=residual)
