"""Mixers that carry a state of fixed size per request instead of a cache that grows with the sequence:
a matrix memory with exponential gates (mLSTM), retention (linear attention with a fixed decay per head) and a
state-space layer with a short causal convolution (the recurrence of Mamba-2). Their state lives in 32-bit floats in the request's state slot, starts at
zero with a sequence's first token and is carried from step to step; prompts, portions and single decoded
tokens run through the same kernels (csrc/kernels/recurrent.cu), entry by entry, row by row.

Both offer `mix(h, ctx, cache, state)`, the mixer's output [T, D] in float32 without the residual stream,
for an arrangement that joins several mixers, beside the usual `forward`, whose last product adds the stream.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Runtime, StateSpec, register_mixer
from .util import matrix, vector


@register_mixer("mlstm")
class MatrixMemory:
    """Per head a matrix S [dim x vdim], a normaliser n [dim] and a running maximum m of the gates' logarithms:

        log_i = cap(W_i h + b_i), log_f = logsigmoid(cap(W_f h + b_f)), cap(x) = gate_cap tanh(x / gate_cap)
        m' = max(log_f + m, log_i)
        S' = exp(log_f + m - m') S + exp(log_i - m') k v^T,   n' likewise with k alone
        o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6),       q = W_q h dim^-1/2, k = W_k h, v = W_v h

    S, n and m start at zero. Each head's o is divided by its root mean square, the heads are concatenated,
    multiplied by `norm`, by sigmoid(W_g h), and projected by W_o.

    params: n_heads, head_dim, v_head_dim, gate_cap (0: none), norm_eps.
    weights (matrices stored [out, in]): w_q, w_k [H * head_dim, D], w_v, w_gate [H * v_head_dim, D], w_out
    [D, H * v_head_dim], norm [H * v_head_dim], w_i, w_f [H, D], b_i, b_f [H].
    The four wide projections run as one product; the gates' as a 32-bit one of their own."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.n_heads, self.head_dim, self.v_head_dim = int(params["n_heads"]), int(params["head_dim"]), int(params["v_head_dim"])
        self.gate_cap, self.norm_eps = float(params.get("gate_cap", 0.0)), float(params["norm_eps"])
        self.qk_width, self.v_width = self.n_heads * self.head_dim, self.n_heads * self.v_head_dim
        stacked = [weights["w_q"], weights["w_k"], weights["w_v"], weights["w_gate"]]
        if [w.shape[0] for w in stacked] != [self.qk_width, self.qk_width, self.v_width, self.v_width] or \
                weights["w_out"].shape[1] != self.v_width or weights["w_i"].shape[0] != self.n_heads:
            raise ValueError(f"mlstm: projections {[tuple(w.shape) for w in stacked]} and an output of {tuple(weights['w_out'].shape)} "
                             f"do not fit {self.n_heads} heads of {self.head_dim} x {self.v_head_dim}")
        self.w_in = matrix(torch.cat(stacked, dim=0), rt)
        self.w_out = matrix(weights["w_out"], rt)
        self.norm = vector(weights["norm"], rt)
        self.w_gates = vector(torch.cat([weights["w_i"], weights["w_f"]], dim=0), rt)   # float32: the gates enter the recurrence
        self.b_gates = vector(torch.cat([weights["b_i"], weights["b_f"]], dim=0), rt)
        self._state_floats = None

    cache_spec = None
    capturable = True

    def matrices(self):
        return [self.w_in, self.w_out]

    @property
    def state_spec(self) -> StateSpec:
        if self._state_floats is None:
            self._state_floats = self.n_heads * ops.mlstm_state_floats(self.head_dim, self.v_head_dim)
        return StateSpec((self._state_floats,), torch.float32)

    def _inner(self, h, ctx, state):
        proj = ops.linear(h, self.w_in, None, w_is_nk=True)
        gates = ops.small_linear(h, self.w_gates, self.b_gates)
        a, b = self.qk_width, 2 * self.qk_width
        o = ops.mlstm_scan(proj[:, :a], proj[:, a:b], proj[:, b: b + self.v_width], gates, self.gate_cap, self.head_dim ** -0.5,
                           state, ctx.q_start, ctx.state_slot, ctx.fresh, self.n_heads, self.head_dim, self.v_head_dim)
        return ops.group_norm_gated(o, proj[:, b + self.v_width:], self.norm, self.n_heads, self.norm_eps, False, proj.dtype)

    def mix(self, h, ctx, cache=None, state=None, writes_cache: bool = True):
        return ops.linear(self._inner(h, ctx, state), self.w_out, None, w_is_nk=True, out_dtype=torch.float32)

    def forward(self, h, residual, ctx, cache=None, state=None, writes_cache: bool = True):
        return ops.linear(self._inner(h, ctx, state), self.w_out, None, w_is_nk=True, residual=residual)


@register_mixer("retention")
class Retention:
    """Linear attention with one fixed decay per head and neither softmax nor denominator. Per head:

        S' = decay S + k v^T   (S: [head_dim x v_head_dim], from zero),   o = S'^T q
        q = rotate(W_q h), k = rotate(W_k h) head_dim^-1/2, v = W_v h

    (rotation: of each head the first rot_dims dimensions, dimension i with i + rot_dims / 2, by the angle position *
    rot_freqs[i]). Each head's o is divided by its root mean square (no gain), the heads are concatenated, multiplied by
    silu(W_g h) and projected by W_o. The rotation happens inside the recurrence's kernel, in float32: what enters the
    recurrence is the projections' values and nothing rounded after them.

    params: n_heads, head_dim, v_head_dim, decay (one number per head), rot_dims, rot_freqs, norm_eps.
    weights (stored [out, in], no biases): w_q, w_k [H head_dim, D], w_v, w_gate [H v_head_dim, D], w_out [D, H v_head_dim]."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.n_heads, self.head_dim, self.v_head_dim = int(params["n_heads"]), int(params["head_dim"]), int(params["v_head_dim"])
        self.norm_eps, self.rot_dims = float(params["norm_eps"]), int(params.get("rot_dims", 0))
        decay, freqs = [float(x) for x in params["decay"]], [float(f) for f in params.get("rot_freqs", ())]
        if len(decay) != self.n_heads or self.rot_dims % 2 or not 0 <= self.rot_dims <= self.head_dim or len(freqs) != self.rot_dims // 2:
            raise ValueError(f"retention: {len(decay)} decays for {self.n_heads} heads, {self.rot_dims} rotated dimensions of "
                             f"{self.head_dim} with {len(freqs)} frequencies")
        self.qk_width, self.v_width = self.n_heads * self.head_dim, self.n_heads * self.v_head_dim
        stacked = [weights["w_q"], weights["w_k"], weights["w_v"], weights["w_gate"]]
        if [w.shape[0] for w in stacked] != [self.qk_width, self.qk_width, self.v_width, self.v_width] or weights["w_out"].shape[1] != self.v_width:
            raise ValueError(f"retention: projections {[tuple(w.shape) for w in stacked]} and an output of {tuple(weights['w_out'].shape)} "
                             f"do not fit {self.n_heads} heads of {self.head_dim} x {self.v_head_dim}")
        self.w_in = matrix(torch.cat(stacked, dim=0), rt)
        self.w_out = matrix(weights["w_out"], rt)
        # decays and frequencies: exact in float64, rounded once to float32
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(rt.device)
        self.freqs = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(rt.device)

    cache_spec = None
    capturable = True

    def matrices(self):
        return [self.w_in, self.w_out]

    @property
    def state_spec(self) -> StateSpec:
        return StateSpec((self.n_heads * self.head_dim * self.v_head_dim,), torch.float32)

    def _inner(self, h, ctx, state):
        proj = ops.linear(h, self.w_in, None, w_is_nk=True)
        a, b = self.qk_width, 2 * self.qk_width
        o = ops.retention_scan(proj[:, :a], proj[:, a:b], proj[:, b: b + self.v_width], self.decay, self.head_dim ** -0.5, self.freqs,
                               self.rot_dims, ctx.positions, state, ctx.q_start, ctx.state_slot, ctx.fresh, self.n_heads, self.head_dim,
                               self.v_head_dim)
        return ops.group_norm_gated(o, proj[:, b + self.v_width:], None, self.n_heads, self.norm_eps, "silu_after", proj.dtype)

    def mix(self, h, ctx, cache=None, state=None, writes_cache: bool = True):
        return ops.linear(self._inner(h, ctx, state), self.w_out, None, w_is_nk=True, out_dtype=torch.float32)

    def forward(self, h, residual, ctx, cache=None, state=None, writes_cache: bool = True):
        return ops.linear(self._inner(h, ctx, state), self.w_out, None, w_is_nk=True, residual=residual)


@register_mixer("ssd")
class StateSpace:
    """inner = n_heads * v_head_dim; W_in h is laid out [z: inner | x: inner | B: groups * n_state | C: groups * n_state |
    dt: n_heads]. x, B and C pass a causal convolution per channel (taps [channels, conv_taps], the last column the
    current token's, zeros before the start) and silu. dt = softplus(dt + dt_bias). Per head (head i uses group
    i // (n_heads / groups)):

        S' = exp(-exp(A_log) dt) S + dt B x^T   (S: [n_state x v_head_dim]),   y = S'^T C + D x

    y (heads concatenated) is multiplied by silu(z), RMS-normed in norm_groups equal parts, times `norm`, then W_o. The
    state is S and the convolution's last conv_taps - 1 inputs.

    params: n_heads, v_head_dim, n_state, n_groups, conv_taps, norm_groups, norm_eps.
    weights: w_in [2 inner + 2 groups n_state + n_heads, D], conv [channels, conv_taps], conv_b [channels], dt_bias, a_log,
    d_skip [n_heads], norm [inner], w_out [D, inner]. The step sizes' rows of w_in run as a 32-bit product of their own."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.n_heads, self.v_head_dim, self.n_state = int(params["n_heads"]), int(params["v_head_dim"]), int(params["n_state"])
        self.n_groups, self.conv_taps = int(params["n_groups"]), int(params["conv_taps"])
        self.norm_groups, self.norm_eps = int(params["norm_groups"]), float(params["norm_eps"])
        self.inner = self.n_heads * self.v_head_dim
        self.bc_width = self.n_groups * self.n_state
        self.channels = self.inner + 2 * self.bc_width
        w_in = weights["w_in"]
        if w_in.shape[0] != self.inner + self.channels + self.n_heads or tuple(weights["conv"].shape) != (self.channels, self.conv_taps) \
                or weights["w_out"].shape[1] != self.inner or self.n_heads % self.n_groups or self.inner % self.norm_groups:
            raise ValueError(f"ssd: w_in {tuple(w_in.shape)}, conv {tuple(weights['conv'].shape)}, w_out {tuple(weights['w_out'].shape)} do not "
                             f"fit {self.n_heads} heads of {self.v_head_dim}, {self.n_groups} groups of {self.n_state}, {self.conv_taps} taps")
        self.w_in = matrix(w_in[: self.inner + self.channels], rt)
        self.w_steps = vector(w_in[self.inner + self.channels:], rt)
        self.conv, self.conv_b = vector(weights["conv"], rt), vector(weights["conv_b"], rt)
        self.dt_bias, self.a_log, self.d_skip = (vector(weights[k], rt) for k in ("dt_bias", "a_log", "d_skip"))
        self.norm = vector(weights["norm"], rt)
        self.w_out = matrix(weights["w_out"], rt)
        self.conv_state_off = self.n_heads * self.n_state * self.v_head_dim

    cache_spec = None
    capturable = True

    def matrices(self):
        return [self.w_in, self.w_out]

    @property
    def state_spec(self) -> StateSpec:
        return StateSpec((self.conv_state_off + (self.conv_taps - 1) * self.channels,), torch.float32)

    def _inner(self, h, ctx, state):
        proj = ops.linear(h, self.w_in, None, w_is_nk=True)
        steps = ops.small_linear(h, self.w_steps, None)
        z, xbc = proj[:, : self.inner], proj[:, self.inner:]
        mixed = ops.causal_conv(xbc, self.conv, self.conv_b, state, self.conv_state_off, ctx.row_entry, ctx.q_start,
                                ctx.state_slot, ctx.fresh)
        x, b = mixed[:, : self.inner], mixed[:, self.inner: self.inner + self.bc_width]
        y = ops.ssd_scan(x, b, mixed[:, self.inner + self.bc_width:], steps, self.dt_bias, self.a_log, self.d_skip, state,
                         ctx.q_start, ctx.state_slot, ctx.fresh, self.n_heads, self.n_groups, self.n_state, self.v_head_dim,
                         conv_in=xbc, conv_taps=self.conv_taps, conv_state_off=self.conv_state_off)
        return ops.group_norm_gated(y, z, self.norm, self.norm_groups, self.norm_eps, True, proj.dtype)

    def mix(self, h, ctx, cache=None, state=None, writes_cache: bool = True):
        return ops.linear(self._inner(h, ctx, state), self.w_out, None, w_is_nk=True, out_dtype=torch.float32)

    def forward(self, h, residual, ctx, cache=None, state=None, writes_cache: bool = True):
        return ops.linear(self._inner(h, ctx, state), self.w_out, None, w_is_nk=True, residual=residual)


@register_mixer("side_by_side")
class SideBySide:
    """Two mixers read the same input; each one's output is RMS-normed over the model width with a plain gain of its
    own, and `share` times their sum joins the stream: x + share (norm(left(h)) w_left + norm(right(h)) w_right).

    params: left, right: {"kind": mixer kind, "params": {...}}; eps; share (default 0.5).
    weights: left_out, right_out [D], and each mixer's own weights under the prefixes "left." and "right.".
    Either mixer may keep a per-token cache and either a per-request state, but only one of each."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        from .base import registry

        self.eps, self.share = float(params["eps"]), float(params.get("share", 0.5))
        self.sides = []
        for side in ("left", "right"):
            spec = params[side]
            own = {name[len(side) + 1:]: t for name, t in weights.items() if name.startswith(side + ".")}
            part = registry("mixer")[spec["kind"]](spec["params"], own, rt)
            if not hasattr(part, "mix"):
                raise ValueError(f"side_by_side: a mixer of kind {spec['kind']!r} has no `mix` (its output without the stream)")
            self.sides.append(part)
        self.w_left, self.w_right = vector(weights["left_out"], rt), vector(weights["right_out"], rt)
        for what in ("cache_spec", "state_spec"):
            if sum(getattr(p, what, None) is not None for p in self.sides) > 1:
                raise ValueError(f"side_by_side: both mixers have a {what}; a layer has one cache member and one state member")
        self.capturable = all(getattr(p, "capturable", False) for p in self.sides)

    def _of(self, what):
        return next((getattr(p, what) for p in self.sides if getattr(p, what, None) is not None), None)

    @property
    def cache_spec(self):
        return self._of("cache_spec")

    @property
    def state_spec(self):
        return self._of("state_spec")

    def matrices(self):
        return [m for p in self.sides for m in p.matrices()]

    def forward(self, h, residual, ctx, cache=None, state=None, writes_cache: bool = True):
        left, right = (p.mix(h, ctx, cache, state, writes_cache) for p in self.sides)
        return ops.pair_norm_add(residual, left, right, self.w_left, self.w_right, self.eps, self.share)
