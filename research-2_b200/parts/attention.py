"""Multi-head (or grouped) causal attention over the paged cache.

Formulas of the reference (kelpie-models/kelpie_models/models/torch/gpt2.py:104-131 and
kernels/ops/paged_attention.py): one fused projection to q, k, v (in that order along the
output), keys and values written to the cache before attention reads it, scores scaled by
`scale`, causal mask (and a window when `window` > 0), softmax and P.V in float32, then the
output projection, whose epilogue adds the residual stream.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import MemberSpec, Runtime, register_mixer
from .util import matrix, vector


@register_mixer("attention")
class PagedAttention:
    """params: n_heads, n_kv_heads, head_dim, scale, window (0 = none).
    weights: w_qkv [D, (n_heads + 2 n_kv_heads) * head_dim] stored [in, out], b_qkv,
    w_out [n_heads * head_dim, D] stored [in, out], b_out."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window = int(params.get("window", 0))
        if self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"attention: n_heads {self.n_heads} is not a multiple of n_kv_heads {self.n_kv_heads}")
        if self.head_dim % 16 != 0 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"attention: head sizes come in steps of 16 from 16 to 256, got {self.head_dim}")
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        self.w_qkv = matrix(weights["w_qkv"], rt)
        self.b_qkv = vector(weights["b_qkv"], rt)
        self.w_out = matrix(weights["w_out"], rt)
        self.b_out = vector(weights["b_out"], rt)
        if self.w_qkv.shape[1] != self.q_width + 2 * self.kv_width or self.w_out.shape[0] != self.q_width:
            raise ValueError(f"attention: weights {tuple(self.w_qkv.shape)} / {tuple(self.w_out.shape)} do not fit "
                             f"{self.n_heads} heads, {self.n_kv_heads} kv heads of {self.head_dim}")
        self.rotary = None  # a positions part that changes q and k may be attached by the model

    def matrices(self):
        """The weight matrices in the order in which forward() uses them."""
        return [self.w_qkv, self.w_out]

    @property
    def cache_spec(self) -> MemberSpec:
        return MemberSpec(self.n_kv_heads, self.head_dim, self.window)

    state_spec = None
    capturable = True  # nothing here depends on the batch's contents, only on its shape
    takes_lazy_norm = True  # the input goes straight into ops.linear

    def resident_attention(self) -> dict | None:
        """For the one-kernel form of a decode step; None while a positions part rotates q and k."""
        if self.rotary is not None or self.w_out.shape[1] != self.w_qkv.shape[0]:
            return None
        return {"w_qkv": self.w_qkv, "b_qkv": self.b_qkv, "w_out": self.w_out, "b_out": self.b_out, "n_heads": self.n_heads,
                "n_kv_heads": self.n_kv_heads, "head_dim": self.head_dim, "scale": self.scale, "window": self.window,
                "width": self.w_qkv.shape[0]}

    def forward(self, h, residual, ctx, cache, state=None, writes_cache: bool = True):
        in_cache = False
        if writes_cache and not ctx.decode_only and self.rotary is None:
            # keys and values leave the product's epilogue for their cache slots (where that kernel takes the shape)
            qkv, in_cache = ops.linear(h, self.w_qkv, self.b_qkv, kv=ops.kv_scatter(
                ctx.slot_mapping[cache.group], cache.k, cache.v, cache.page_stride, cache.page_size, cache.n_pages,
                self.q_width, self.kv_width, self.head_dim))
        else:
            qkv = ops.linear(h, self.w_qkv, self.b_qkv)
        q = qkv[:, : self.q_width]
        k = qkv[:, self.q_width: self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        if self.rotary is not None:
            self.rotary.rotate(q, k, ctx)
        if writes_cache and ctx.decode_only:
            mixed = ops.decode_attention_fused(
                q, k, v, ctx.slot_mapping[cache.group], cache.k, cache.v, cache.page_stride, cache.page_size,
                cache.n_pages, ctx.block_tables[cache.group], ctx.row_entry, ctx.positions, ctx.seq_lens, self.n_heads,
                self.n_kv_heads, self.head_dim, self.scale, self.window, ctx.max_context)
            if mixed is not None:
                return ops.linear(mixed, self.w_out, self.b_out, residual=residual)
        if writes_cache and not in_cache:
            ops.kv_write(k, v, cache.k, cache.v, ctx.slot_mapping[cache.group], self.n_kv_heads, self.head_dim,
                         cache.page_size, cache.page_stride, cache.n_pages)
        mixed = ops.paged_attention(
            q, cache.k, cache.v, cache.page_stride, cache.page_size, cache.n_pages, ctx.block_tables[cache.group],
            ctx.row_entry, ctx.positions, ctx.seq_lens, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
            self.window, decode_only=ctx.decode_only, max_context=ctx.max_context, q_start=ctx.q_start,
            n_tiles=ctx.n_attention_tiles)
        return ops.linear(mixed, self.w_out, self.b_out, residual=residual)


@register_mixer("qk_norm_attention")
class QKNormAttention:
    """Grouped causal attention over the paged cache with an RMS norm of every query and key head, and,
    each chosen by a parameter: a window that keeps a sequence's first keys, a sink in the softmax's
    denominator, an output gate, a value head size of its own. No rotation; positions enter the mask only.

    params: n_heads, n_kv_heads, head_dim, v_head_dim, scale, qk_norm_eps, qk_norm_unit_offset (false: the
    norms' weights are plain gains), window (0 = none; a row at position p reads the keys (p - window, p]),
    keep_first (with a window: keys at positions below it stay visible), sink (the softmax's denominator is
    1 + the sum of the exponentials: an extra exp(0) term, so the weights sum to less than one).
    weights, all matrices stored [out, in] and without biases: w_q [H * head_dim, D], w_k [G * head_dim, D],
    w_v [G * v_head_dim, D], w_out [D, H * v_head_dim], q_norm [head_dim], k_norm [head_dim], and optionally
    w_gate [H * v_head_dim, D]: the heads' outputs are multiplied by sigmoid(w_gate h) before w_out.

    The projections of one input run as one product over the stacked matrix [q; k; v; gate]; the norms work in
    place on its query and key columns; keys are cached after their norm."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.n_heads, self.n_kv_heads = int(params["n_heads"]), int(params["n_kv_heads"])
        self.head_dim, self.v_head_dim = int(params["head_dim"]), int(params["v_head_dim"])
        self.scale = float(params["scale"])
        self.window, self.keep_first = int(params.get("window", 0)), int(params.get("keep_first", 0))
        self.sink = bool(params.get("sink", False))
        self.norm_eps = float(params["qk_norm_eps"])
        self.norm_unit_offset = bool(params.get("qk_norm_unit_offset", False))
        if self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"attention: n_heads {self.n_heads} is not a multiple of n_kv_heads {self.n_kv_heads}")
        if not (1 <= self.head_dim <= 256 and 1 <= self.v_head_dim <= 256):
            raise ValueError(f"attention: head sizes lie in 1 .. 256, got {self.head_dim} and {self.v_head_dim}")
        self.q_width, self.k_width = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        self.v_width, self.o_width = self.n_kv_heads * self.v_head_dim, self.n_heads * self.v_head_dim
        stacked = [weights["w_q"], weights["w_k"], weights["w_v"]]
        self.gated = weights.get("w_gate") is not None
        if self.gated:
            stacked.append(weights["w_gate"])
        want = [self.q_width, self.k_width, self.v_width] + ([self.o_width] if self.gated else [])
        if [w.shape[0] for w in stacked] != want or weights["w_out"].shape[1] != self.o_width:
            raise ValueError(f"attention: projections of {[tuple(w.shape) for w in stacked]} and an output of "
                             f"{tuple(weights['w_out'].shape)} do not fit {self.n_heads} heads, {self.n_kv_heads} kv heads "
                             f"of {self.head_dim} (values {self.v_head_dim})")
        self.w_in = matrix(torch.cat(stacked, dim=0), rt)
        self.w_out = matrix(weights["w_out"], rt)
        self.q_norm, self.k_norm = vector(weights["q_norm"], rt), vector(weights["k_norm"], rt)

    def matrices(self):
        return [self.w_in, self.w_out]

    @property
    def cache_spec(self) -> MemberSpec:
        return MemberSpec(self.n_kv_heads, self.head_dim, self.window, self.v_head_dim, self.keep_first)

    state_spec = None
    capturable = True

    def forward(self, h, residual, ctx, cache, state=None, writes_cache: bool = True):
        return self.forward_projected(ops.linear(h, self.w_in, None, w_is_nk=True), residual, ctx, cache, state, writes_cache)

    def input_matrix(self):
        """The stacked projections of the mixer's input, [q; k; v; gate] x D stored [out, in]: a block whose
        parts all read one normed input may run them as one product and call `forward_projected`."""
        return self.w_in

    def forward_projected(self, proj, residual, ctx, cache, state=None, writes_cache: bool = True):
        """`proj` [T, q + k + v (+ gate) columns]: the input's projections, not yet normed."""
        at = self.q_width
        q, k = proj[:, :at], proj[:, at: at + self.k_width]
        at += self.k_width
        v = proj[:, at: at + self.v_width]
        gate = proj[:, at + self.v_width: at + self.v_width + self.o_width] if self.gated else None
        fused_decode = writes_cache and ctx.decode_only and self.v_head_dim == self.head_dim
        # the norms work in place; where the attention kernel does not write the cache itself, the same launch
        # puts the normed keys and the values into the rows' slots
        scatter = None
        if writes_cache and not fused_decode:
            scatter = ops.kv_scatter(ctx.slot_mapping[cache.group], cache.k, cache.v, cache.page_stride, cache.page_size,
                                     cache.n_pages, at, self.v_width, self.v_head_dim)
        ops.head_norm(proj, self.n_heads, self.n_kv_heads, self.head_dim, self.q_norm, self.k_norm, self.norm_eps,
                      self.norm_unit_offset, kv=scatter)
        if fused_decode:
            # one new token per row: the kernel puts the new key and value into the cache itself
            mixed = ops.decode_attention_fused(
                q, k, v, ctx.slot_mapping[cache.group], cache.k, cache.v, cache.page_stride, cache.page_size,
                cache.n_pages, ctx.block_tables[cache.group], ctx.row_entry, ctx.positions, ctx.seq_lens, self.n_heads,
                self.n_kv_heads, self.head_dim, self.scale, self.window, ctx.max_context, keep_first=self.keep_first,
                sink=self.sink, gate=gate, exact_weights=ops.exact_weights())
            if mixed is not None:
                return ops.linear(mixed, self.w_out, None, w_is_nk=True, residual=residual)
            ops.kv_write(k, v, cache.k, cache.v, ctx.slot_mapping[cache.group], self.n_kv_heads, self.head_dim,
                         cache.page_size, cache.page_stride, cache.n_pages, v_head_dim=self.v_head_dim)
        mixed = ops.paged_attention(
            q, cache.k, cache.v, cache.page_stride, cache.page_size, cache.n_pages, ctx.block_tables[cache.group],
            ctx.row_entry, ctx.positions, ctx.seq_lens, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
            self.window, decode_only=ctx.decode_only, max_context=ctx.max_context, q_start=ctx.q_start,
            n_tiles=ctx.n_attention_tiles, v_head_dim=self.v_head_dim, keep_first=self.keep_first, sink=self.sink, gate=gate)
        return ops.linear(mixed, self.w_out, None, w_is_nk=True, residual=residual)


@register_mixer("rotary_window_attention")
class RotaryWindowAttention:
    """Grouped causal attention over the paged cache with, each chosen by a parameter: a rotation of queries and keys
    by position, a cap on the scores, a sliding window, a learned sink per head, one output gate per head, and a
    value head size of its own.

        q, k <- rotate(q, k): of each head the first rot_dims dimensions, dimension i paired with i + rot_dims / 2, by
                the angle position * rot_base^(-2 i / rot_dims); the other dimensions pass unchanged
        s = (q . k) * scale, then softcap * tanh(s / softcap)                   (softcap 0: no cap)
        position p sees the keys (p - window, p]                               (window 0: every key up to p)
        weights = exp(s) / (sum over seen keys of exp(s) + exp(sink[head]))     (the sink has no key and no value)
        head's output * sigmoid(w_gate h)[head], then w_out

    With `qk_norm_eps` every query and key head is RMS-normed before its rotation (weights q_norm, k_norm [head_dim], plain
    gains shared by the heads of a kind), in the rotation's launch. The rotation's frequencies are rot_base^(-2 i / rot_dims), or
    the list `rot_freqs` (stretched ones, made by the caller), with cos and sin times `rot_magnitude`. A layer without w_k and
    w_v has no keys and values of its own: it reads a cache member that another layer writes (keys as that layer cached
    them, after norm and rotation) and must be scheduled with `writes_cache=False`.

    params: n_heads, n_kv_heads, head_dim, v_head_dim, scale, softcap, window, rot_dims, rot_base | rot_freqs, rot_magnitude,
    qk_norm_eps.
    weights (matrices stored [out, in], no biases): w_q [H * head_dim, D], w_k [G * head_dim, D], w_v [G * v_head_dim, D],
    w_out [D, H * v_head_dim], and optionally sink [H], w_gate [H, D], q_norm [head_dim], k_norm [head_dim].
    Keys are cached after their rotation. Norms, angles, scores, softmax, sink and gate are computed in float32."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.n_heads, self.n_kv_heads = int(params["n_heads"]), int(params["n_kv_heads"])
        self.head_dim, self.v_head_dim = int(params["head_dim"]), int(params["v_head_dim"])
        self.scale, self.softcap = float(params["scale"]), float(params.get("softcap", 0.0))
        self.window = int(params.get("window", 0))
        self.rot_dims, self.rot_base = int(params.get("rot_dims", 0)), float(params.get("rot_base", 1.0))
        if self.n_heads % self.n_kv_heads != 0:
            raise ValueError(f"attention: n_heads {self.n_heads} is not a multiple of n_kv_heads {self.n_kv_heads}")
        if not (1 <= self.head_dim <= 256 and 1 <= self.v_head_dim <= 256):
            raise ValueError(f"attention: head sizes lie in 1 .. 256, got {self.head_dim} and {self.v_head_dim}")
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.head_dim:
            raise ValueError(f"attention: {self.rot_dims} rotated dimensions of a head of {self.head_dim}")
        self.q_width, self.k_width = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        self.v_width, self.o_width = self.n_kv_heads * self.v_head_dim, self.n_heads * self.v_head_dim
        self.own_kv = weights.get("w_k") is not None     # else: the keys and values of another layer's cache member
        stacked = [weights["w_q"], weights["w_k"], weights["w_v"]] if self.own_kv else [weights["w_q"]]
        want = [self.q_width, self.k_width, self.v_width][: len(stacked)]
        if [w.shape[0] for w in stacked] != want or weights["w_out"].shape[1] != self.o_width:
            raise ValueError(f"attention: projections of {[tuple(w.shape) for w in stacked]} and an output of "
                             f"{tuple(weights['w_out'].shape)} do not fit {self.n_heads} heads, {self.n_kv_heads} kv heads "
                             f"of {self.head_dim} (values {self.v_head_dim})")
        self.w_in = matrix(torch.cat(stacked, dim=0), rt)
        self.w_out = matrix(weights["w_out"], rt)
        self.sinks = vector(weights["sink"], rt) if weights.get("sink") is not None else None
        self.w_gate = vector(weights["w_gate"], rt) if weights.get("w_gate") is not None else None   # float32: one gate per head
        self.norm_eps = float(params["qk_norm_eps"]) if params.get("qk_norm_eps") is not None else None
        self.q_norm = self.k_norm = None
        if self.norm_eps is not None:
            self.q_norm = vector(weights["q_norm"], rt)
            self.k_norm = vector(weights["k_norm"], rt) if self.own_kv else None
            if any(w is not None and tuple(w.shape) != (self.head_dim,) for w in (self.q_norm, self.k_norm)):
                raise ValueError(f"attention: the query and key norms' weights must be [{self.head_dim}]")
        # the rotation's frequencies: exact in float64, then rounded once to float32
        half = self.rot_dims // 2
        self.rot_magnitude = float(params.get("rot_magnitude", 1.0))
        if params.get("rot_freqs") is not None:
            freqs = [float(f) for f in params["rot_freqs"]]
            if len(freqs) != half:
                raise ValueError(f"attention: {len(freqs)} frequencies for {self.rot_dims} rotated dimensions")
        else:
            freqs = [self.rot_base ** (-2.0 * i / self.rot_dims) for i in range(half)]
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(rt.device)

    def matrices(self):
        return [self.w_in, self.w_out]

    @property
    def cache_spec(self) -> MemberSpec:
        return MemberSpec(self.n_kv_heads, self.head_dim, self.window, self.v_head_dim, 0)

    state_spec = None
    capturable = True

    def _inner(self, h, ctx, cache, writes_cache):
        if writes_cache and not self.own_kv:
            raise ValueError("attention: a layer without keys and values of its own reads a cache member that another layer writes")
        proj = ops.linear(h, self.w_in, None, w_is_nk=True)
        gate = ops.small_linear(h, self.w_gate, None) if self.w_gate is not None else None
        at = self.q_width + self.k_width
        q, k, v = proj[:, : self.q_width], proj[:, self.q_width: at], proj[:, at:]
        fused_decode = ctx.decode_only and self.v_head_dim == self.head_dim
        turned = self.n_heads + (self.n_kv_heads if self.own_kv else 0)    # the heads that are normed and rotated
        norms = dict(q_norm=self.q_norm, k_norm=self.k_norm, n_q_heads=self.n_heads, norm_eps=self.norm_eps or 0.0,
                     magnitude=self.rot_magnitude)
        if writes_cache and not fused_decode:
            # the rotation's launch also puts the rotated keys and the values into the rows' cache slots
            scatter = ops.kv_scatter(ctx.slot_mapping[cache.group], cache.k, cache.v, cache.page_stride, cache.page_size,
                                     cache.n_pages, at, self.v_width, self.v_head_dim)
            ops.rotate_half(proj, turned, self.head_dim, self.rot_dims, self.inv_freq, ctx.positions,
                            kv=scatter, n_kv_heads=self.n_kv_heads, k_col=self.q_width, **norms)
        elif self.rot_dims or self.q_norm is not None:
            ops.rotate_half(proj, turned, self.head_dim, self.rot_dims, self.inv_freq, ctx.positions, **norms)
        if fused_decode:
            # one new token per row: the kernel puts the new key and value into the cache itself (a layer that reads another's
            # cache member hands it none: that layer wrote them earlier in this step)
            mixed = ops.decode_attention_fused(
                q, k if writes_cache else None, v if writes_cache else None, ctx.slot_mapping[cache.group], cache.k, cache.v, cache.page_stride,
                cache.page_size, cache.n_pages, ctx.block_tables[cache.group], ctx.row_entry, ctx.positions, ctx.seq_lens, self.n_heads,
                self.n_kv_heads, self.head_dim, self.scale, self.window, ctx.max_context, exact_weights=ops.exact_weights(), softcap=self.softcap,
                sinks=self.sinks, head_gate=gate)
            if mixed is not None:
                return mixed
            if writes_cache:
                ops.kv_write(k, v, cache.k, cache.v, ctx.slot_mapping[cache.group], self.n_kv_heads, self.head_dim,
                             cache.page_size, cache.page_stride, cache.n_pages, v_head_dim=self.v_head_dim)
        return ops.paged_attention(
            q, cache.k, cache.v, cache.page_stride, cache.page_size, cache.n_pages, ctx.block_tables[cache.group],
            ctx.row_entry, ctx.positions, ctx.seq_lens, self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
            self.window, decode_only=ctx.decode_only, max_context=ctx.max_context, q_start=ctx.q_start,
            n_tiles=ctx.n_attention_tiles, v_head_dim=self.v_head_dim, softcap=self.softcap, sinks=self.sinks, head_gate=gate)

    def mix(self, h, ctx, cache=None, state=None, writes_cache: bool = True):
        """The mixer's output [T, D] in float32, without the residual stream."""
        return ops.linear(self._inner(h, ctx, cache, writes_cache), self.w_out, None, w_is_nk=True, out_dtype=torch.float32)

    def forward(self, h, residual, ctx, cache, state=None, writes_cache: bool = True):
        return ops.linear(self._inner(h, ctx, cache, writes_cache), self.w_out, None, w_is_nk=True, residual=residual)


@register_mixer("latent_attention")
class LatentAttention:
    """Attention whose keys and values are made from ONE small latent per token, with a sliding window:

        q = W_q h, per head [head_dim plain | rot_dim rotated]
        W_dkv h = [kv_rank numbers | rot_dim numbers]: the first part, RMS-normed (weight `dkv_norm`), is the latent c; the second,
            rotated, is a key part k_rot that all heads share
        head n: k_plain = W_uk[n] c, v = W_uv[n] c; score = (q_plain . k_plain + q_rot . k_rot) * scale; softmax over the keys
            (p - window, p] (window 0: all up to p); output W_o [heads' sum_j p_j v_j]

    Rotation: of the rotated parts the first rot_dims dimensions, the pairs (2i, 2i + 1), by the angle position * rot_freqs[i],
    with cos and sin multiplied by rot_magnitude (the caller makes the frequencies: plain or stretched ones).

    Only [c | k_rot] is cached (one row per token for all heads; a member whose values lie in its key rows). The products with
    W_uk and W_uv move to the query side: q_lat = W_uk[n]^T q_plain, score = (q_lat . c + q_rot . k_rot) * scale, and
    v-side W_uv[n] (sum_j p_j c_j), so that every head reads the same cache rows: multi-query attention over rows of
    kv_rank + rot_dim numbers.

    Each chosen by what the weights hold: the queries may pass a latent of their own, q = W_uq rms_norm(W_dq h) with the weight
    `dq_norm` (`w_dq`, `dq_norm`, `w_uq` instead of `w_q`); a learned sink per head, exp(sink[n]) in the softmax's denominator
    without key or value (`sink`); an output gate, the heads' outputs times sigmoid(W_g h) element by element (`w_gate`).

    params: n_heads, head_dim, rot_dim, v_head_dim, kv_rank, scale, window, rot_dims, rot_freqs, rot_magnitude, norm_eps.
    weights (stored [out, in], no biases): w_q [H (head_dim + rot_dim), D] or w_dq [q_rank, D], dq_norm [q_rank], w_uq
    [H (head_dim + rot_dim), q_rank]; w_dkv [kv_rank + rot_dim, D], dkv_norm [kv_rank], w_uk [H head_dim, kv_rank], w_uv
    [H v_head_dim, kv_rank], w_out [D, H v_head_dim]; optionally sink [H], w_gate [H v_head_dim, D]."""

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.n_heads, self.head_dim, self.rot_dim = int(params["n_heads"]), int(params["head_dim"]), int(params["rot_dim"])
        self.v_head_dim, self.kv_rank = int(params["v_head_dim"]), int(params["kv_rank"])
        self.scale, self.window, self.norm_eps = float(params["scale"]), int(params.get("window", 0)), float(params["norm_eps"])
        self.rot_dims, self.rot_magnitude = int(params.get("rot_dims", 0)), float(params.get("rot_magnitude", 1.0))
        freqs = [float(f) for f in params.get("rot_freqs", ())]
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.rot_dim or len(freqs) != self.rot_dims // 2:
            raise ValueError(f"latent attention: {self.rot_dims} rotated dimensions of {self.rot_dim} with {len(freqs)} frequencies")
        self.q_head, self.row = self.head_dim + self.rot_dim, self.kv_rank + self.rot_dim
        H = self.n_heads
        shapes = {"w_dkv": (self.row, None), "dkv_norm": (self.kv_rank,), "w_uk": (H * self.head_dim, self.kv_rank),
                  "w_uv": (H * self.v_head_dim, self.kv_rank), "w_out": (None, H * self.v_head_dim)}
        self.q_rank = int(weights["w_dq"].shape[0]) if weights.get("w_dq") is not None else 0   # 0: queries straight from the input
        if self.q_rank:
            shapes.update({"w_dq": (self.q_rank, None), "dq_norm": (self.q_rank,), "w_uq": (H * self.q_head, self.q_rank)})
        else:
            shapes["w_q"] = (H * self.q_head, None)
        if weights.get("sink") is not None:
            shapes["sink"] = (H,)
        if weights.get("w_gate") is not None:
            shapes["w_gate"] = (H * self.v_head_dim, None)
        for name, want in shapes.items():
            have = tuple(weights[name].shape)
            if len(have) != len(want) or any(w is not None and w != g for w, g in zip(want, have)):
                raise ValueError(f"latent attention: {name} {have} does not fit {H} heads of {self.head_dim} + {self.rot_dim} "
                                 f"(values {self.v_head_dim}) over a latent of {self.kv_rank}")
        if self.row > 1024:
            raise ValueError(f"latent attention: cache rows of {self.row} numbers exceed the kernels' 1,024")
        # one product for everything that reads the layer's input: [queries or their latent | latent and key part | gate]
        self.gated = weights.get("w_gate") is not None
        stacked = [weights["w_dq"] if self.q_rank else weights["w_q"], weights["w_dkv"]] + ([weights["w_gate"]] if self.gated else [])
        self.w_in = matrix(torch.cat(stacked, dim=0), rt)
        self.kv_col = stacked[0].shape[0]
        self.w_uq = matrix(weights["w_uq"], rt) if self.q_rank else None
        self.dq_norm = vector(weights["dq_norm"], rt) if self.q_rank else None
        self.sinks = vector(weights["sink"], rt) if weights.get("sink") is not None else None
        self.w_uk, self.w_uv = matrix(weights["w_uk"], rt), matrix(weights["w_uv"], rt)
        self.w_out = matrix(weights["w_out"], rt)
        self.dkv_norm = vector(weights["dkv_norm"], rt)
        # frequencies: made in float64 by the caller, rounded once to float32
        self.freqs = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(rt.device)

    def matrices(self):
        return [self.w_in] + ([self.w_uq] if self.q_rank else []) + [self.w_uk, self.w_uv, self.w_out]

    @property
    def cache_spec(self) -> MemberSpec:
        return MemberSpec(1, self.row, self.window, self.kv_rank, 0, values_in_keys=True)

    state_spec = None
    capturable = True

    def _inner(self, h, ctx, cache, writes_cache):
        H, d, c = self.n_heads, self.head_dim, self.kv_rank
        proj = ops.linear(h, self.w_in, None, w_is_nk=True)
        queries = torch.empty(proj.shape[0], H * self.row, dtype=proj.dtype, device=proj.device)
        to_cache = dict(k_cache=cache.k if writes_cache else None, slot_mapping=ctx.slot_mapping[cache.group],
                        page_size=cache.page_size, page_stride=cache.page_stride, n_pages=cache.n_pages)
        if self.q_rank:
            # norms of both latents, the key part's rotation and the cache write: one launch; then the queries from their latent,
            # and their rotated parts turned and copied
            ops.latent_prepare(proj, 0, 0, 0, self.rot_dim, self.rot_dims, self.kv_col, c, self.dkv_norm, self.norm_eps, self.freqs,
                               self.rot_magnitude, ctx.positions, also_norm=(0, self.q_rank, self.dq_norm), **to_cache)
            q = ops.linear(proj[:, : self.q_rank], self.w_uq, None, w_is_nk=True)
            ops.latent_prepare(q, H, self.q_head, d, self.rot_dim, self.rot_dims, -1, 0, None, self.norm_eps, self.freqs,
                               self.rot_magnitude, ctx.positions, q_out=queries, q_out_head_dim=self.row, q_out_off=c)
        else:
            # norm of the latent, both rotations, the cache write and the copy of the rotated query parts: one launch
            q = proj
            ops.latent_prepare(proj, H, self.q_head, d, self.rot_dim, self.rot_dims, self.kv_col, c, self.dkv_norm, self.norm_eps,
                               self.freqs, self.rot_magnitude, ctx.positions, q_out=queries, q_out_head_dim=self.row, q_out_off=c,
                               **to_cache)
        ops.head_linear(q, self.q_head, self.w_uk, False, queries, self.row, H, d, c)
        mixed = ops.paged_attention(
            queries, cache.k, cache.k, cache.page_stride, cache.page_size, cache.n_pages, ctx.block_tables[cache.group], ctx.row_entry,
            ctx.positions, ctx.seq_lens, H, 1, self.row, self.scale, self.window, decode_only=ctx.decode_only,
            max_context=ctx.max_context, q_start=ctx.q_start, n_tiles=ctx.n_attention_tiles, v_head_dim=c, values_in_keys=True,
            sinks=self.sinks)
        out = torch.empty(proj.shape[0], H * self.v_head_dim, dtype=proj.dtype, device=proj.device)
        gate = proj[:, self.kv_col + self.row:] if self.gated else None     # the gate's columns of the input product
        ops.head_linear(mixed, c, self.w_uv, True, out, self.v_head_dim, H, c, self.v_head_dim, gate=gate)
        return out

    def mix(self, h, ctx, cache=None, state=None, writes_cache: bool = True):
        """The mixer's output [T, D] in float32, without the residual stream."""
        return ops.linear(self._inner(h, ctx, cache, writes_cache), self.w_out, None, w_is_nk=True, out_dtype=torch.float32)

    def forward(self, h, residual, ctx, cache, state=None, writes_cache: bool = True):
        return ops.linear(self._inner(h, ctx, cache, writes_cache), self.w_out, None, w_is_nk=True, residual=residual)
