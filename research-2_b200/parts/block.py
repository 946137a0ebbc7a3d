"""Arrangements of norms, a mixer and a feed-forward around the float32 residual stream."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import register_block


@register_block("pre_norm")
class PreNormBlock:
    """x + mixer(norm_1 x), then x + feed_forward(norm_2 x); both additions happen in the
    epilogue of each part's last matrix product
    (kelpie-models/kelpie_models/models/torch/gpt2.py:91-97)."""

    def __init__(self, norm_1, mixer, norm_2, feed_forward, compute_dtype):
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward
        self.compute_dtype = compute_dtype

    def forward(self, x, ctx, cache=None, state=None, writes_cache: bool = True):
        h = self._normed(self.norm_1, x, self.mixer)
        x = self.mixer.forward(h, x, ctx, cache, state, writes_cache)
        if self.feed_forward is None:   # a layer without a feed-forward (and without a second norm)
            return x
        h = self._normed(self.norm_2, x, self.feed_forward)
        return self.feed_forward.forward(h, x, ctx)

    def resident_layer(self) -> dict | None:
        """What the one-kernel form of a decode step (parts/resident.py) needs to know of this layer, or
        None if one of its parts is not of a kind that the kernel is written for."""
        asks = (getattr(self.norm_1, "layer_norm_params", None), getattr(self.mixer, "resident_attention", None),
                getattr(self.norm_2, "layer_norm_params", None), getattr(self.feed_forward, "resident_mlp", None))
        if any(ask is None for ask in asks):
            return None
        n1, attention, n2, mlp = (ask() for ask in asks)
        if attention is None or mlp is None or attention["width"] != mlp["width"]:
            return None
        return {**attention, **mlp, "ln1_g": n1[0], "ln1_b": n1[1], "eps1": n1[2], "ln2_g": n2[0], "ln2_b": n2[1], "eps2": n2[2]}

    def _normed(self, norm, x, consumer):
        """A part that says `takes_lazy_norm` gets the norm unevaluated and may fuse it into its
        first matrix product; any other part gets a tensor."""
        if getattr(consumer, "takes_lazy_norm", False) and getattr(norm, "can_be_lazy", False):
            return norm.forward(x, self.compute_dtype, lazy=True)
        return norm.forward(x, self.compute_dtype)


@register_block("parallel")
class ParallelBlock:
    """x + mixer(h) + feed_forward(h) with h = norm_1(x): one norm, and both sublayers read its output. Each
    sublayer's last matrix product adds its result to the float32 stream that it is handed, the mixer's to x
    and the feed-forward's to that sum. A layer may have no feed-forward (None); there is no second norm."""

    def __init__(self, norm_1, mixer, norm_2, feed_forward, compute_dtype):
        if norm_2 is not None:
            raise ValueError("a parallel block has one norm")
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, None, feed_forward
        self.compute_dtype = compute_dtype
        # Both sublayers read the same h: where each offers the stacked matrix of its input projections
        # (`input_matrix` / `forward_projected`), the block runs them as ONE product over both stacks. The
        # parts keep views into the joint matrix, so they still work on their own.
        self.w_in = None
        ask = [getattr(p, "input_matrix", None) for p in (mixer, feed_forward)]
        if feed_forward is not None and all(ask):
            a, b = ask[0](), ask[1]()
            if a.dtype == b.dtype and a.shape[1] == b.shape[1] and a.device == b.device:
                self.w_in = torch.cat([a, b], dim=0)
                self.split = a.shape[0]
                mixer.w_in, feed_forward.w_gate_up = self.w_in[: self.split], self.w_in[self.split:]

    def forward(self, x, ctx, cache=None, state=None, writes_cache: bool = True):
        if self.w_in is not None:
            # (the norm stays a kernel of its own: computed inside the joint product's kernel, where every CTA of a
            # product several thousand columns wide normalises the rows again, a decode step of 8 rows and 12
            # layers measured 0.48 ms against 0.40)
            h = self.norm_1.forward(x, self.compute_dtype)
            proj = ops.linear(h, self.w_in, None, w_is_nk=True)
            x = self.mixer.forward_projected(proj[:, : self.split], x, ctx, cache, state, writes_cache)
            return self.feed_forward.forward_projected(proj[:, self.split:], x, ctx)
        h = self.norm_1.forward(x, self.compute_dtype)
        x = self.mixer.forward(h, x, ctx, cache, state, writes_cache)
        if self.feed_forward is not None:
            x = self.feed_forward.forward(h, x, ctx)
        return x


@register_block("sandwich")
class SandwichBlock:
    """A norm before AND after each sublayer: x + post_1(mixer(norm_1 x)), then x + post_2(feed_forward(norm_2 x)). The
    sublayers hand over their output in float32 without the stream (`mix`); one launch normalises it, adds it to the stream
    and, after the mixer, also gives the feed-forward's normed input. The post norms are RMS norms (`gain`, `eps`). A layer
    may have no feed-forward (None; then no norm_2 and no post_norm_2)."""

    def __init__(self, norm_1, mixer, norm_2, feed_forward, compute_dtype, post_norm_1=None, post_norm_2=None):
        if post_norm_1 is None or (feed_forward is not None and (norm_2 is None or post_norm_2 is None)):
            raise ValueError("a sandwich block needs a norm after every sublayer that it has")
        for part, what in ((mixer, "mixer"), (feed_forward, "feed-forward")):
            if part is not None and not hasattr(part, "mix"):
                raise ValueError(f"a sandwich block's {what} must offer `mix` (its output without the stream)")
        for norm in (post_norm_1, post_norm_2, norm_2):
            if norm is not None and not hasattr(norm, "gain"):
                raise ValueError("a sandwich block's norms after the sublayers, and the one between them, must be RMS norms")
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward
        self.post_norm_1, self.post_norm_2 = post_norm_1, post_norm_2
        self.compute_dtype = compute_dtype

    def forward(self, x, ctx, cache=None, state=None, writes_cache: bool = True):
        h = self.norm_1.forward(x, self.compute_dtype)
        y = self.mixer.mix(h, ctx, cache, state, writes_cache)
        if self.feed_forward is None:
            return ops.norm_add(x, y, self.post_norm_1.gain, self.post_norm_1.eps)
        x, h = ops.norm_add(x, y, self.post_norm_1.gain, self.post_norm_1.eps, self.norm_2.gain, self.norm_2.eps, self.compute_dtype)
        y = self.feed_forward.mix(h, ctx)
        return ops.norm_add(x, y, self.post_norm_2.gain, self.post_norm_2.eps)


@register_block("post_norm")
class PostNormBlock:
    """The norm AFTER each sum: x <- norm_1(alpha x + mixer(x)), then x <- norm_2(alpha x + feed_forward(x)). The sublayers read
    the stream itself (in the compute dtype) and hand over their output in float32 without it (`mix`); one launch scales the
    stream, adds the output, normalises the sum and writes the new rows twice: in float32 (the stream) and in the compute
    dtype (what the next sublayer's products read). The norms are RMS norms (`gain`, `eps`). A layer may have no feed-forward
    (None; then no norm_2). `alpha` is the factor on the stream inside the sums.

    The compute-dtype copy of the rows that this block returns travels to the next block in `ctx.stream_rounded` as the pair
    (stream tensor, its copy); a block that is handed another tensor (the embedding's rows) makes the copy itself."""

    def __init__(self, norm_1, mixer, norm_2, feed_forward, compute_dtype, alpha: float = 1.0):
        if feed_forward is not None and norm_2 is None:
            raise ValueError("a post-norm block needs a norm after every sublayer that it has")
        for part, what in ((mixer, "mixer"), (feed_forward, "feed-forward")):
            if part is not None and not hasattr(part, "mix"):
                raise ValueError(f"a post-norm block's {what} must offer `mix` (its output without the stream)")
        for norm in (norm_1, norm_2):
            if norm is not None and not hasattr(norm, "gain"):
                raise ValueError("a post-norm block's norms must be RMS norms")
        self.norm_1, self.mixer, self.norm_2, self.feed_forward = norm_1, mixer, norm_2, feed_forward
        self.compute_dtype, self.alpha = compute_dtype, float(alpha)
        self.rounds = compute_dtype != torch.float32

    def _read(self, x, ctx):
        """The stream's rows as the sublayers' products read them."""
        if not self.rounds:
            return x
        carried = getattr(ctx, "stream_rounded", None)
        if carried is not None and carried[0] is x:
            return carried[1]
        return ops.round_rows(x, self.compute_dtype)

    def _join(self, x, y, norm):
        if not self.rounds:
            x = ops.add_norm(x, y, self.alpha, norm.gain, norm.eps)
            return x, x
        return ops.add_norm(x, y, self.alpha, norm.gain, norm.eps, self.compute_dtype)

    def forward(self, x, ctx, cache=None, state=None, writes_cache: bool = True):
        h = self._read(x, ctx)
        x, h = self._join(x, self.mixer.mix(h, ctx, cache, state, writes_cache), self.norm_1)
        if self.feed_forward is not None:
            x, h = self._join(x, self.feed_forward.mix(h, ctx), self.norm_2)
        ctx.stream_rounded = (x, h)
        return x
