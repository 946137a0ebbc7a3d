"""Norms of rows with statistics in float32: LayerNorm
(reference: kelpie-models/kelpie_models/kernels/ops/layer_norm.py:21-23) and RMS norm."""

from __future__ import annotations

from ..kernels import ops
from .base import Runtime, register_norm
from .util import vector


@register_norm("layer_norm")
class LayerNorm:
    """params: eps. weights: gamma, beta."""

    can_be_lazy = True

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.eps = float(params["eps"])
        self.gamma = vector(weights["gamma"], rt)
        self.beta = vector(weights["beta"], rt)

    def layer_norm_params(self):
        """(gain, shift, eps): for a kernel that normalises rows itself."""
        return self.gamma, self.beta, self.eps

    def forward(self, x, out_dtype, rows=None, lazy: bool = False):
        """Normalised rows in out_dtype. With `lazy` the result is an `ops.NormedRows` that a
        following `ops.linear` may compute inside its own kernel."""
        if lazy:
            return ops.NormedRows(x, self.gamma, self.beta, self.eps, out_dtype, rows=rows)
        return ops.layer_norm(x, self.gamma, self.beta, self.eps, out_dtype, rows=rows)


@register_norm("rms_norm")
class RMSNorm:
    """x / sqrt(mean(x^2) + eps) * gain. params: eps; unit_offset (the stored weight is the gain's offset from one:
    gain = 1 + weight; default false: the weight is the gain); gain_scale (default 1: a constant factor on the normalised
    rows, folded into the gain, for instance the factor on a model's logits in its last norm); width (needed where the stored
    weight is ONE number, the gain of all coordinates: it is spread over `width` coordinates here). weights: weight."""

    can_be_lazy = True

    def __init__(self, params: dict, weights: dict, rt: Runtime):
        self.eps = float(params["eps"])
        self.unit_offset = bool(params.get("unit_offset", False))
        weight = vector(weights["weight"], rt)
        if weight.dim() == 0 or (weight.numel() == 1 and "width" in params):   # one gain for all coordinates
            weight = weight.reshape(1).expand(int(params["width"])).contiguous()
        self.gain = weight + 1.0 if self.unit_offset else weight   # in float32, as the kernels would add it
        if float(params.get("gain_scale", 1.0)) != 1.0:
            self.gain = self.gain * float(params["gain_scale"])

    def forward(self, x, out_dtype, rows=None, lazy: bool = False):
        """Normalised rows in out_dtype. With `lazy` the result is an `ops.NormedRows` that a following
        `ops.linear` may compute inside its own kernel."""
        if lazy:
            return ops.NormedRows(x, self.gain, None, self.eps, out_dtype, rows=rows)
        return ops.rms_norm(x, self.gain, self.eps, out_dtype, rows=rows)
