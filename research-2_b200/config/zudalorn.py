"""The typed Zudalorn configuration, read from the design's own config.json keys.

A Zudalorn config.json names its model with `"architecture": "Zudalorn"` and lists its layers one by one: every
entry of `layers` gives the layer's `type` (which mixer it has: `latent_attention`, attention whose keys and values are
made from one small latent per token, or `retention`, linear attention with a fixed decay per head), the mixer's sizes and
constants (`mixer`), and its feed-forward (`mlp`: `kind` `dense` or `moe`, or null for a layer without one). Beside the
layers stand `vocab`, `width` and `norm.eps`. No size has a default: a size that is missing is an error that names it. A
mechanism that a file does not mention is not there: no `mask` is no window, no `rot` no rotation, no `rot.scaling` plain
frequencies, no `router.groups` one group of all experts, no `shared` no expert that every token uses.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

from .registry import ConfigError
from .zirunex import _get, _int, _number

NAME = "Zudalorn"
MIXER_TYPES = ("latent_attention", "retention")
MLP_KINDS = ("dense", "moe")


def _optional(data, key: str):
    return data.get(key) if isinstance(data, dict) else None


@dataclass(frozen=True)
class FrequencyScaling:
    """Stretches the slow frequencies of a rotation by `factor`; frequencies that make more than `fast` turns within
    `original` positions stay as they are, those that make fewer than `slow` are divided, a linear ramp between."""

    factor: float
    original: float
    fast: float
    slow: float

    @staticmethod
    def from_json(data: dict, where: str) -> "FrequencyScaling":
        return FrequencyScaling(*(_number(data, key, where) for key in ("factor", "original", "fast", "slow")))

    def to_json(self) -> dict:
        original = int(self.original) if float(self.original).is_integer() else self.original
        return {"factor": self.factor, "fast": self.fast, "original": original, "slow": self.slow}


@dataclass(frozen=True)
class Rotation:
    dims: int      # the first `dims` dimensions of the rotated vector turn, in pairs
    base: float
    scaling: FrequencyScaling | None = None

    @staticmethod
    def from_json(data: dict, where: str, most: int) -> "Rotation":
        dims = _int(data, "dims", where, minimum=0)
        if dims % 2 or dims > most:
            raise ConfigError(f"config.json: {where}'dims' must be even and at most {most}, got {dims}")
        scaling = _optional(data, "scaling")
        return Rotation(dims, _number(data, "base", where),
                        FrequencyScaling.from_json(scaling, where + "scaling.") if scaling is not None else None)

    def to_json(self) -> dict:
        out = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = self.scaling.to_json()
        return out

    def frequencies(self) -> tuple[list[float], float]:
        """(angle per position for every pair, the factor on cos and sin), in double precision.

        Plain: f_i = base^(-2i / dims). Scaled: with n(t) = dims ln(original / (2 pi t)) / (2 ln base), the pair index at
        which a frequency makes t turns within `original` positions, lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)),
        dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1): f_i (1 - ramp_i) + f_i / factor ramp_i; cos and
        sin are multiplied by 0.1 ln(factor) + 1."""
        half = self.dims // 2
        plain = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        s = self.scaling
        if s is None:
            return plain, 1.0

        def index_of(turns: float) -> float:
            return self.dims * math.log(s.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

        lo, hi = max(math.floor(index_of(s.fast)), 0), min(math.ceil(index_of(s.slow)), self.dims - 1)
        out = []
        for i, f in enumerate(plain):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / s.factor * ramp + f * (1.0 - ramp))
        return out, 0.1 * math.log(s.factor) + 1.0


@dataclass(frozen=True)
class LatentAttentionMixer:
    heads: int
    dim: int        # a head's query/key dimensions that are not rotated
    rot_dim: int    # ... and those that are; the rotated key part is one per token, shared by all heads
    vdim: int
    kv_rank: int    # size of the latent from which keys and values are made (what is cached, with the rotated key part)
    scale: float
    window: int     # position i sees j when 0 <= i - j < window; 0: every earlier position
    rot: Rotation | None

    @staticmethod
    def from_json(data: dict, where: str) -> "LatentAttentionMixer":
        rot_dim = _int(data, "rot_dim", where, minimum=0)
        mask, rot = _optional(data, "mask"), _optional(data, "rot")
        return LatentAttentionMixer(
            heads=_int(data, "heads", where), dim=_int(data, "dim", where, minimum=0), rot_dim=rot_dim, vdim=_int(data, "vdim", where),
            kv_rank=_int(data, "kv_rank", where), scale=_number(data, "scale", where),
            window=_int(mask, "size", where + "mask.") if mask is not None and mask.get("size") is not None else 0,
            rot=Rotation.from_json(rot, where + "rot.", rot_dim) if rot is not None else None)

    def to_json(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}
        if self.window:
            out["mask"] = {"size": self.window}
        if self.rot is not None:
            out["rot"] = self.rot.to_json()
        return out


@dataclass(frozen=True)
class RetentionMixer:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]   # per head: the state is multiplied by it from token to token
    rot: Rotation | None

    @staticmethod
    def from_json(data: dict, where: str) -> "RetentionMixer":
        heads, dim = _int(data, "heads", where), _int(data, "dim", where)
        decay = _get(data, "decay", where)
        if not isinstance(decay, list) or len(decay) != heads or any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in decay):
            raise ConfigError(f"config.json: {where}'decay' must list one number per head ({heads}), got {decay!r}")
        rot = _optional(data, "rot")
        return RetentionMixer(heads=heads, dim=dim, vdim=_int(data, "vdim", where) if "vdim" in data else dim,
                              decay=tuple(float(x) for x in decay),
                              rot=Rotation.from_json(rot, where + "rot.", dim) if rot is not None else None)

    def to_json(self) -> dict:
        out = {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.rot is not None:
            out["rot"] = self.rot.to_json()
        return out


@dataclass(frozen=True)
class DenseMlp:
    ff: int

    def to_json(self) -> dict:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class ExpertsMlp:
    experts: int
    top: int
    ff: int             # inner width of a routed expert
    groups: int         # the experts form this many equal groups of neighbours ...
    keep_groups: int    # ... and only experts of the best keep_groups groups can be chosen
    shared_ff: int      # inner width of the expert that every token uses; 0: none

    def to_json(self) -> dict:
        out = {"expert": {"ff": self.ff}, "kind": "moe",
               "router": {"experts": self.experts, "groups": {"count": self.groups, "keep": self.keep_groups}, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


def _mlp_from_json(data: dict, where: str):
    kind = _get(data, "kind", where)
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: {where}'kind' {kind!r} is not supported (supported: {', '.join(MLP_KINDS)})")
    if kind == "dense":
        return DenseMlp(ff=_int(data, "ff", where))
    router, expert = _get(data, "router", where), _get(data, "expert", where)
    experts, top = _int(router, "experts", where + "router."), _int(router, "top", where + "router.")
    groups_json = _optional(router, "groups")
    groups = _int(groups_json, "count", where + "router.groups.") if groups_json is not None else 1
    keep = _int(groups_json, "keep", where + "router.groups.") if groups_json is not None else 1
    if experts % groups or keep > groups:
        raise ConfigError(f"config.json: {where}router.groups: {groups} groups (keep {keep}) do not fit {experts} experts")
    if top > experts // groups * keep:
        raise ConfigError(f"config.json: {where}router.'top' ({top}) exceeds the experts that can be chosen ({experts // groups * keep})")
    shared = _optional(data, "shared")
    return ExpertsMlp(experts=experts, top=top, ff=_int(expert, "ff", where + "expert."), groups=groups, keep_groups=keep,
                      shared_ff=_int(shared, "ff", where + "shared.") if shared is not None else 0)


@dataclass(frozen=True)
class ZudalornLayer:
    type: str
    mixer: LatentAttentionMixer | RetentionMixer
    mlp: DenseMlp | ExpertsMlp | None


@dataclass(frozen=True)
class ZudalornConfig:
    vocab_size: int
    width: int
    norm_eps: float
    layers: tuple[ZudalornLayer, ...]

    eos_token_id = None  # the design names no end-of-sequence token

    @staticmethod
    def from_json(data: dict) -> "ZudalornConfig":
        layers_json = _get(data, "layers", "")
        if not isinstance(layers_json, list) or not layers_json:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_json):
            where = f"layers[{i}]."
            kind = _get(entry, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}'type' {kind!r} is not supported (supported: {', '.join(MIXER_TYPES)})")
            mixer_json = _get(entry, "mixer", where)
            mixer = (LatentAttentionMixer if kind == "latent_attention" else RetentionMixer).from_json(mixer_json, where + "mixer.")
            mlp_json = entry.get("mlp")
            layers.append(ZudalornLayer(kind, mixer, None if mlp_json is None else _mlp_from_json(mlp_json, where + "mlp.")))
        return ZudalornConfig(vocab_size=_int(data, "vocab", ""), width=_int(data, "width", ""),
                              norm_eps=_number(_get(data, "norm", ""), "eps", "norm."), layers=tuple(layers))

    def to_json(self) -> dict:
        layers = [{"mixer": layer.mixer.to_json(), "mlp": None if layer.mlp is None else layer.mlp.to_json(), "type": layer.type}
                  for layer in self.layers]
        return {"architecture": NAME, "layers": layers, "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.width}
