"""The typed Pidodra configuration, read from the design's own config.json keys.

A Pidodra config.json names its model with `"architecture": "Pidodra"` and lists its layers one by one: every entry of
`layers` gives the layer's `type` (which mixer it has: `latent_attention`, attention whose keys and values are made from one
small latent per token and whose queries pass a latent of their own, or `attention`, grouped attention with normed and
rotated queries and keys), the mixer's sizes and constants (`mixer`), and its feed-forward (`mlp`: `kind` `moe`, or null for
a layer without one). Beside the layers stand `vocab`, `width`, `norm.eps`, `embedding.scale` and `postln_alpha`, the factor
on the stream inside the sum that a layer's norm follows. No size has a default: a size that is missing is an error that
names it. A mechanism that a file does not mention is not there: no `rot` is no rotation, no `rot.scaling` plain
frequencies, no `q_rank` queries straight from the input, no `kv_from` keys and values of the layer's own, no `router.groups`
one group of all experts; `embedding.scale`, `postln_alpha` and `router.scale` left out are one, `kv_heads` and `vdim` left out
equal `heads` and `dim`.
"""

from __future__ import annotations

from dataclasses import dataclass

from .registry import ConfigError
from .zirunex import _get, _int, _number
from .zudalorn import Rotation, _optional

NAME = "Pidodra"
MIXER_TYPES = ("latent_attention", "attention")
MLP_KINDS = ("moe",)


def _number_or_one(data, key: str, where: str) -> float:
    return _number(data, key, where) if isinstance(data, dict) and key in data else 1.0


@dataclass(frozen=True)
class LatentAttentionMixer:
    heads: int
    dim: int        # a head's query/key dimensions that are not rotated
    rot_dim: int    # ... and those that are; the rotated key part is one per token, shared by all heads
    vdim: int
    kv_rank: int    # size of the latent from which keys and values are made (what is cached, with the rotated key part)
    q_rank: int     # size of the latent that the queries are made from; 0: queries straight from the layer's input
    scale: float
    rot: Rotation | None

    @staticmethod
    def from_json(data: dict, where: str) -> "LatentAttentionMixer":
        rot_dim = _int(data, "rot_dim", where, minimum=0)
        rot = _optional(data, "rot")
        return LatentAttentionMixer(
            heads=_int(data, "heads", where), dim=_int(data, "dim", where, minimum=0), rot_dim=rot_dim, vdim=_int(data, "vdim", where),
            kv_rank=_int(data, "kv_rank", where), q_rank=_int(data, "q_rank", where) if data.get("q_rank") is not None else 0,
            scale=_number(data, "scale", where), rot=Rotation.from_json(rot, where + "rot.", rot_dim) if rot is not None else None)

    def to_json(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}
        if self.q_rank:
            out["q_rank"] = self.q_rank
        if self.rot is not None:
            out["rot"] = self.rot.to_json()
        return out


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotation | None
    kv_from: int | None   # the layer whose cached keys and values this layer reads; None: its own

    @staticmethod
    def from_json(data: dict, where: str) -> "AttentionMixer":
        heads, dim = _int(data, "heads", where), _int(data, "dim", where)
        kv_heads = _int(data, "kv_heads", where) if "kv_heads" in data else heads
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
        rot = _optional(data, "rot")
        return AttentionMixer(
            heads=heads, kv_heads=kv_heads, dim=dim, vdim=_int(data, "vdim", where) if "vdim" in data else dim,
            scale=_number(data, "scale", where), rot=Rotation.from_json(rot, where + "rot.", dim) if rot is not None else None,
            kv_from=_int(data, "kv_from", where, minimum=0) if data.get("kv_from") is not None else None)

    def to_json(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        if self.rot is not None:
            out["rot"] = self.rot.to_json()
        return out


@dataclass(frozen=True)
class ExpertsMlp:
    experts: int
    top: int
    ff: int             # inner width of an expert
    groups: int         # the experts form this many equal groups of neighbours ...
    keep_groups: int    # ... and only experts of the best keep_groups groups can be chosen
    scale: float        # the chosen experts' scores are multiplied by it

    @staticmethod
    def from_json(data: dict, where: str) -> "ExpertsMlp":
        kind = _get(data, "kind", where)
        if kind not in MLP_KINDS:
            raise ConfigError(f"config.json: {where}'kind' {kind!r} is not supported (supported: {', '.join(MLP_KINDS)})")
        router, expert = _get(data, "router", where), _get(data, "expert", where)
        experts, top = _int(router, "experts", where + "router."), _int(router, "top", where + "router.")
        groups_json = _optional(router, "groups")
        groups = _int(groups_json, "count", where + "router.groups.") if groups_json is not None else 1
        keep = _int(groups_json, "keep", where + "router.groups.") if groups_json is not None else 1
        if experts % groups or keep > groups:
            raise ConfigError(f"config.json: {where}router.groups: {groups} groups (keep {keep}) do not fit {experts} experts")
        if top > experts // groups * keep:
            raise ConfigError(f"config.json: {where}router.'top' ({top}) exceeds the experts that can be chosen ({experts // groups * keep})")
        return ExpertsMlp(experts=experts, top=top, ff=_int(expert, "ff", where + "expert."), groups=groups, keep_groups=keep,
                          scale=_number_or_one(router, "scale", where + "router."))

    def to_json(self) -> dict:
        return {"expert": {"ff": self.ff}, "kind": "moe",
                "router": {"experts": self.experts, "groups": {"count": self.groups, "keep": self.keep_groups}, "scale": self.scale, "top": self.top}}


@dataclass(frozen=True)
class PidodraLayer:
    type: str
    mixer: LatentAttentionMixer | AttentionMixer
    mlp: ExpertsMlp | None


@dataclass(frozen=True)
class PidodraConfig:
    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    alpha: float      # a layer's sums are norm(alpha x + sublayer(x))
    layers: tuple[PidodraLayer, ...]

    eos_token_id = None  # the design names no end-of-sequence token

    @staticmethod
    def from_json(data: dict) -> "PidodraConfig":
        layers_json = _get(data, "layers", "")
        if not isinstance(layers_json, list) or not layers_json:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: list[PidodraLayer] = []
        for i, entry in enumerate(layers_json):
            where = f"layers[{i}]."
            kind = _get(entry, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}'type' {kind!r} is not supported (supported: {', '.join(MIXER_TYPES)})")
            mixer_json = _get(entry, "mixer", where)
            mixer = (LatentAttentionMixer if kind == "latent_attention" else AttentionMixer).from_json(mixer_json, where + "mixer.")
            if isinstance(mixer, AttentionMixer) and mixer.kv_from is not None:
                j = mixer.kv_from
                lender = layers[j].mixer if j < i else None
                if not isinstance(lender, AttentionMixer) or lender.kv_from is not None:
                    raise ConfigError(f"config.json: {where}mixer.'kv_from' ({j}) must name an earlier attention layer with keys and values of its own")
                if (lender.kv_heads, lender.dim, lender.vdim, lender.rot) != (mixer.kv_heads, mixer.dim, mixer.vdim, mixer.rot):
                    raise ConfigError(f"config.json: {where}mixer: head counts, head sizes and rotation must equal those of layer {j}, whose keys it reads")
            mlp_json = entry.get("mlp")
            layers.append(PidodraLayer(kind, mixer, None if mlp_json is None else ExpertsMlp.from_json(mlp_json, where + "mlp.")))
        return PidodraConfig(vocab_size=_int(data, "vocab", ""), width=_int(data, "width", ""),
                             norm_eps=_number(_get(data, "norm", ""), "eps", "norm."),
                             embedding_scale=_number_or_one(data.get("embedding"), "scale", "embedding."),
                             alpha=_number_or_one(data, "postln_alpha", ""), layers=tuple(layers))

    def to_json(self) -> dict:
        layers = [{"mixer": layer.mixer.to_json(), "mlp": None if layer.mlp is None else layer.mlp.to_json(), "type": layer.type}
                  for layer in self.layers]
        return {"architecture": NAME, "embedding": {"scale": self.embedding_scale}, "layers": layers, "norm": {"eps": self.norm_eps},
                "postln_alpha": self.alpha, "vocab": self.vocab_size, "width": self.width}
