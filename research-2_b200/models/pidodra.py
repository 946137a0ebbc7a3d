"""Pidodra as data: its tensor names, its random initialisation, and its ModelSpec.

A decoder whose norms come AFTER the sums (parts/block.py: `post_norm`): x <- norm1(alpha x + mixer(x)), then
x <- norm2(alpha x + feed_forward(x)), RMS norms with a gain per coordinate; the sublayers read the stream itself. The token
table's rows are scaled on their way in; the head is a table of its own behind one more norm. A layer's mixer is attention
over a latent cache whose queries pass a latent of their own, with a learned sink per head and an output gate element by
element (parts/attention.py: `latent_attention`), or grouped attention with normed and rotated queries and keys, stretched
rotation frequencies and one gate per head (`rotary_window_attention` with `qk_norm_eps`); such a layer may read the cached keys
and values of an earlier one instead of making its own (a schedule entry that names the other layer's cache member and does
not write it). The feed-forward is a mixture of gated silu experts chosen by softmax scores inside the best groups of experts
(parts/mlp.py: `routed_experts` with `scoring: softmax`).

Tensor names (matrices stored [out, in]): `embed`, `head`, `final.norm`, and for layer i `l<i>.norm1`, with a feed-forward
`l<i>.norm2`, the mixer's under `l<i>.mix.` and the feed-forward's under `l<i>.mlp.`:
  latent_attention  dq dq.norm uq (or q) dkv dkv.norm uk uv sink g o
  attention         q k v q.norm k.norm g o  (no k, v, k.norm where the layer reads another's keys and values)
  moe               e<j>.{gate up down}, router
"""

from __future__ import annotations

import torch

from ..config.pidodra import NAME, LatentAttentionMixer, PidodraConfig
from ..config.registry import Architecture, register_architecture
from ..parts import LayerSpec, PartSpec, Runtime
from ..weights.loader import TensorSpec, WeightSpec
from .decoder import DecoderModel, ModelSpec, ScheduleEntry

# No mixer limits a sequence's length (rotations take any position): the engine's options bound it.
UNBOUNDED_SEQ_LEN = 1 << 30


def _mixer_names(layer, p: str, width: int) -> dict[str, tuple[str, tuple[int, ...]]]:
    """The mixer part's weight name -> (tensor name, shape)."""
    def entry(name, *shape):
        return (f"{p}.mix.{name}", tuple(shape))

    m = layer.mixer
    if isinstance(m, LatentAttentionMixer):
        q_head = m.dim + m.rot_dim
        if m.q_rank:
            out = {"w_dq": entry("dq", m.q_rank, width), "dq_norm": entry("dq.norm", m.q_rank), "w_uq": entry("uq", m.heads * q_head, m.q_rank)}
        else:
            out = {"w_q": entry("q", m.heads * q_head, width)}
        out.update({"w_dkv": entry("dkv", m.kv_rank + m.rot_dim, width), "dkv_norm": entry("dkv.norm", m.kv_rank),
                    "w_uk": entry("uk", m.heads * m.dim, m.kv_rank), "w_uv": entry("uv", m.heads * m.vdim, m.kv_rank),
                    "sink": entry("sink", m.heads), "w_gate": entry("g", m.heads * m.vdim, width), "w_out": entry("o", width, m.heads * m.vdim)})
        return out
    out = {"w_q": entry("q", m.heads * m.dim, width)}
    if m.kv_from is None:
        out.update({"w_k": entry("k", m.kv_heads * m.dim, width), "w_v": entry("v", m.kv_heads * m.vdim, width)})
    out["q_norm"] = entry("q.norm", m.dim)
    if m.kv_from is None:
        out["k_norm"] = entry("k.norm", m.dim)
    out.update({"w_gate": entry("g", m.heads, width), "w_out": entry("o", width, m.heads * m.vdim)})
    return out


def _mlp_names(layer, p: str, width: int) -> dict[str, tuple[str, tuple[int, ...]]]:
    mlp, out = layer.mlp, {}
    for j in range(mlp.experts):
        out.update({f"e{j}.w_gate": (f"{p}.mlp.e{j}.gate", (mlp.ff, width)), f"e{j}.w_up": (f"{p}.mlp.e{j}.up", (mlp.ff, width)),
                    f"e{j}.w_down": (f"{p}.mlp.e{j}.down", (width, mlp.ff))})
    out["router"] = (f"{p}.mlp.router", (mlp.experts, width))
    return out


def weight_spec(cfg: PidodraConfig) -> WeightSpec:
    d = cfg.width
    tensors = [TensorSpec("embed", (cfg.vocab_size, d))]
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        tensors += [TensorSpec(f"{p}.{name}", (d,)) for name in (("norm1", "norm2") if layer.mlp is not None else ("norm1",))]
        tensors += [TensorSpec(name, shape) for name, shape in _mixer_names(layer, p, d).values()]
        if layer.mlp is not None:
            tensors += [TensorSpec(name, shape) for name, shape in _mlp_names(layer, p, d).values()]
    tensors += [TensorSpec("final.norm", (d,)), TensorSpec("head", (cfg.vocab_size, d))]
    return WeightSpec(tensors=tuple(tensors))


def random_weights(cfg: PidodraConfig, seed: int, std: float = 0.05, norm_std: float = 0.1) -> dict[str, torch.Tensor]:
    """Float32 draws from ONE CPU generator, in the order of `weight_spec`: matrices and tables N(0, std) (those over a latent
    or over the heads' outputs by their input's size, so that queries, keys and values keep their size); gains 1 + N(0,
    norm_std); sinks N(0, 1)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for ts in weight_spec(cfg).tensors:
        draw = torch.randn(ts.shape, generator=gen, dtype=torch.float32)
        if len(ts.shape) == 2:
            out[ts.name] = (std if ts.shape[1] >= cfg.width else ts.shape[1] ** -0.5) * draw
        elif ts.name.endswith(".sink"):
            out[ts.name] = draw
        else:
            out[ts.name] = 1.0 + norm_std * draw
    return out


def model_spec(cfg: PidodraConfig) -> ModelSpec:
    eps, d = cfg.norm_eps, cfg.width
    layers, schedule, member_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        weights = {own: name for own, (name, _) in _mixer_names(layer, p, d).items()}
        freqs, magnitude = m.rot.frequencies() if m.rot is not None else ([], 1.0)
        rot_dims = m.rot.dims if m.rot is not None else 0
        if isinstance(m, LatentAttentionMixer):
            mixer = PartSpec("latent_attention", {
                "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale,
                "window": 0, "rot_dims": rot_dims, "rot_freqs": freqs, "rot_magnitude": magnitude, "norm_eps": eps}, weights)
        else:
            mixer = PartSpec("rotary_window_attention", {
                "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim, "scale": m.scale, "window": 0,
                "rot_dims": rot_dims, "rot_freqs": freqs, "rot_magnitude": magnitude, "qk_norm_eps": eps}, weights)
        # every layer with keys and values of its own gets a cache member; a layer that reads another's names that member
        lender = getattr(m, "kv_from", None)
        if lender is None:
            member_of[i] = len(member_of)
            schedule.append(ScheduleEntry(layer=i, cache=member_of[i], writes_cache=True))
        else:
            schedule.append(ScheduleEntry(layer=i, cache=member_of[lender], writes_cache=False))
        feed_forward = norm_2 = None
        if layer.mlp is not None:
            e = layer.mlp
            feed_forward = PartSpec("routed_experts", {
                "n_experts": e.experts, "top": e.top, "scoring": "softmax", "n_groups": e.groups, "keep_groups": e.keep_groups,
                "group_mark": "best", "normalise": False, "route_scale": e.scale, "activation": "silu"},
                {own: name for own, (name, _) in _mlp_names(layer, p, d).items()})
            norm_2 = PartSpec("rms_norm", {"eps": eps}, {"weight": f"{p}.norm2"})
        layers.append(LayerSpec(block="post_norm", mixer=mixer, feed_forward=feed_forward,
                                norm_1=PartSpec("rms_norm", {"eps": eps}, {"weight": f"{p}.norm1"}), norm_2=norm_2,
                                block_params={"alpha": cfg.alpha}))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden=d, max_seq_len=UNBOUNDED_SEQ_LEN, eos_token=None, embedding="embed", head="head",
        positions=None, layers=tuple(layers), final_norm=PartSpec("rms_norm", {"eps": eps}, {"weight": "final.norm"}),
        schedule=tuple(schedule), embedding_scale=cfg.embedding_scale)


def build(cfg: PidodraConfig, tensors: dict[str, torch.Tensor], rt: Runtime) -> DecoderModel:
    return DecoderModel(model_spec(cfg), tensors, rt, config=cfg)


PIDODRA = register_architecture(Architecture(
    name=NAME, parse_config=PidodraConfig.from_json, weight_spec=weight_spec, random_weights=random_weights,
    build=build, config_to_json=PidodraConfig.to_json,
))
