"""Zudalorn as data: its tensor names, its random initialisation, and its ModelSpec.

A decoder with a norm before AND after each sublayer (parts/block.py: `sandwich`): x + norm1b(mixer(norm1 x)), then
x + norm2b(feed_forward(norm2 x)); every one of these norms, and the last one, is an RMS norm whose gain is ONE number. A
layer's mixer is attention over a latent cache with a sliding window and stretched rotation frequencies
(parts/attention.py: `latent_attention`) or retention, linear attention with a fixed decay per head and a state of fixed size
(parts/recurrent.py: `retention`). Its feed-forward is W_down xIELU(W_up h) (parts/mlp.py: `act_mlp`) or a mixture of gated
silu experts chosen by sigmoid scores inside the best groups of experts, plus one gated expert that every token uses
(`routed_experts` with `scoring: sigmoid`). The head is a table of its own.

Tensor names (matrices stored [out, in]): `embed`, `head`, `final.norm`, and for layer i `l<i>.norm1`, `l<i>.norm1b`, and with
a feed-forward `l<i>.norm2`, `l<i>.norm2b` (all of shape []), the mixer's under `l<i>.mix.` and the feed-forward's under
`l<i>.mlp.`:
  latent_attention  q dkv dkv.norm uk uv o
  retention         q k v g o
  dense             up down act
  moe               e<j>.{gate up down}, router, correction, shared.{gate up down sg}
"""

from __future__ import annotations

import torch

from ..config.registry import Architecture, register_architecture
from ..config.zudalorn import NAME, DenseMlp, ExpertsMlp, LatentAttentionMixer, ZudalornConfig
from ..parts import LayerSpec, PartSpec, Runtime
from ..weights.loader import TensorSpec, WeightSpec
from .decoder import DecoderModel, ModelSpec

# Neither mixer limits a sequence's length (a window and a state of fixed size): the engine's options bound it.
UNBOUNDED_SEQ_LEN = 1 << 30


def _mixer_names(layer, p: str, width: int) -> dict[str, tuple[str, tuple[int, ...]]]:
    """The mixer part's weight name -> (tensor name, shape)."""
    def entry(name, *shape):
        return (f"{p}.mix.{name}", tuple(shape))

    m = layer.mixer
    if isinstance(m, LatentAttentionMixer):
        return {"w_q": entry("q", m.heads * (m.dim + m.rot_dim), width), "w_dkv": entry("dkv", m.kv_rank + m.rot_dim, width),
                "dkv_norm": entry("dkv.norm", m.kv_rank), "w_uk": entry("uk", m.heads * m.dim, m.kv_rank),
                "w_uv": entry("uv", m.heads * m.vdim, m.kv_rank), "w_out": entry("o", width, m.heads * m.vdim)}
    return {"w_q": entry("q", m.heads * m.dim, width), "w_k": entry("k", m.heads * m.dim, width), "w_v": entry("v", m.heads * m.vdim, width),
            "w_gate": entry("g", m.heads * m.vdim, width), "w_out": entry("o", width, m.heads * m.vdim)}


def _mlp_names(layer, p: str, width: int) -> dict[str, tuple[str, tuple[int, ...]]]:
    def unit(own: str, stored: str, ff: int):
        return {f"{own}w_gate": (f"{p}.mlp.{stored}gate", (ff, width)), f"{own}w_up": (f"{p}.mlp.{stored}up", (ff, width)),
                f"{own}w_down": (f"{p}.mlp.{stored}down", (width, ff))}

    mlp = layer.mlp
    if isinstance(mlp, DenseMlp):
        return {"w_up": (f"{p}.mlp.up", (mlp.ff, width)), "w_down": (f"{p}.mlp.down", (width, mlp.ff)), "act": (f"{p}.mlp.act", (2,))}
    out = {}
    for j in range(mlp.experts):
        out.update(unit(f"e{j}.", f"e{j}.", mlp.ff))
    out.update({"router": (f"{p}.mlp.router", (mlp.experts, width)), "correction": (f"{p}.mlp.correction", (mlp.experts,))})
    if mlp.shared_ff:
        out.update(unit("shared.", "shared.", mlp.shared_ff))
        out["shared.w_sg"] = (f"{p}.mlp.shared.sg", (1, width))
    return out


def weight_spec(cfg: ZudalornConfig) -> WeightSpec:
    d = cfg.width
    tensors = [TensorSpec("embed", (cfg.vocab_size, d))]
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        norms = ("norm1", "norm2", "norm1b", "norm2b") if layer.mlp is not None else ("norm1", "norm1b")
        tensors += [TensorSpec(f"{p}.{name}", ()) for name in norms]
        tensors += [TensorSpec(name, shape) for name, shape in _mixer_names(layer, p, d).values()]
        if layer.mlp is not None:
            tensors += [TensorSpec(name, shape) for name, shape in _mlp_names(layer, p, d).values()]
    tensors += [TensorSpec("final.norm", ()), TensorSpec("head", (cfg.vocab_size, d))]
    return WeightSpec(tensors=tuple(tensors))


def random_weights(cfg: ZudalornConfig, seed: int, std: float = 0.05, norm_std: float = 0.1) -> dict[str, torch.Tensor]:
    """Float32 draws from ONE CPU generator, in the order of `weight_spec`: matrices and tables N(0, std) (the small
    matrices over a latent wider, so that keys and values keep their size); gains 1 + N(0, norm_std), those after a sublayer
    smaller; router corrections and the activations' numbers small."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for ts in weight_spec(cfg).tensors:
        draw = torch.randn(ts.shape, generator=gen, dtype=torch.float32)
        last = ts.name.rsplit(".", 1)[-1]
        if len(ts.shape) == 2:
            out[ts.name] = (std if ts.shape[1] >= cfg.width else ts.shape[1] ** -0.5) * draw
        elif last in ("norm1", "norm2", "norm"):
            out[ts.name] = 1.0 + norm_std * draw
        elif last in ("norm1b", "norm2b"):
            out[ts.name] = 0.5 + norm_std * draw
        elif last == "correction":
            out[ts.name] = 0.1 * draw
        else:
            out[ts.name] = 0.5 * draw      # the two numbers of an activation
    return out


def model_spec(cfg: ZudalornConfig) -> ModelSpec:
    eps, d = cfg.norm_eps, cfg.width
    one_gain = {"eps": eps, "width": d}    # a stored gain of shape [] is spread over the width
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        weights = {own: name for own, (name, _) in _mixer_names(layer, p, d).items()}
        freqs, magnitude = m.rot.frequencies() if m.rot is not None else ([], 1.0)
        rot_dims = m.rot.dims if m.rot is not None else 0
        if isinstance(m, LatentAttentionMixer):
            mixer = PartSpec("latent_attention", {
                "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale,
                "window": min(m.window, UNBOUNDED_SEQ_LEN), "rot_dims": rot_dims, "rot_freqs": freqs, "rot_magnitude": magnitude,
                "norm_eps": eps}, weights)
        else:
            # retention's rotation has no factor on cos and sin: a stretched rotation there keeps its frequencies only
            mixer = PartSpec("retention", {
                "n_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim, "decay": list(m.decay), "rot_dims": rot_dims,
                "rot_freqs": freqs, "norm_eps": eps}, weights)
        feed_forward = norm_2 = post_2 = None
        if layer.mlp is not None:
            ff_weights = {own: name for own, (name, _) in _mlp_names(layer, p, d).items()}
            if isinstance(layer.mlp, DenseMlp):
                feed_forward = PartSpec("act_mlp", {"activation": "xielu"}, ff_weights)
            else:
                e: ExpertsMlp = layer.mlp
                feed_forward = PartSpec("routed_experts", {
                    "n_experts": e.experts, "top": e.top, "scoring": "sigmoid", "n_groups": e.groups, "keep_groups": e.keep_groups,
                    "activation": "silu", "shared": bool(e.shared_ff)}, ff_weights)
            norm_2 = PartSpec("rms_norm", one_gain, {"weight": f"{p}.norm2"})
            post_2 = PartSpec("rms_norm", one_gain, {"weight": f"{p}.norm2b"})
        layers.append(LayerSpec(block="sandwich", mixer=mixer, feed_forward=feed_forward,
                                norm_1=PartSpec("rms_norm", one_gain, {"weight": f"{p}.norm1"}), norm_2=norm_2,
                                post_norm_1=PartSpec("rms_norm", one_gain, {"weight": f"{p}.norm1b"}), post_norm_2=post_2))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden=d, max_seq_len=UNBOUNDED_SEQ_LEN, eos_token=None, embedding="embed", head="head",
        positions=None, layers=tuple(layers), final_norm=PartSpec("rms_norm", one_gain, {"weight": "final.norm"}))


def build(cfg: ZudalornConfig, tensors: dict[str, torch.Tensor], rt: Runtime) -> DecoderModel:
    return DecoderModel(model_spec(cfg), tensors, rt, config=cfg)


ZUDALORN = register_architecture(Architecture(
    name=NAME, parse_config=ZudalornConfig.from_json, weight_spec=weight_spec, random_weights=random_weights,
    build=build, config_to_json=ZudalornConfig.to_json,
))
