"""Pidodra, stated plainly: one function per mechanism, float64, a Python loop per token where a softmax runs over
the earlier positions. Nothing here is shared with the engine; the tests compare the engine with it.

A model is a dict of tensors by checkpoint name and the config.json dict. Notation: h [T, D] is a sublayer's input,
rows are the positions 0 .. T - 1 of ONE sequence. The stream is normalised AFTER every sum:
x <- norm1(alpha x + mixer(x)), x <- norm2(alpha x + experts(x)).
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def lin(w, h):
    """Matrices are stored [out, in]."""
    return h @ w.to(F64).T


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return unit_rms(x, eps) * gain.to(F64)


# A test may set this to a function that disturbs the stream's rows on their way into every sublayer (and into the head):
# how far the logits of a position move under small disturbances says how well-conditioned the position is.
DISTURB = None
# A test may set this to a list: every router then appends, per position, how narrowly its choice was made (the smallest
# gap between something chosen and something not, among experts and among groups).
MARGINS = None


# ---- rotations ---------------------------------------------------------------------------------
def frequencies(rot):
    """-> (angle per position of every pair, the factor on cos and sin)."""
    dims, base = rot["dims"], float(rot["base"])
    plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return plain, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def corner(turns):   # the pair index whose frequency makes `turns` turns within `original` positions
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(corner(float(scaling["fast"]))), 0)
    hi = min(math.ceil(corner(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(plain):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, layout, magnitude=1.0):
    """x [T, ..., n]: the first 2 * len(freqs) dimensions are rotated pair by pair, the rest pass.
    layout "interleaved": (2i, 2i + 1); "half": (i, i + len(freqs))."""
    half = len(freqs)
    out = x.clone()
    if half == 0:
        return out
    ang = torch.tensor(positions, dtype=F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]   # [T, half]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    cos, sin = torch.cos(ang) * magnitude, torch.sin(ang) * magnitude
    if layout == "interleaved":
        u, v = x[..., 0: 2 * half: 2], x[..., 1: 2 * half: 2]
        out[..., 0: 2 * half: 2] = u * cos - v * sin
        out[..., 1: 2 * half: 2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half: 2 * half]
        out[..., :half] = u * cos - v * sin
        out[..., half: 2 * half] = v * cos + u * sin
    return out


def softmax_with_sink(s, sink=None):
    """s [H, J] scores of the keys a position sees -> weights [H, J]. With `sink` [H] the denominator holds exp(sink) too:
    a term without key or value, so the weights sum to less than one."""
    if sink is None:
        return torch.softmax(s, dim=-1)
    top = torch.maximum(s.max(dim=-1).values, sink)
    e = torch.exp(s - top[:, None])
    return e / (e.sum(dim=-1) + torch.exp(sink - top))[:, None]


# ---- latent attention --------------------------------------------------------------------------
def latent_keys_values(h, w, p, cfg, eps, positions):
    """What a layer caches per token: the normed latent c [T, kv_rank] and the rotated key part [T, rot_dim]."""
    c_dim = cfg["kv_rank"]
    freqs, mag = frequencies(cfg["rot"]) if cfg.get("rot") else ([], 1.0)
    down = lin(w[p + "dkv"], h)
    return rms_norm(down[:, :c_dim], w[p + "dkv.norm"], eps), rotate(down[:, c_dim:], positions, freqs, "interleaved", mag)


def latent_attention(h, w, p, cfg, eps):
    """Queries from a normed latent of their own, per head [dim plain | rot_dim rotated]; keys and values from a latent of
    kv_rank numbers per token plus ONE rotated key part that all heads share. Every earlier position is seen; a sink per
    head in the softmax; the heads' outputs times sigmoid(W_g h), element by element."""
    T = h.shape[0]
    H, d, r, dv = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"]
    pos = list(range(T))
    freqs, mag = frequencies(cfg["rot"]) if cfg.get("rot") else ([], 1.0)
    if cfg.get("q_rank"):
        q = lin(w[p + "uq"], rms_norm(lin(w[p + "dq"], h), w[p + "dq.norm"], eps)).view(T, H, d + r)
    else:
        q = lin(w[p + "q"], h).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], pos, freqs, "interleaved", mag)
    latent, k_rot = latent_keys_values(h, w, p, cfg, eps, pos)
    k_plain = lin(w[p + "uk"], latent).view(T, H, d)
    v = lin(w[p + "uv"], latent).view(T, H, dv)
    sink = w[p + "sink"].to(F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        s = (torch.einsum("hd,jhd->hj", q_plain[i], k_plain[: i + 1]) + torch.einsum("hr,jr->hj", q_rot[i], k_rot[: i + 1])) * cfg["scale"]
        out[i] = torch.einsum("hj,jhv->hv", softmax_with_sink(s, sink), v[: i + 1])
    gate = torch.sigmoid(lin(w[p + "g"], h))
    return lin(w[p + "o"], out.reshape(T, H * dv) * gate)


# ---- grouped attention --------------------------------------------------------------------------
def attention_keys_values(h, w, p, cfg, eps):
    """What a layer caches per token: keys [T, G, dim] after their norm and rotation, values [T, G, vdim]."""
    T = h.shape[0]
    d = cfg["dim"]
    G, dv = cfg.get("kv_heads", cfg["heads"]), cfg.get("vdim", d)
    freqs, mag = frequencies(cfg["rot"]) if cfg.get("rot") else ([], 1.0)
    k = rms_norm(lin(w[p + "k"], h).view(T, G, d), w[p + "k.norm"], eps)
    return rotate(k, list(range(T)), freqs, "half", mag), lin(w[p + "v"], h).view(T, G, dv)


def attention(h, w, p, cfg, eps, keys_values=None):
    """Grouped attention: an RMS norm of every query and key head, rotation of a head's first rot.dims dimensions (i with
    i + dims / 2), ordinary softmax over every earlier position, one sigmoid gate per head. With `keys_values` the layer
    has no keys and values of its own and reads another layer's."""
    T = h.shape[0]
    H, d = cfg["heads"], cfg["dim"]
    G, dv = cfg.get("kv_heads", H), cfg.get("vdim", d)
    freqs, mag = frequencies(cfg["rot"]) if cfg.get("rot") else ([], 1.0)
    q = rms_norm(lin(w[p + "q"], h).view(T, H, d), w[p + "q.norm"], eps)
    q = rotate(q, list(range(T)), freqs, "half", mag)
    k, v = keys_values if keys_values is not None else attention_keys_values(h, w, p, cfg, eps)
    per = H // G                                       # query head n uses key/value head n // per
    k_of, v_of = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        s = torch.einsum("jhd,hd->hj", k_of[: i + 1], q[i]) * cfg["scale"]
        out[i] = torch.einsum("hj,jhv->hv", torch.softmax(s, dim=-1), v_of[: i + 1])
    gate = torch.sigmoid(lin(w[p + "g"], h))          # [T, H]
    return lin(w[p + "o"], (out * gate[:, :, None]).reshape(T, H * dv)), (k, v)


# ---- mixture of experts -------------------------------------------------------------------------
def gated_unit(h, w, p):
    g = lin(w[p + "gate"], h)
    return lin(w[p + "down"], g * torch.sigmoid(g) * lin(w[p + "up"], h))


def route(z, top, n_groups, keep, scale):
    """z [T, E] router logits -> (chosen [T, top], weights [T, top]). Scores are the softmax over ALL experts; a group of
    neighbours counts by its largest score; inside the best `keep` groups the `top` largest scores are chosen; their weights
    are the scores times `scale` (they are not made to sum to one)."""
    T, E = z.shape
    s = torch.softmax(z, dim=-1)
    size = E // n_groups
    chosen, weights, margins = [], [], []
    for t in range(T):
        c = s[t].clone()
        margin = math.inf
        if keep < n_groups:
            marks = [float(c[g * size: (g + 1) * size].max()) for g in range(n_groups)]
            ranked = sorted(range(n_groups), key=lambda g: (-marks[g], g))
            margin = marks[ranked[keep - 1]] - marks[ranked[keep]]
            for g in ranked[keep:]:
                c[g * size: (g + 1) * size] = -math.inf
        ranked = sorted(range(E), key=lambda e: (-float(c[e]), e))
        if top < E and float(c[ranked[top]]) > -math.inf:
            margin = min(margin, float(c[ranked[top - 1]] - c[ranked[top]]))
        margins.append(margin)
        chosen.append(ranked[:top])
        weights.append(s[t][ranked[:top]] * scale)
    if MARGINS is not None:
        MARGINS.append(torch.tensor(margins, dtype=F64))
    return chosen, weights


def experts(h, w, p, cfg):
    r = cfg["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    chosen, weights = route(lin(w[p + "router"], h), r["top"], groups["count"], groups["keep"], float(r.get("scale", 1.0)))
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            out[t] += wt * gated_unit(h[t: t + 1], w, f"{p}e{e}.")[0]
    return out


# ---- the model ---------------------------------------------------------------------------------
def forward(config, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence; `layers_out` (a list) receives the stream after every layer."""
    eps, alpha = config["norm"]["eps"], float(config["postln_alpha"])
    def read(rows):
        return DISTURB(rows) if DISTURB is not None else rows

    eps, alpha = config["norm"]["eps"], float(config.get("postln_alpha", 1.0))
    x = w["embed"].to(F64)[torch.tensor(tokens)] * float((config.get("embedding") or {}).get("scale", 1.0))
    cached = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "latent_attention":
            y = latent_attention(read(x), w, p + "mix.", m, eps)
        else:
            y, cached[i] = attention(read(x), w, p + "mix.", m, eps, cached[m["kv_from"]] if m.get("kv_from") is not None else None)
        x = rms_norm(alpha * x + y, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = rms_norm(alpha * x + experts(read(x), w, p + "mlp.", layer["mlp"]), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(w["head"], read(rms_norm(x, w["final.norm"], eps)))


def read_model(folder):
    """(config.json as a dict, tensors by name in float64)."""
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), {n: t.to(F64) for n, t in load_file(str(folder / "model.safetensors")).items()}


def generate(config: dict, w: dict, prompt: list[int], n_new: int) -> list[int]:
    """Greedy continuation, recomputing the whole sequence for every token (first index on ties)."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(config, w, seq)[-1].argmax()))
    return seq[len(prompt):]
