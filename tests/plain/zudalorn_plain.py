"""Zudalorn, stated plainly: one function per mechanism, float64, a Python loop per token where the design
has a recurrence or a window. Nothing here is shared with the engine; the tests compare the engine with it.

A model is a dict of tensors by checkpoint name and the config.json dict. Notation: h [T, D] is a sublayer's
input, rows are the positions 0 .. T - 1 of ONE sequence.
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


# A test may set this to a function that disturbs every normalised row on its way into a sublayer (and into the head):
# how far the logits of a position move under small disturbances says how well-conditioned the position is.
DISTURB = None
# A test may set this to a list: every router then appends, per position, how narrowly its choice was made (the smallest
# gap between something chosen and something not, among experts and among groups).
MARGINS = None


def scalar_norm(x, g, eps, entering=False):
    """RMS norm whose gain is ONE number for all coordinates."""
    out = unit_rms(x, eps) * float(g)
    return DISTURB(out) if (entering and DISTURB is not None) else out


# ---- rotations ---------------------------------------------------------------------------------
def plain_frequencies(dims, base):
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def yarn_frequencies(dims, base, scaling):
    """-> (frequencies, the factor on cos and sin). Frequencies that turn fast (short wavelengths) stay, slow ones
    are divided by `factor`, with a linear ramp over the pair index between the two corner indices."""
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def corner(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(corner(float(scaling["fast"]))), 0)
    hi = min(math.ceil(corner(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(dims, base)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, layout, magnitude=1.0):
    """x [T, ..., n]: the first 2 * len(freqs) dimensions are rotated pair by pair, the rest pass.
    layout "interleaved": (2i, 2i + 1); "half": (i, i + len(freqs))."""
    half = len(freqs)
    out = x.clone()
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


# ---- latent attention --------------------------------------------------------------------------
def latent_attention(h, w, p, cfg, eps):
    """Queries per head [dim plain | rot_dim rotated]; keys and values are made from a latent of kv_rank numbers per
    token, plus ONE rotated key part per token that all heads share. Sliding window, ordinary softmax."""
    T = h.shape[0]
    H, d, r, dv, c_dim = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    rot = cfg.get("rot")
    if not rot:
        freqs, mag = [], 1.0
    elif rot.get("scaling"):
        freqs, mag = yarn_frequencies(rot["dims"], rot["base"], rot["scaling"])
    else:
        freqs, mag = plain_frequencies(rot["dims"], rot["base"]), 1.0
    pos = list(range(T))
    q = lin(w[p + "q"], h).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], pos, freqs, "interleaved", mag)
    down = lin(w[p + "dkv"], h)
    latent = unit_rms(down[:, :c_dim], eps) * w[p + "dkv.norm"].to(F64)
    k_rot = rotate(down[:, c_dim:], pos, freqs, "interleaved", mag)                 # [T, r], one for all heads
    k_plain = lin(w[p + "uk"], latent).view(T, H, d)
    v = lin(w[p + "uv"], latent).view(T, H, dv)
    window = cfg.get("mask", {}).get("size") if cfg.get("mask") else None
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        first = 0 if not window else max(0, i - window + 1)
        s = (torch.einsum("hd,jhd->hj", q_plain[i], k_plain[first: i + 1])
             + torch.einsum("hr,jr->hj", q_rot[i], k_rot[first: i + 1])) * cfg["scale"]
        out[i] = torch.einsum("hj,jhv->hv", torch.softmax(s, dim=-1), v[first: i + 1])
    return lin(w[p + "o"], out.reshape(T, H * dv))


# ---- retention ---------------------------------------------------------------------------------
def retention_cells(q, k, v, decay):
    """S <- decay S + k v^T, o = S^T q, from S = 0. q, k [T, H, d], v [T, H, dv], decay [H] -> [T, H, dv]."""
    T, H, d = k.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=F64)
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def retention(h, w, p, cfg, eps):
    T = h.shape[0]
    H, d, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    q, k = lin(w[p + "q"], h).view(T, H, d), lin(w[p + "k"], h).view(T, H, d)
    v = lin(w[p + "v"], h).view(T, H, dv)
    rot = cfg.get("rot")
    if rot:
        freqs, pos = plain_frequencies(rot["dims"], rot["base"]), list(range(T))
        q, k = rotate(q, pos, freqs, "half"), rotate(k, pos, freqs, "half")
    k = k * d ** -0.5
    o = retention_cells(q, k, v, torch.tensor(cfg["decay"], dtype=F64))
    o = unit_rms(o, eps).reshape(T, H * dv)
    gate = lin(w[p + "g"], h)
    return lin(w[p + "o"], o * gate * torch.sigmoid(gate))


# ---- feed-forwards -----------------------------------------------------------------------------
def xielu(z, p, q):
    """For z > 0: softplus(p) z^2 + z / 2; else (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
    sp, sq = math.log1p(math.exp(p)), math.log1p(math.exp(q))
    neg = torch.clamp(z, max=0.0)
    return torch.where(z > 0, sp * z * z + 0.5 * z, (0.5 + sq) * (torch.expm1(neg) - neg) + 0.5 * z)


def dense(h, w, p):
    a, b = (float(x) for x in w[p + "act"].to(F64))
    return lin(w[p + "down"], xielu(lin(w[p + "up"], h), a, b))


def gated_unit(h, w, p):
    g = lin(w[p + "gate"], h)
    return lin(w[p + "down"], g * torch.sigmoid(g) * lin(w[p + "up"], h))


def route(z, correction, top, n_groups, keep):
    """z [T, E] router logits -> (chosen [T, top], weights [T, top]). Choice by sigmoid + correction inside the best
    `keep` of `n_groups` groups of neighbours (a group counts by the sum of its two best choice scores); weights are
    the chosen experts' plain sigmoids over their sum."""
    T, E = z.shape
    s = torch.sigmoid(z)
    choice = s + correction.to(F64)
    chosen, weights, margins = [], [], []
    size = E // n_groups
    for t in range(T):
        c = choice[t].clone()
        margin = math.inf
        if keep < n_groups:
            marks = [float(torch.topk(c[g * size: (g + 1) * size], min(2, size)).values.sum()) for g in range(n_groups)]
            ranked = sorted(range(n_groups), key=lambda g: (-marks[g], g))
            margin = marks[ranked[keep - 1]] - marks[ranked[keep]]
            for g in ranked[keep:]:
                c[g * size: (g + 1) * size] = -math.inf
        ranked = sorted(range(E), key=lambda e: (-float(c[e]), e))
        order = ranked[:top]
        if top < E and float(c[ranked[top]]) > -math.inf:
            margin = min(margin, float(c[ranked[top - 1]] - c[ranked[top]]))
        margins.append(margin)
        sel = s[t][order]
        chosen.append(order)
        weights.append(sel / (sel.sum() + 1e-20))
    if MARGINS is not None:
        MARGINS.append(torch.tensor(margins, dtype=F64))
    return chosen, weights


def experts(h, w, p, cfg):
    r = cfg["router"]
    z = lin(w[p + "router"], h)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    chosen, weights = route(z, w[p + "correction"], r["top"], groups["count"], groups["keep"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            out[t] += wt * gated_unit(h[t: t + 1], w, f"{p}e{e}.")[0]
    if cfg.get("shared"):
        out = out + torch.sigmoid(lin(w[p + "shared.sg"], h)) * gated_unit(h, w, p + "shared.")
    return out


# ---- the model ---------------------------------------------------------------------------------
def forward(config, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence; `layers_out` (a list) receives the stream after every layer."""
    eps = config["norm"]["eps"]
    x = w["embed"].to(F64)[torch.tensor(tokens)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = scalar_norm(x, w[p + "norm1"], eps, entering=True)
        mixer = latent_attention if layer["type"] == "latent_attention" else retention
        x = x + scalar_norm(mixer(h, w, p + "mix.", layer["mixer"], eps), w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = scalar_norm(x, w[p + "norm2"], eps, entering=True)
            y = dense(h, w, p + "mlp.") if layer["mlp"]["kind"] == "dense" else experts(h, w, p + "mlp.", layer["mlp"])
            x = x + scalar_norm(y, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(w["head"], scalar_norm(x, w["final.norm"], eps, entering=True))


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
