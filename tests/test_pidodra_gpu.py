"""Pidodra on the GPU against the plain implementation (tests/plain/pidodra_plain.py): each mechanism alone, one key
that stands out far back, at pages' borders and at a sequence's first token, then whole models through the step function
and the cache manager in every cutting, then generation through the engine."""

from __future__ import annotations

import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import traces
from tests.pidodra_cases import CASES, assert_close_to_plain, attention, latent, layer, make_model_dir, model, plain_logits, random_case, random_tokens
from tests.plain import pidodra_plain as plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
F64 = torch.float64

LENGTHS = {"a": (70, 45, 128, 33, 2, 97), "b": (60, 9, 41, 3, 77, 50, 30), "c": (150, 66, 5, 90, 17, 2, 120, 64), "d": (90, 66, 5, 131, 40)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: make_model_dir(tmp_path_factory.mktemp(f"pd_{name}"), case) for name, case in CASES.items()}


def requests_for(name: str) -> dict[str, list[int]]:
    vocab = CASES[name]["config"]["vocab"]
    return {f"r{i}": random_tokens(300 + i, n, vocab) for i, n in enumerate(LENGTHS[name])}


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def tol_of(dtype):
    return 3e-5 if dtype == torch.float32 else 3e-2


def close(got, want, dtype, what=""):
    err = float((got.double().cpu() - want).abs().max())
    assert err <= tol_of(dtype) * max(1.0, float(want.abs().max())), (what, err)


# ---------------------------------------------------------------------------------------------
# each mechanism alone


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_with_softmax_scores_and_groups(dtype):
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(1)
    shapes = [  # rows, width, experts, top, groups, kept groups, factor on the weights
        (37, 40, 6, 2, 3, 1, 2.0), (9, 64, 8, 4, 4, 3, 1.0), (130, 96, 3, 3, 1, 1, 0.5), (4, 200, 33, 4, 11, 3, 2.5), (50, 24, 12, 4, 2, 1, 1.0),
        (21, 32, 5, 2, 5, 3, 3.0), (64, 48, 16, 8, 4, 4, 1.0), (17, 16, 2, 1, 2, 1, 0.1),
    ]
    for rows, width, experts, top, groups, keep, factor in shapes:
        h = torch.randn(rows, width, generator=gen).to(dtype)
        w = (torch.randn(experts, width, generator=gen) * 0.4).to(torch.bfloat16).float()
        z = h.double() @ w.double().T
        plain.MARGINS = []
        try:
            want_chosen, want_weights = plain.route(z, top, groups, keep, factor)
            clear = plain.MARGINS[0] > 1e-5
        finally:
            plain.MARGINS = None
        dense, chosen, weight, gates = ops.route_scored(h.to(DEV), w.to(DEV), None, top, groups, keep, scoring="softmax", group_mark="best",
                                                        normalise=False, weight_scale=factor)
        assert gates is None and int(clear.sum()) > rows // 2
        for t in range(rows):
            if not bool(clear[t]):
                continue
            got = dict(zip(chosen[t].cpu().tolist(), weight[t].cpu().tolist()))
            assert sorted(got) == sorted(want_chosen[t]), (rows, t, got, want_chosen[t])
            for e, wt in zip(want_chosen[t], want_weights[t].tolist()):
                assert abs(got[e] - wt) < 1e-5 * max(1.0, factor) and abs(float(dense[t, e]) - wt) < 1e-5 * max(1.0, factor)
            assert int((dense[t] != 0).sum()) == top
        if top == experts:   # every expert chosen: the scores of a softmax sum to one, the weights to the factor
            assert float((dense.sum(dim=1) - factor).abs().max()) < 1e-5 * max(1.0, factor)
    # equal logits: the lower index wins, among groups and among experts; every score is 1 / 6
    h = torch.zeros(3, 16, dtype=dtype)
    _, chosen, weight, _ = ops.route_scored(h.to(DEV), torch.zeros(6, 16, device=DEV), None, 2, 3, 1, scoring="softmax", group_mark="best",
                                            normalise=False, weight_scale=3.0)
    assert [sorted(r) for r in chosen.cpu().tolist()] == [[0, 1]] * 3 and torch.allclose(weight.cpu(), torch.full((3, 2), 0.5))
    # a group counts by its best expert alone: logits (2, -2 | 1.8, 1.8 | -1, 3) keep groups 2 and 0, although group 1's two scores sum to more
    w = torch.zeros(6, 16)
    w[:, 0] = torch.tensor([2.0, -2.0, 1.8, 1.8, -1.0, 3.0])
    h = torch.zeros(1, 16, dtype=dtype)
    h[0, 0] = 1.0
    _, chosen, _, _ = ops.route_scored(h.to(DEV), w.to(DEV), None, 3, 3, 2, scoring="softmax", group_mark="best", normalise=False)
    assert sorted(chosen[0].cpu().tolist()) == [0, 4, 5]
    _, chosen, _, _ = ops.route_scored(h.to(DEV), w.to(DEV), None, 3, 3, 2, scoring="softmax", group_mark="two_best", normalise=False)
    assert sorted(chosen[0].cpu().tolist()) == [2, 3, 5], "the other mark, for comparison"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_norm_after_a_sum(dtype):
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(2)
    rows = 23
    for width, alpha, eps in ((50, 2.5, 1e-6), (64, 1.0, 1e-3), (3, 0.5, 1e-5), (2048, 2.0, 1e-6), (2500, 4.0, 1e-6)):
        x, y = torch.randn(rows, width, generator=gen), torch.randn(rows, width, generator=gen) * 5
        x[3], y[3] = 0.0, 0.0     # a row of zeros stays zero: eps stands inside the root
        gain = 1.0 + 0.3 * torch.randn(width, generator=gen)
        want = plain.rms_norm(alpha * x.double() + y.double(), gain, eps)
        got = ops.add_norm(x.to(DEV), y.to(DEV), alpha, gain.to(DEV), eps)
        assert got.dtype == torch.float32 and float((got.double().cpu() - want).abs().max()) < 1e-5 * max(1.0, float(want.abs().max()))
        assert float(got[3].abs().max()) == 0.0
        new, rounded = ops.add_norm(x.to(DEV), y.to(DEV), alpha, gain.to(DEV), eps, dtype)
        assert torch.equal(new, got) and rounded.dtype == dtype and torch.equal(rounded, new.to(dtype)), "the copy is the stream, rounded once"
        assert torch.equal(ops.round_rows(new, dtype), new.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 2, 16, 16, 8), (1, 1, 24, 8, 40), (6, 2, 64, 64, 64), (8, 1, 32, 0, 32), (3, 3, 80, 30, 16), (5, 0, 12, 12, 12)])
def test_head_norms_and_rotation_in_one_launch(dtype, shape):
    """Every query and key head by its own root mean square times a gain per kind, then the rotation of the first dimensions
    (i with i + dims / 2) with a magnitude on cos and sin, and the cache write of the turned keys and the values; a row
    without keys (a layer that reads another's) has its queries alone normed and turned."""
    from research_2_b200.kernels import ops

    heads, kv_heads, dim, rot_dims, vdim = shape
    gen = torch.Generator().manual_seed(7)
    rows, page, eps, magnitude = 61, 4, 1e-5, 1.14
    q_w, k_w = heads * dim, kv_heads * dim
    proj = (torch.randn(rows, q_w + k_w + kv_heads * vdim + 3, generator=gen) * 2).to(dtype)
    positions = torch.randint(0, 3000, (rows,), generator=gen).tolist()
    freqs = [900.0 ** (-2.0 * i / max(rot_dims, 1)) for i in range(rot_dims // 2)]
    gq, gk = 1.0 + 0.3 * torch.randn(dim, generator=gen), 1.0 + 0.3 * torch.randn(dim, generator=gen)
    want_q = plain.rotate(plain.rms_norm(proj[:, :q_w].double().view(rows, heads, dim), gq, eps), positions, freqs, "half", magnitude)
    n_pages = 20
    dev = proj.to(DEV)
    inv_freq = torch.tensor(freqs, dtype=F64).float().to(DEV)
    kv = None
    if kv_heads:
        want_k = plain.rotate(plain.rms_norm(proj[:, q_w: q_w + k_w].double().view(rows, kv_heads, dim), gk, eps), positions, freqs, "half", magnitude)
        slots = (torch.randperm((n_pages - 1) * page, generator=gen)[:rows] + page).to(torch.int32).to(DEV)
        # (keys and values in pools of their own here, both laid out with ONE page stride, as the kernel takes it)
        stride = kv_heads * page * max(dim, vdim)
        k_cache = torch.full((n_pages * stride,), 7.0, dtype=dtype, device=DEV)
        v_cache = torch.full((n_pages * stride,), 7.0, dtype=dtype, device=DEV)
        kv = ops.kv_scatter(slots, k_cache, v_cache, stride, page, n_pages, q_w + k_w, kv_heads * vdim, vdim)
    ops.rotate_half(dev, heads + kv_heads, dim, rot_dims, inv_freq, i32(positions), kv=kv, n_kv_heads=kv_heads, k_col=q_w,
                    q_norm=gq.to(DEV), k_norm=gk.to(DEV) if kv_heads else None, n_q_heads=heads, norm_eps=eps, magnitude=magnitude)
    angle_tol = 3e-3 if dtype == torch.float32 else 6e-2   # the angle is a float32 product of a position in the thousands
    got = dev.double().cpu()
    assert float((got[:, :q_w].view(rows, heads, dim) - want_q).abs().max()) <= angle_tol
    assert torch.equal(got[:, q_w + k_w:], proj[:, q_w + k_w:].double()), "values and the columns after them changed"
    if kv_heads:
        assert float((got[:, q_w: q_w + k_w].view(rows, kv_heads, dim) - want_k).abs().max()) <= angle_tol
        for t in (0, rows // 2, rows - 1):
            pg, off = int(slots[t]) // page, int(slots[t]) % page
            for g in range(kv_heads):
                at = pg * stride + (g * page + off) * dim
                assert torch.equal(k_cache[at: at + dim], dev[t, q_w + g * dim: q_w + (g + 1) * dim]), "the cached key is the turned key"
                at = pg * stride + (g * page + off) * vdim
                assert torch.equal(v_cache[at: at + vdim], dev[t, q_w + k_w + g * vdim: q_w + k_w + (g + 1) * vdim])
        assert float(k_cache[:stride].min()) == 7.0 and float(v_cache[:stride].min()) == 7.0, "the null page was written"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 16, 8, 32, 24, 24), (1, 20, 4, 44, 12, 50), (3, 12, 6, 10, 20, 7), (6, 64, 32, 96, 80, 48), (2, 8, 16, 8, 8, 130)])
def test_latent_rows_with_a_latent_for_the_queries(dtype, shape):
    """The two launches around the queries' up-projection: norms of both latents, the key part's rotation and the cache row in
    the first (the rows hold no query heads yet); the heads' rotated parts turned and copied in the second (the rows hold
    nothing else). Then the values' small products with a gate in their epilogue."""
    from research_2_b200.kernels import ops

    heads, dim, rot_dim, rank, vdim, q_rank = shape
    gen = torch.Generator().manual_seed(6)
    rows, page, eps, magnitude = 83, 4, 1e-4, 1.17
    q_head, row = dim + rot_dim, rank + rot_dim
    proj = torch.randn(rows, q_rank + row + heads * vdim, generator=gen).to(dtype)
    positions = torch.randint(0, 3000, (rows,), generator=gen).tolist()
    freqs = [300.0 ** (-2.0 * i / rot_dim) for i in range(rot_dim // 2)]
    f32 = torch.tensor(freqs, dtype=F64).float().to(DEV)
    wq, wc = 1.0 + 0.3 * torch.randn(q_rank, generator=gen), torch.randn(rank, generator=gen)
    want_cq = plain.rms_norm(proj[:, :q_rank].double(), wq, eps)
    want_c = plain.rms_norm(proj[:, q_rank: q_rank + rank].double(), wc, eps)
    want_k_rot = plain.rotate(proj[:, q_rank + rank: q_rank + row].double(), positions, freqs, "interleaved", magnitude)
    n_pages = 24
    cache = torch.full((n_pages * page * row,), 7.0, dtype=dtype, device=DEV)
    slots = torch.randperm((n_pages - 1) * page, generator=gen)[:rows] + page
    dev = proj.to(DEV)
    ops.latent_prepare(dev, 0, 0, 0, rot_dim, rot_dim, q_rank, rank, wc.to(DEV), eps, f32, magnitude, i32(positions), k_cache=cache,
                       slot_mapping=slots.to(torch.int32).to(DEV), page_size=page, page_stride=page * row, n_pages=n_pages,
                       also_norm=(0, q_rank, wq.to(DEV)))
    angle_tol = 2e-3 if dtype == torch.float32 else 4e-2
    got = dev.double().cpu()
    close(dev[:, :q_rank], want_cq, dtype, "the queries' latent")
    close(dev[:, q_rank: q_rank + rank], want_c, dtype, "latent")
    assert float((got[:, q_rank + rank: q_rank + row] - want_k_rot).abs().max()) <= angle_tol
    assert torch.equal(got[:, q_rank + row:], proj[:, q_rank + row:].double()), "the gate's columns changed"
    stored = cache.view(n_pages * page, row)[slots.to(DEV)]
    assert torch.equal(stored, dev[:, q_rank: q_rank + row]), "the cache row is the prepared row"
    assert float(cache.view(n_pages * page, row)[:page].min()) == 7.0, "the null page was written"
    # the second launch: query heads alone
    q = torch.randn(rows, heads * q_head, generator=gen).to(dtype)
    want_q_rot = plain.rotate(q.double().view(rows, heads, q_head)[..., dim:], positions, freqs, "interleaved", magnitude)
    queries = torch.zeros(rows, heads * row, dtype=dtype, device=DEV)
    qd = q.to(DEV)
    ops.latent_prepare(qd, heads, q_head, dim, rot_dim, rot_dim, -1, 0, None, eps, f32, magnitude, i32(positions), q_out=queries,
                       q_out_head_dim=row, q_out_off=rank)
    assert float((qd.double().cpu().view(rows, heads, q_head)[..., dim:] - want_q_rot).abs().max()) <= angle_tol
    assert torch.equal(qd.view(rows, heads, q_head)[..., :dim], q.to(DEV).view(rows, heads, q_head)[..., :dim]), "the plain query parts changed"
    assert torch.equal(queries.view(rows, heads, row)[..., rank:], qd.view(rows, heads, q_head)[..., dim:])
    # out = sigmoid(gate) * W_uv[h] mixed
    mixed = torch.randn(rows, heads * rank, generator=gen).to(dtype)
    w_uv = (torch.randn(heads * vdim, rank, generator=gen) * 0.3).to(dtype)
    out = torch.zeros(rows, heads * vdim, dtype=dtype, device=DEV)
    gate = dev[:, q_rank + row:]
    ops.head_linear(mixed.to(DEV), rank, w_uv.to(DEV), True, out, vdim, heads, rank, vdim, gate=gate)
    want = torch.einsum("thc,hvc->thv", mixed.double().view(rows, heads, rank), w_uv.double().view(heads, vdim, rank)).reshape(rows, -1)
    close(out, want * torch.sigmoid(gate.double().cpu()), dtype, "gated values")


def plain_attention_over_latents(q, rows_of, positions, kv_rank, scale, sinks):
    """q [T, H, row] float64, rows_of[t]: the cache rows [len, row] of the token's sequence, positions[t]: the token's place.
    Head h of token t: softmax with a sink over the keys up to p of scale * q . row, times the rows' first kv_rank numbers."""
    out = torch.zeros(q.shape[0], q.shape[1], kv_rank, dtype=F64)
    for t in range(q.shape[0]):
        keys = rows_of[t][: positions[t] + 1]
        out[t] = plain.softmax_with_sink((q[t] @ keys.T) * scale, sinks) @ keys[:, :kv_rank]
    return out


# heads, cache row, latent's part of it, page size
LATENT_SHAPES = [(12, 160, 128, 16), (3, 40, 24, 8), (5, 33, 20, 3), (70, 48, 48, 32), (1, 256, 200, 16), (16, 96, 64, 64)]


@pytest.mark.parametrize("cut", ["prompts", "decoded", "portions", "many"])
@pytest.mark.parametrize("shape", LATENT_SHAPES)
def test_attention_over_a_cache_of_latents_with_sinks(shape, cut):
    """The bfloat16 kernel whose tiles hold all heads of a few tokens, alone, with a learned term per head in the softmax's
    denominator (some far above every score, some far below, some among them): entries of unequal lengths whose pages lie
    scattered in a pool full of large numbers, as whole prompts, single decoded tokens, portions that start in the middle,
    and 42 entries of which every other one is a single token."""
    from research_2_b200.kernels import ops

    heads, row, rank, page = shape
    gen = torch.Generator().manual_seed(heads * 1000 + row)
    lengths = [1, 2, 63, 64, 65, 130, 200] * (6 if cut == "many" else 1)
    scale = 1.0 / math.sqrt(row)
    sinks = torch.randn(heads, generator=gen) * 2
    sinks[0] = 30.0
    sinks[-1] = -30.0
    per_seq = [(torch.randn(n, row, generator=gen) * 1.5).to(torch.bfloat16) for n in lengths]
    table_width = max(-(-n // page) for n in lengths)
    n_pages = 1 + len(lengths) * table_width
    order = (torch.randperm(n_pages - 1, generator=gen) + 1).tolist()
    cache = torch.full((n_pages, page, row), 300.0, dtype=torch.bfloat16)
    tables = torch.zeros(len(lengths), table_width, dtype=torch.int32)
    for e, (n, rows_) in enumerate(zip(lengths, per_seq)):
        for b in range(-(-n // page)):
            tables[e, b] = order.pop()
            piece = rows_[b * page: (b + 1) * page]
            cache[tables[e, b], : piece.shape[0]] = piece
    if cut == "prompts":
        spans = [(0, n) for n in lengths]
    elif cut == "decoded":
        spans = [(n - 1, n) for n in lengths]
    elif cut == "many":
        spans = [(n - 1, n) if e % 2 else (n // 3, n - n // 4) for e, n in enumerate(lengths)]
    else:
        spans = [(n // 3, n - n // 4) for n in lengths]
    entry_rows = [b - a for a, b in spans]
    q_start = [sum(entry_rows[:i]) for i in range(len(lengths) + 1)]
    positions = [p for a, b in spans for p in range(a, b)]
    row_entry = [e for e, (a, b) in enumerate(spans) for _ in range(a, b)]
    q = (torch.randn(len(positions), heads * row, generator=gen) * 1.5).to(torch.bfloat16)
    want = plain_attention_over_latents(q.double().view(-1, heads, row), [per_seq[e].double() for e in row_entry], positions, rank, scale, sinks.double())
    args = (cache.to(DEV), cache.to(DEV), page * row, page, n_pages, tables.to(DEV), i32(row_entry), i32(positions),
            i32([b for _, b in spans]), heads, 1, row, scale, 0)
    kwargs = dict(decode_only=cut == "decoded", max_context=max(lengths), q_start=i32(q_start), n_tiles=sum(-(-r // 64) for r in entry_rows),
                  v_head_dim=rank, values_in_keys=True, sinks=sinks.to(DEV))
    before = ops.kernel_uses().get("latent_attention", 0)
    got = ops.paged_attention(q.to(DEV), *args, **kwargs)
    assert ops.kernel_uses().get("latent_attention", 0) == before + 1, "another kernel took the call"
    close(got.view(-1, heads, rank), want, torch.bfloat16, f"{shape} {cut}")
    if heads > 1:
        assert float(got.view(-1, heads, rank)[:, 0].abs().max()) < 0.01 * float(want[:, -1].abs().max()), "a sink far above every score takes nearly all"
    # the general kernel (what float32 runs on) gives the same
    old = ops.use_fast_attention(False)
    try:
        slow = ops.paged_attention(q.to(DEV), *args, **kwargs)
    finally:
        ops.use_fast_attention(old)
    close(slow.view(-1, heads, rank), want, torch.bfloat16, f"{shape} {cut} on the general kernel")


# ---------------------------------------------------------------------------------------------
# one key that stands out: far back, at pages' borders, at the first token


QUERY_TOKEN, KEY_TOKEN = 1, 2


def _write(folder: Path, config: dict, w: dict) -> Path:
    from research_2_b200.config.registry import architecture_of
    from research_2_b200.weights.safetensors_io import write_file

    arch = architecture_of(config)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(arch.config_to_json(arch.parse_config(config))))
    write_file(folder / "model.safetensors", {n: t.to(torch.bfloat16) for n, t in w.items()})
    return folder


def _planted_embedding(w):
    """Coordinate 0 of the stream is the asking token's alone, coordinate 1 the planted token's."""
    w["embed"][:, :2] = 0.0
    w["embed"][QUERY_TOKEN] *= 0.1
    w["embed"][KEY_TOKEN] *= 0.1
    w["embed"][QUERY_TOKEN, 0] = 6.0
    w["embed"][KEY_TOKEN, 1] = 6.0


def planted_latent_model(folder: Path) -> Path:
    """One layer of latent attention whose weights are made so that the token QUERY_TOKEN asks, in head 0, for exactly the key
    that the token KEY_TOKEN leaves in the cache: coordinate 0 of the stream drives the queries' latent, coordinate 1 the keys'
    latent, and W_uq turns the one into a multiple of W_uk applied to the other. Such a key's weight in the softmax is nearly
    one wherever it is visible (the sinks are small beside it), so the logits at the asking position say whether it was seen."""
    from research_2_b200 import models  # noqa: F401  (registers the architectures)
    from research_2_b200.config.registry import architecture_of

    heads, dim, rot_dim, vdim, rank, q_rank, width = 2, 16, 8, 16, 24, 12, 32
    config = model(64, width, [layer(latent(heads, dim, rot_dim, vdim, rank, 0.2, q_rank=q_rank, rot=(8, 10000.0)))], eps=1e-5, alpha=0.05)
    arch = architecture_of(config)
    w = arch.random_weights(arch.parse_config(config), 17, std=0.08)
    gen = torch.Generator().manual_seed(18)
    _planted_embedding(w)
    latent_dir, ask_dir = torch.randn(rank, generator=gen), torch.randn(q_rank, generator=gen)
    w["l0.mix.dkv"][:, 1] = torch.cat([latent_dir, torch.zeros(rot_dim)])
    w["l0.mix.dq"][:, 0] = ask_dir
    c = latent_dir / latent_dir.pow(2).mean().sqrt() * w["l0.mix.dkv.norm"]
    cq = ask_dir / ask_dir.pow(2).mean().sqrt() * w["l0.mix.dq.norm"]
    key = w["l0.mix.uk"][:dim] @ c                                    # head 0's plain key of the planted token
    # W_uq cq = key * gain in head 0's plain part: a score of about 30 above the others
    w["l0.mix.uq"][:dim] = torch.outer(key, cq) * (30.0 / (0.2 * float(key @ key) * float(cq @ cq)))
    w["l0.mix.sink"] = torch.tensor([0.5, -0.5])
    w["l0.mix.g"][:, :2] = 0.0
    w["l0.mix.g"] *= 0.2
    w["l0.mix.o"] *= 5.0          # what the layer fetches weighs as much in the sum as the stream does
    w["l0.norm1"] = torch.ones(width)
    return _write(folder, config, w)


def planted_attention_model(folder: Path) -> Path:
    """Two layers of grouped attention, the second reading the first one's keys: in both, head 0 of the asking token asks for
    the planted token's key of key head 0. The query and the key live in the dimensions that do not turn (8 of 16 do), so the
    score is the same at every distance: after the heads' norms it is scale * 16 * cos(angle between them) = 32 at its best."""
    from research_2_b200 import models  # noqa: F401
    from research_2_b200.config.registry import architecture_of

    heads, kv_heads, dim, vdim, width = 4, 2, 16, 24, 32
    rot = (8, 10000.0, (2.0, 64, 4.0, 1.0))
    config = model(64, width, [layer(attention(heads, kv_heads, dim, vdim, 2.0, rot=rot)),
                               layer(attention(2, kv_heads, dim, vdim, 2.0, rot=rot, kv_from=0))], eps=1e-5, alpha=0.3)
    arch = architecture_of(config)
    w = arch.random_weights(arch.parse_config(config), 19, std=0.08)
    gen = torch.Generator().manual_seed(20)
    _planted_embedding(w)
    direction = torch.cat([torch.zeros(8), torch.randn(8, generator=gen)])
    w["l0.mix.k"][:, 1] = 0.0
    w["l0.mix.k"][:dim, 1] = direction
    for name in ("l0.mix.q", "l1.mix.q"):
        w[name][:, 0] = 0.0
        w[name][:dim, 0] = direction
    for name in ("l0.mix.q.norm", "l0.mix.k.norm", "l1.mix.q.norm", "l0.norm1", "l1.norm1"):
        w[name] = torch.ones_like(w[name])
    for name in ("l0.mix.o", "l1.mix.o"):
        w[name] *= 10.0           # what a layer fetches weighs as much in the sum as the stream does
    w["l0.mix.o"][0] = 0.0        # ... but coordinate 0 stays the asking token's mark for the second layer
    return _write(folder, config, w)


def planted_sequence(n: int, ask_at: int, distance: int, seed: int = 0) -> list[int]:
    ids = [3 + t for t in random_tokens(seed, n, 61)]
    ids[ask_at] = QUERY_TOKEN
    if 0 <= ask_at - distance < ask_at:
        ids[ask_at - distance] = KEY_TOKEN
    return ids


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["prompt", "decoded", "portion_between"])
@pytest.mark.parametrize("kind", ["latent", "attention"])
def test_one_key_that_stands_out(tmp_path, dtype, how, kind):
    """The key 600 places back among hundreds, at the sequence's first token, and just before, at and after pages' borders
    (pages of 16: keys in rows 111, 112, 127, 128), with the asking row in a prompt, decoded alone, or first in a portion that
    begins between the key and the row. Every earlier key is visible, so the logits with the key differ from those without."""
    cases = [(650, 600), (229, 229), (229, 1), (130, 2), (130, 3), (130, 18), (130, 19), (143, 15), (144, 16), (144, 17), (77, 77), (300, 172)]
    page = 16
    folder = (planted_latent_model if kind == "latent" else planted_attention_model)(tmp_path / kind)
    for ask_at, distance in cases:
        ids = planted_sequence(ask_at + 6, ask_at, distance, seed=ask_at)
        truth = plain_logits(folder, ids)[ask_at]
        without = plain_logits(folder, planted_sequence(ask_at + 6, ask_at, 0, seed=ask_at))[ask_at]
        gap = float(np.abs(truth - without).max())
        assert gap > 0.3 * float(np.abs(truth).max()), (kind, ask_at, distance, gap)
        tb = traces.TraceBuilder()
        n = len(ids)
        if how == "prompt":
            tb.step([("x", ids, list(range(n)))], end=["x"])
        elif how == "decoded":
            first = max(1, ask_at - 3)
            tb.step([("x", ids[:first], list(range(first)))])
            for t in range(first, n):
                tb.step([("x", ids[t: t + 1], [0])], end=["x"] if t == n - 1 else [])
        else:
            cut_at = max(1, ask_at - max(1, distance // 2))
            tb.step([("x", ids[:cut_at], list(range(cut_at)))])
            tb.step([("x", ids[cut_at: ask_at + 2], list(range(ask_at + 2 - cut_at)))])
            tb.step([("x", ids[ask_at + 2:], list(range(n - ask_at - 2)))], end=["x"])
        outputs, _, _ = run_trace(folder, tb, dtype, page)
        per = compare(folder, {"x": ids}, tb, outputs, dtype, f"{kind} {how} row {ask_at} distance {distance}")
        got = per["x"][ask_at]
        assert float(np.abs(got - truth).max()) < 0.25 * gap, f"{kind} {how} row {ask_at} distance {distance}: the key was not seen"


# ---------------------------------------------------------------------------------------------
# whole models in every cutting


def cut(requests, mode: str) -> traces.TraceBuilder:
    if mode == "whole":
        return traces.whole(requests)
    if mode == "decode":
        return traces.prefill_then_decode(requests, 48)
    if mode == "portions":
        return traces.portions(requests)
    if mode == "tiny_portions":
        return traces.portions(requests, sizes=(2, 3, 2, 5, 2, 2, 9))
    return traces.mixed(requests, max_live=4)


def run_trace(folder, tb, dtype, page_size, max_tokens=None, max_seq_len=0):
    """Replays the trace in a pool of the trace's own peak demand plus one page (or `max_tokens`), the cache filled with
    loud values first. -> ({step: logits}, how many pages had two owners or more, the replay)."""
    from research_2_b200.engine.replay import Replay

    live, round_to = traces.max_live(tb), 64
    if max_tokens is None:
        max_tokens, round_to = (traces.peak_pages(tb, page_size) + 1) * page_size, page_size
    replay = Replay(str(folder), dtype, max_tokens, block_size=page_size, max_live=max(live, 1), round_to=round_to, max_seq_len=max_seq_len)
    replay.step_fn.arena.fill_(64.0)
    owners: dict[tuple[int, int], set] = {}
    out = {}
    for record in tb.steps:
        logits = replay.step(record)
        if logits is not None:
            out[record["step"]] = logits
        for rid, per_group in replay.pages_of_last_step.items():
            for g, pages in enumerate(per_group):
                for page in pages:
                    owners.setdefault((g, page), set()).add(rid)
    assert replay.cache.check() == ""
    for g in range(len(replay.cache.groups)):
        assert replay.cache.n_free(g) == replay.cache.groups[g].num_pages, "pages were lost"
    return out, sum(len(v) >= 2 for v in owners.values()), replay


def compare(folder, requests, tb, outputs, dtype, what):
    assert sorted(outputs) == sorted(tb.rows)
    per_request: dict[str, dict[int, np.ndarray]] = {}
    for step, rows in tb.rows.items():
        for (rid, pos), logits in zip(rows, outputs[step]):
            assert pos not in per_request.setdefault(rid, {}), f"{what}: position {pos} of {rid} written twice"
            per_request[rid][pos] = logits
    for rid, ids in requests.items():
        assert sorted(per_request[rid]) == list(range(len(ids))), f"{what}: request {rid} misses positions"
        got = np.stack([per_request[rid][p] for p in range(len(ids))])
        assert_close_to_plain(got, folder, ids, dtype, what=f"{what} request {rid}")
    return per_request


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
@pytest.mark.parametrize("mode", ["whole", "decode", "portions", "tiny_portions", "mixed"])
def test_cuttings(folders, name, dtype, mode):
    folder, requests = folders[name], requests_for(name)
    if mode == "tiny_portions":
        requests = dict(list(requests.items())[:3])
    tb = cut(requests, mode)
    outputs, reused, replay = run_trace(folder, tb, dtype, CASES[name]["page_size"])
    compare(folder, requests, tb, outputs, dtype, f"{name}/{dtype}/{mode}")
    if mode == "mixed":
        assert traces.max_live(tb) == 4 and len(requests) > 4, "request slots are used again"
        assert reused >= 2, f"only {reused} pages passed from one request to another"
        assert len(replay.cache.groups) == 1, "no layer has a window: one cache group"


def test_the_stream_after_every_layer(folders):
    """The stream after each layer (not only the logits), in float32: a layer that is wrong and then drowned by the next
    norm shows here."""
    from research_2_b200.engine.replay import Replay

    for name in ("a", "c", "d"):
        folder = folders[name]
        ids = random_tokens(9, 50, CASES[name]["config"]["vocab"])
        cfg, w = plain.read_model(folder)
        want: list = []
        plain.forward(cfg, w, ids, layers_out=want)
        replay = Replay(str(folder), "float32", 64, block_size=CASES[name]["page_size"], max_live=1)
        got = []
        blocks = replay.model.blocks
        originals = [b.forward for b in blocks]
        for b, original in zip(blocks, originals):
            def tapped(*args, _original=original, **kwargs):
                x = _original(*args, **kwargs)
                got.append(x.detach().double().cpu().clone())
                return x
            b.forward = tapped
        replay.step({"step": 0, "entries": [{"id": "x", "tokens": ids, "want": [len(ids) - 1]}], "end": ["x"]})
        assert len(got) == len(want)
        for i, (a, b) in enumerate(zip(got, want)):
            assert float((a[: len(ids)] - b).abs().max()) <= 3e-5 * float(b.abs().max()), (name, i)


def test_rows_wider_than_the_tensor_core_kernel_takes(tmp_path):
    """A latent of 300 numbers and heads of 272: cache rows of 308 numbers go to the general kernel in both dtypes."""
    case = {"config": model(61, 48, [layer(latent(2, 272, 8, 40, 300, 0.05, q_rank=20, rot=(8, 1000.0)), None)], alpha=1.5), "seed": 4, "std": 0.06}
    folder = make_model_dir(tmp_path / "wide", case)
    ids = random_tokens(2, 70, 61)
    for dtype in ("float32", "bfloat16"):
        tb = traces.prefill_then_decode({"x": ids}, n_decode=6)
        outputs, _, _ = run_trace(folder, tb, dtype, 16)
        compare(folder, {"x": ids}, tb, outputs, dtype, f"wide rows {dtype}")


def test_a_decode_step_whose_keys_are_cut_over_several_ctas(folders):
    """Single decoded tokens of long sequences: the latent kernel cuts a token's key tiles over CTAs and a second launch
    merges them (with the sinks); the logits equal those of one CTA a token within rounding, and the plain ones."""
    from research_2_b200.kernels import ops

    folder, name = folders["d"], "d"
    ids = random_tokens(11, 700, CASES[name]["config"]["vocab"])
    tb = traces.prefill_then_decode({"x": ids}, n_decode=5)
    results = {}
    for on in (True, False):
        old = ops.use_latent_slices(on)
        try:
            results[on] = compare(folder, {"x": ids}, tb, run_trace(folder, tb, "bfloat16", CASES[name]["page_size"])[0], "bfloat16", f"slices {on}")
        finally:
            ops.use_latent_slices(old)
    for pos in range(len(ids) - 5, len(ids)):
        a, b = results[True]["x"][pos], results[False]["x"][pos]
        assert float(np.abs(a - b).max()) <= 2e-2 * float(np.abs(b).max()), pos


def test_which_kernels_serve_bfloat16(folders):
    """Case d has the shapes that the fast kernels are written for: its latent layer runs on the latent kernel in prompts and
    decode steps, its grouped attention on the tensor-core prefill kernel and the fused decode kernel (which writes the new
    key itself; for the layer that reads another's keys it writes nothing)."""
    from research_2_b200.kernels import ops

    folder, name = folders["d"], "d"
    ids = random_tokens(3, 150, CASES[name]["config"]["vocab"])
    tb = traces.prefill_then_decode({"x": ids}, n_decode=4)
    before = dict(ops.kernel_uses())
    outputs, _, _ = run_trace(folder, tb, "bfloat16", CASES[name]["page_size"])
    compare(folder, {"x": ids}, tb, outputs, "bfloat16", "kernels of case d")
    used = {k: v - before.get(k, 0) for k, v in ops.kernel_uses().items()}
    assert used.get("latent_attention", 0) == 5 and used.get("attention_decode_fused", 0) == 8 and used.get("attention_prefill", 0) == 2, used
    assert used.get("attention_simt", 0) == 0, used


@pytest.mark.parametrize("seed", range(100, 112))
def test_configurations_drawn_at_random(seed, tmp_path):
    """Layers in any order and sizes of any kind: float32 within its floor in three cuttings, bfloat16 within its own
    (a router's close calls excused)."""
    case = random_case(seed)
    folder = make_model_dir(tmp_path / "model", case)
    ids = random_tokens(seed, case["length"], case["config"]["vocab"])
    requests = {"x": ids, "y": ids[: max(3, len(ids) // 3)], "z": ids[5:]}
    for dtype, modes in (("float32", ("whole", "portions", "mixed")), ("bfloat16", ("mixed",))):
        for mode in modes:
            tb = cut(requests, mode) if mode != "mixed" else traces.mixed(requests, max_live=2)
            outputs, _, _ = run_trace(folder, tb, dtype, case["page_size"])
            compare(folder, requests, tb, outputs, dtype, f"seed {seed} {dtype} {mode}")


def test_float32_logits_do_not_depend_on_the_cutting_at_all(folders):
    for name in ("a", "b", "c"):
        folder, requests = folders[name], requests_for(name)
        results = {}
        for mode in ("whole", "decode", "portions", "mixed"):
            tb = cut(requests, mode)
            results[mode] = compare(folder, requests, tb, run_trace(folder, tb, "float32", CASES[name]["page_size"])[0], "float32", f"{name}/{mode}")
        for mode in ("decode", "portions", "mixed"):
            for rid, rows in results["whole"].items():
                for pos, logits in rows.items():
                    assert np.array_equal(logits, results[mode][rid][pos]), f"{name}: {mode} differs from whole at {rid}[{pos}]"


def test_long_decoding(folders):
    """400 tokens, 390 of them decoded one by one through 26 pages: every decoded token reads all that came before it."""
    for name in ("a", "d"):
        folder, page = folders[name], CASES[name]["page_size"]
        ids = random_tokens(21, 400, CASES[name]["config"]["vocab"])
        tb = traces.prefill_then_decode({"x": ids}, n_decode=390)
        for dtype in ("float32", "bfloat16"):
            outputs, _, _ = run_trace(folder, tb, dtype, page, max_tokens=448)
            compare(folder, {"x": ids}, tb, outputs, dtype, f"long decoding {name} {dtype}")


def test_first_tokens(folders):
    for name in ("a", "b", "c", "d"):
        folder = folders[name]
        ids = random_tokens(7, 5, CASES[name]["config"]["vocab"])
        tb = traces.TraceBuilder()
        tb.step([("x", ids[:1], [0])])
        tb.step([("x", ids[1:2], [0])])
        tb.step([("x", ids[2:4], [0, 1])])
        tb.step([("x", ids[4:5], [0])], end=["x"])
        for dtype in ("float32", "bfloat16"):
            compare(folder, {"x": ids}, tb, run_trace(folder, tb, dtype, CASES[name]["page_size"], max_tokens=64)[0], dtype, f"first tokens {name} {dtype}")


def test_trace_run_program(folders, tmp_path):
    folder, name = folders["a"], "a"
    requests = {k: v for k, v in list(requests_for(name).items())[:3]}
    tb = traces.mixed(requests, max_live=3)
    out = tmp_path / "out"
    text = "".join(json.dumps(s) + "\n" for s in tb.steps)
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "bfloat16",
         "--out", str(out), "--max-tokens", str(sum(-(-len(v) // 64) * 64 for v in requests.values()))],
        input=text, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done ")] == [f"done {i}" for i in range(len(tb.steps))]
    vocab = CASES[name]["config"]["vocab"]
    outputs = {int(p.stem): np.fromfile(p, dtype="<f4").reshape(-1, vocab) for p in out.glob("*.f32")}
    compare(folder, requests, tb, outputs, "bfloat16", "trace_run program")


# ---------------------------------------------------------------------------------------------
# generation through the entry point and the scheduler


def test_greedy_generation_through_the_engine(folders):
    """Prompts of unequal length through `generate` (scheduler, portions under a small token budget, CUDA graphs): float32
    tokens equal the plain implementation's; bfloat16 tokens are (nearly) the best by the plain logits of the sequence so
    far."""
    import research_2_b200

    for name in ("a", "d"):
        folder, vocab = folders[name], CASES[name]["config"]["vocab"]
        prompts = [random_tokens(40 + i, n, vocab) for i, n in enumerate((5, 61, 18, 33))]
        cfg, w = plain.read_model(folder)
        want = [plain.generate(cfg, w, p, 10) for p in prompts]
        got = research_2_b200.generate(folder, prompts, max_new_tokens=10, dtype="float32", device=DEV, block_size=8,
                                       max_batch_tokens=32, max_requests=3, max_seq_len=128)
        assert got == want, (name, got, want)
        got16 = research_2_b200.generate(folder, prompts, max_new_tokens=10, dtype="bfloat16", device=DEV, block_size=16,
                                         max_batch_tokens=48, max_requests=4, max_seq_len=128)
        for prompt, tokens in zip(prompts, got16):
            assert len(tokens) == 10
            logits = plain_logits(folder, (prompt + tokens)[:-1])
            slack = 2 * 3e-2 * float(np.abs(logits).max())
            near_best = [float(logits[len(prompt) - 1 + i][tok]) >= float(logits[len(prompt) - 1 + i].max()) - slack
                         for i, tok in enumerate(tokens)]
            assert all(0 <= tok < vocab for tok in tokens) and sum(near_best) >= 8, (name, tokens, near_best)


def test_generation_in_a_pool_that_forces_preemption(folders):
    """A preempted request is computed again from its first token, in pages that others held meanwhile."""
    import research_2_b200

    name = "c"
    folder, vocab = folders[name], CASES[name]["config"]["vocab"]
    prompts = [random_tokens(60 + i, n, vocab) for i, n in enumerate((30, 44, 25))]
    cfg, w = plain.read_model(folder)
    want = [plain.generate(cfg, w, p, 10) for p in prompts]
    got = research_2_b200.generate(folder, prompts, max_new_tokens=10, dtype="float32", device=DEV, block_size=4,
                                   max_batch_tokens=16, max_requests=3, max_seq_len=64, num_slabs=30)
    assert got == want, (got, want)


def test_command_line(folders):
    folder = folders["b"]
    proc = subprocess.run([sys.executable, "-m", "research_2_b200", "generate", "--model", str(folder), "--prompt-tokens", "5,17,3",
                           "--max-new-tokens", "4", "--dtype", "float32", "--max-seq-len", "64"],
                          capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    tokens = json.loads(proc.stdout.strip().splitlines()[-1])["tokens"]
    cfg, w = plain.read_model(folder)
    assert tokens == plain.generate(cfg, w, [5, 17, 3], 4)
