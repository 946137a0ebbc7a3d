"""Zudalorn on the GPU against the plain implementation (tests/plain/zudalorn_plain.py): each mechanism alone, one
key that stands out at every edge of a window, then whole models through the step function, the cache manager and the
state slots in every cutting, then generation through the engine."""

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
from tests.plain import zudalorn_plain as plain
from tests.zudalorn_cases import CASES, assert_close_to_plain, layer, latent, make_model_dir, model, plain_logits, random_case, random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
F64 = torch.float64

LENGTHS = {"a": (70, 45, 128, 33, 2, 97), "b": (60, 9, 41, 3, 77), "c": (150, 66, 5, 90, 17, 2), "d": (90, 66, 5, 131, 40)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: make_model_dir(tmp_path_factory.mktemp(f"zx_{name}"), case) for name, case in CASES.items()}


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
def test_router_with_sigmoid_scores_and_groups(dtype):
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(1)
    shapes = [  # rows, width, experts, top, groups, kept groups, further gates
        (37, 40, 6, 2, 3, 1, 0), (9, 64, 8, 3, 4, 2, 1), (130, 96, 3, 3, 1, 1, 0), (4, 200, 33, 4, 11, 3, 1), (50, 24, 12, 4, 2, 1, 1),
        (21, 32, 5, 2, 5, 3, 0), (64, 48, 16, 8, 4, 4, 0), (17, 16, 2, 1, 2, 1, 1),
    ]
    for rows, width, experts, top, groups, keep, extra in shapes:
        h = torch.randn(rows, width, generator=gen).to(dtype)
        w = (torch.randn(experts + extra, width, generator=gen) * 0.4).to(torch.bfloat16).float()
        correction = torch.randn(experts, generator=gen) * (0.3 if rows % 2 else 3.0)   # large ones: choice scores below zero
        z = h.double() @ w.double().T
        plain.MARGINS = []
        try:
            want_chosen, want_weights = plain.route(z[:, :experts], correction, top, groups, keep)
            clear = plain.MARGINS[0] > 1e-4
        finally:
            plain.MARGINS = None
        dense, chosen, weight, gates = ops.route_scored(h.to(DEV), w.to(DEV), correction.to(DEV), top, groups, keep, n_extra=extra)
        assert int(clear.sum()) > rows // 2
        for t in range(rows):
            if not bool(clear[t]):
                continue
            got = dict(zip(chosen[t].cpu().tolist(), weight[t].cpu().tolist()))
            assert sorted(got) == sorted(want_chosen[t]), (rows, t, got, want_chosen[t])
            for e, wt in zip(want_chosen[t], want_weights[t].tolist()):
                assert abs(got[e] - wt) < 1e-5 and abs(float(dense[t, e]) - wt) < 1e-5
            assert int((dense[t] != 0).sum()) == top
        if extra:
            assert float((gates.double().cpu() - z[:, experts:]).abs().max()) < 1e-4
        else:
            assert gates is None
    # equal scores: the lower index wins, among groups (0 and 1 tie behind 2; 0 is kept) and among experts (1, 4 and 5 tie)
    h = torch.zeros(3, 16, dtype=dtype)
    _, chosen, weight, _ = ops.route_scored(h.to(DEV), torch.zeros(6, 16, device=DEV), torch.tensor([0., 1., 1., 0., 1., 1.], device=DEV), 2, 3, 2)
    assert [sorted(r) for r in chosen.cpu().tolist()] == [[1, 4]] * 3 and torch.allclose(weight.cpu(), torch.full((3, 2), 0.5))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations_and_norms_around_a_sublayer(dtype):
    from research_2_b200.kernels import ops

    gen = torch.Generator().manual_seed(2)
    for width in (52, 24, 2056, 3):   # rows of pairs, of 16-byte pieces (in one and in two blocks), of single numbers
        z = (torch.randn(23, width, generator=gen) * 3).to(dtype)
        z[0, :3] = torch.tensor([-0.0, 1e-3, -1e-3]).to(dtype)
        for p, q in ((0.3, -0.2), (-4.0, 2.5)):
            a_pos, a_neg = math.log1p(math.exp(p)), 0.5 + math.log1p(math.exp(q))
            close(ops.xielu(z.to(DEV), a_pos, a_neg), plain.xielu(z.double(), p, q), dtype, f"xielu {width}")
    # gated silu units of several experts with routing weights, and a tail (the expert that every row uses) with a gate per row
    rows, experts, width, tail = 21, 3, 10, 7
    inner = experts * width + tail
    gu = (torch.randn(rows, 2 * inner, generator=gen) * 2).to(dtype)
    g, u = gu[:, :inner].double(), gu[:, inner:].double()
    route = torch.rand(rows, experts, generator=gen)
    route[:, 1] = 0.0
    gate = torch.randn(rows, 1, generator=gen) * 2
    weights = torch.cat([route.double().repeat_interleave(width, dim=1), torch.sigmoid(gate.double()).expand(rows, tail)], dim=1)
    got = ops.expert_act(gu.to(DEV), "silu", route=route.to(DEV), n_experts=experts, expert_width=width, tail_gate=gate.to(DEV))
    close(got, g * torch.sigmoid(g) * u * weights, dtype, "experts")
    assert float(got[:, width: 2 * width].abs().max()) == 0.0
    weights[:, experts * width:] = 1.0
    close(ops.expert_act(gu.to(DEV), "silu", route=route.to(DEV), n_experts=experts, expert_width=width),
          g * torch.sigmoid(g) * u * weights, dtype, "experts, a tail without a gate")
    # a sublayer's output, normalised with one gain, joins the stream; the same launch norms the new stream
    eps = 1e-3
    for width in (50, 64, 320, 1000):
        x, y = torch.randn(rows, width, generator=gen), torch.randn(rows, width, generator=gen) * 40
        y[3] = 0.0     # a row of zeros stays zero: eps stands inside the root
        g1, g2 = torch.full((width,), 0.37), torch.full((width,), -1.4)
        want = x.double() + plain.scalar_norm(y.double(), 0.37, eps)
        assert float((ops.norm_add(x.to(DEV), y.to(DEV), g1.to(DEV), eps).double().cpu() - want).abs().max()) < 1e-5
        new, nxt = ops.norm_add(x.to(DEV), y.to(DEV), g1.to(DEV), eps, g2.to(DEV), 1e-5, dtype)
        assert float((new.double().cpu() - want).abs().max()) < 1e-5 and nxt.dtype == dtype
        close(nxt, plain.scalar_norm(want, -1.4, 1e-5), dtype, "the next sublayer's input")
    # every head by its own root mean square, no gain, times silu of a gate
    heads, size = 3, 20
    o = torch.randn(rows, heads * size, generator=gen) * torch.tensor([0.01, 1.0, 300.0]).repeat_interleave(size)
    gate = torch.randn(rows, heads * size, generator=gen).to(dtype)
    zz = gate.double()
    want = plain.unit_rms(o.double().view(rows, heads, size), eps).reshape(rows, -1) * zz * torch.sigmoid(zz)
    close(ops.group_norm_gated(o.to(DEV), gate.to(DEV), None, heads, eps, "silu_after", dtype), want, dtype, "heads' norm")


def _entries(cuts, slots, fresh):
    starts = [0]
    for n in cuts:
        starts.append(starts[-1] + n)
    return i32(starts), i32(slots), i32(fresh)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 16, 16, 16), (1, 64, 128, 64), (3, 24, 40, 10), (4, 8, 24, 0), (1, 200, 8, 2), (5, 32, 32, 32)])
def test_retention_recurrence_in_portions_and_slots(dtype, shape):
    """Two sequences side by side through state slots, cut into portions down to one row, in slots that held other
    sequences before; against the recurrence run whole. Decays of 0 and 1 among them."""
    from research_2_b200.kernels import ops

    heads, dim, vdim, rot_dims = shape
    gen = torch.Generator().manual_seed(4)
    n_slots = 3
    state = torch.full((n_slots, heads * dim * vdim), 123.0, device=DEV)   # what an earlier request left
    decay = torch.tensor(([0.0, 1.0, 0.93, 0.999, 0.5] * 2)[:heads], dtype=F64)
    freqs = [777.0 ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)]
    inv_freq = torch.tensor(freqs, dtype=F64).float().to(DEV) if rot_dims else None
    seqs = {}
    for name, n in (("x", 45), ("y", 23)):
        q, k = (torch.randn(n, heads * dim, generator=gen).to(dtype) for _ in range(2))
        v = torch.randn(n, heads * vdim, generator=gen).to(dtype)
        pos = list(range(n))
        want = plain.retention_cells(plain.rotate(q.double().view(n, heads, dim), pos, freqs, "half"),
                                     plain.rotate(k.double().view(n, heads, dim), pos, freqs, "half") * dim ** -0.5,
                                     v.double().view(n, heads, vdim), decay).reshape(n, -1)
        seqs[name] = (q, k, v, want)
    plan = [[("x", 17), ("y", 1)], [("y", 2), ("x", 1)], [("x", 1)], [("y", 20), ("x", 26)]]
    slot, fed, got = {"x": 2, "y": 0}, {"x": 0, "y": 0}, {"x": [], "y": []}
    for step in plan:
        parts = [[seqs[name][i][fed[name]: fed[name] + n] for name, n in step] for i in range(3)]
        q, k, v = (torch.cat(p).to(DEV) for p in parts)
        positions = i32([p for name, n in step for p in range(fed[name], fed[name] + n)])
        q_start, slots, fresh = _entries([n for _, n in step], [slot[name] for name, _ in step], [int(fed[name] == 0) for name, _ in step])
        out = ops.retention_scan(q, k, v, decay.float().to(DEV), dim ** -0.5, inv_freq, rot_dims, positions, state, q_start, slots, fresh,
                                 heads, dim, vdim).cpu()
        at = 0
        for name, n in step:
            got[name].append(out[at: at + n])
            at += n
            fed[name] += n
    for name in seqs:
        close(torch.cat(got[name]), seqs[name][3], dtype, f"{shape} {name}")
    assert float(state[1].min()) == 123.0, "a slot of no entry was written"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 16, 8, 8, 32, 24), (1, 20, 4, 2, 44, 12), (3, 12, 6, 6, 10, 20), (6, 64, 32, 32, 96, 80), (2, 8, 16, 16, 8, 8),
                                   (5, 4, 2, 0, 6, 4)])
def test_latent_rows_and_the_products_per_head(dtype, shape):
    """The launch between the input product and the attention kernel: the latent's norm, both rotations (pairs of
    neighbours, stretched magnitude), the cache row, the copy of the rotated query parts; then the small products per head."""
    from research_2_b200.kernels import ops

    heads, dim, rot_dim, rot_dims, rank, vdim = shape
    gen = torch.Generator().manual_seed(6)
    rows, page, eps, magnitude = 83, 4, 1e-4, 1.17
    q_head, row = dim + rot_dim, rank + rot_dim
    proj = torch.randn(rows, heads * q_head + row + 5, generator=gen).to(dtype)
    positions = torch.randint(0, 3000, (rows,), generator=gen).tolist()
    freqs = [300.0 ** (-2.0 * i / max(rot_dims, 1)) for i in range(rot_dims // 2)]
    norm_w = torch.randn(rank, generator=gen)
    q = proj[:, : heads * q_head].double().view(rows, heads, q_head)
    want_q_rot = plain.rotate(q[..., dim:], positions, freqs, "interleaved", magnitude)
    down = proj[:, heads * q_head: heads * q_head + row].double()
    want_c = plain.unit_rms(down[:, :rank], eps) * norm_w.double()
    want_k_rot = plain.rotate(down[:, rank:], positions, freqs, "interleaved", magnitude)
    n_pages = 24
    cache = torch.full((n_pages * page * row,), 7.0, dtype=dtype, device=DEV)
    slots = torch.randperm((n_pages - 1) * page, generator=gen)[:rows] + page
    queries = torch.zeros(rows, heads * row, dtype=dtype, device=DEV)
    dev = proj.to(DEV)
    ops.latent_prepare(dev, heads, q_head, dim, rot_dim, rot_dims, heads * q_head, rank, norm_w.to(DEV), eps,
                       torch.tensor(freqs, dtype=F64).float().to(DEV), magnitude, i32(positions), k_cache=cache, slot_mapping=slots.to(torch.int32).to(DEV),
                       page_size=page, page_stride=page * row, n_pages=n_pages, q_out=queries, q_out_head_dim=row, q_out_off=rank)
    # the angle is a float32 product of a position in the thousands: its rounding is 1e-4 of a turn
    angle_tol = 2e-3 if dtype == torch.float32 else 4e-2
    got = dev.double().cpu()
    assert float((got[:, : heads * q_head].view(rows, heads, q_head)[..., dim:] - want_q_rot).abs().max()) <= angle_tol
    assert torch.equal(got[:, : heads * q_head].view(rows, heads, q_head)[..., :dim], q[..., :dim]), "the plain query parts changed"
    close(dev[:, heads * q_head: heads * q_head + rank], want_c, dtype, "latent")
    assert float((got[:, heads * q_head + rank: heads * q_head + row] - want_k_rot).abs().max()) <= angle_tol
    assert torch.equal(got[:, heads * q_head + row:], proj[:, heads * q_head + row:].double()), "columns after the row changed"
    stored = cache.view(n_pages * page, row)[slots.to(DEV)]
    assert torch.equal(stored, dev[:, heads * q_head: heads * q_head + row]), "the cache row is the prepared row"
    assert float(cache.view(n_pages * page, row)[:page].min()) == 7.0, "the null page was written"
    assert torch.equal(queries.view(rows, heads, row)[..., rank:], dev[:, : heads * q_head].view(rows, heads, q_head)[..., dim:])
    # q_lat = W_uk[h]^T q_plain (matrices stored [out, in] one head after the other), then out = W_uv[h] mixed
    w_uk = (torch.randn(heads * dim, rank, generator=gen) * 0.3).to(dtype)
    ops.head_linear(dev, q_head, w_uk.to(DEV), False, queries, row, heads, dim, rank)
    want = torch.einsum("thd,hdc->thc", q[..., :dim], w_uk.double().view(heads, dim, rank))
    close(queries.view(rows, heads, row)[..., :rank], want, dtype, "queries in the latent's coordinates")
    mixed = torch.randn(rows, heads * rank, generator=gen).to(dtype)
    w_uv = (torch.randn(heads * vdim, rank, generator=gen) * 0.3).to(dtype)
    out = torch.zeros(rows, heads * vdim, dtype=dtype, device=DEV)
    ops.head_linear(mixed.to(DEV), rank, w_uv.to(DEV), True, out, vdim, heads, rank, vdim)
    close(out, torch.einsum("thc,hvc->thv", mixed.double().view(rows, heads, rank), w_uv.double().view(heads, vdim, rank)).reshape(rows, -1), dtype, "values")


def plain_attention_over_latents(q, rows_of, positions, kv_rank, scale, window):
    """q [T, H, row] float64, rows_of[t]: the cache rows [len, row] of the token's sequence, positions[t]: the token's place.
    Head h of token t: softmax over the keys (p - window, p] of scale * q . row, times the rows' first kv_rank numbers."""
    out = torch.zeros(q.shape[0], q.shape[1], kv_rank, dtype=F64)
    for t in range(q.shape[0]):
        p = positions[t]
        first = max(0, p - window + 1) if window else 0
        keys = rows_of[t][first: p + 1]
        weights = torch.softmax((q[t] @ keys.T) * scale, dim=-1)
        out[t] = weights @ keys[:, :kv_rank]
    return out


# heads, cache row, latent's part of it, window, page size
LATENT_SHAPES = [(12, 160, 128, 64, 16), (3, 40, 24, 0, 8), (5, 33, 20, 7, 3), (70, 48, 48, 100, 32), (1, 256, 200, 1, 16), (16, 96, 64, 63, 64),
                 (64, 24, 16, 65, 4), (2, 136, 130, 129, 128)]


@pytest.mark.parametrize("cut", ["prompts", "decoded", "portions", "many"])
@pytest.mark.parametrize("shape", LATENT_SHAPES)
def test_attention_over_a_cache_of_latents(shape, cut):
    """The bfloat16 kernel whose tiles hold all heads of a few tokens, alone: entries of unequal lengths whose pages lie
    scattered in a pool full of large numbers, as whole prompts, as single decoded tokens and as portions that start in the
    middle, and as 42 entries of which every other one is a single token; windows that end inside, at and beyond a tile of 64
    keys; rows that are no multiple of 8 or 16 numbers."""
    from research_2_b200.kernels import ops

    heads, row, rank, window, page = shape
    gen = torch.Generator().manual_seed(heads * 1000 + row)
    lengths = [1, 2, 63, 64, 65, 130, 200] * (6 if cut == "many" else 1)
    scale = 1.0 / math.sqrt(row)
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
    want = plain_attention_over_latents(q.double().view(-1, heads, row), [per_seq[e].double() for e in row_entry], positions, rank, scale, window)
    before = ops.kernel_uses().get("latent_attention", 0)
    got = ops.paged_attention(
        q.to(DEV), cache.to(DEV), cache.to(DEV), page * row, page, n_pages, tables.to(DEV), i32(row_entry), i32(positions),
        i32([b for _, b in spans]), heads, 1, row, scale, window, decode_only=cut == "decoded", max_context=max(lengths),
        q_start=i32(q_start), n_tiles=sum(-(-r // 64) for r in entry_rows), v_head_dim=rank, values_in_keys=True)
    assert ops.kernel_uses().get("latent_attention", 0) == before + 1, "another kernel took the call"
    close(got.view(-1, heads, rank), want, torch.bfloat16, f"{shape} {cut}")


# ---------------------------------------------------------------------------------------------
# one key that stands out, at every edge


QUERY_TOKEN, KEY_TOKEN = 1, 2


def planted_model(folder: Path, window, page_note: str = "") -> Path:
    """One layer of latent attention whose weights are made so that the token QUERY_TOKEN asks, in head 0, for exactly the key
    that the token KEY_TOKEN leaves in the cache: coordinate 0 of the stream drives the query, coordinate 1 the latent, and
    the query's plain part is a multiple of W_uk applied to that latent. Such a key's weight in the softmax is nearly one
    wherever it is visible, so the logits at the asking position say whether it was seen."""
    from research_2_b200 import models  # noqa: F401  (registers the architectures)
    from research_2_b200.config.registry import architecture_of
    from research_2_b200.weights.safetensors_io import write_file

    heads, dim, rot_dim, vdim, rank, width = 2, 16, 8, 16, 24, 32
    config = model(64, width, [layer(latent(heads, dim, rot_dim, vdim, rank, 0.2, window=window, rot=(8, 10000.0, (2.0, 64, 4.0, 1.0))))], eps=1e-5)
    arch = architecture_of(config)
    cfg = arch.parse_config(config)
    w = arch.random_weights(cfg, 17, std=0.08)
    gen = torch.Generator().manual_seed(18)
    w["embed"][:, :2] = 0.0
    w["embed"][QUERY_TOKEN] *= 0.1
    w["embed"][KEY_TOKEN] *= 0.1
    w["embed"][QUERY_TOKEN, 0] = 6.0
    w["embed"][KEY_TOKEN, 1] = 6.0
    latent_dir = torch.randn(rank, generator=gen)
    w["l0.mix.dkv"][:, 1] = torch.cat([latent_dir, torch.zeros(rot_dim)])
    c = latent_dir / latent_dir.pow(2).mean().sqrt() * w["l0.mix.dkv.norm"]
    key = w["l0.mix.uk"][:dim] @ c                                    # head 0's plain key of the planted token
    w["l0.mix.q"][:, 0] = 0.0
    w["l0.mix.q"][:dim, 0] = key * (30.0 / (0.2 * float(key @ key) * width ** 0.5))   # a score of about 30 above the others
    w["l0.norm1"] = torch.tensor(1.0)
    w["l0.norm1b"] = torch.tensor(2.0)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(arch.config_to_json(cfg)))
    write_file(folder / "model.safetensors", {n: t.to(torch.bfloat16) for n, t in w.items()})
    return folder


def planted_sequence(n: int, ask_at: int, distance: int, seed: int = 0) -> list[int]:
    ids = [3 + t for t in random_tokens(seed, n, 61)]
    ids[ask_at] = QUERY_TOKEN
    if 0 <= ask_at - distance < ask_at:
        ids[ask_at - distance] = KEY_TOKEN
    return ids


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["prompt", "decoded", "portion_between"])
def test_one_key_that_stands_out_at_every_edge(tmp_path, dtype, how):
    """The key at the last place inside the window and one place further out, with the asking row in a prompt, decoded
    alone, or first in a portion that begins between the key and the row; at pages' borders (pages of 16: rows 127 and 128);
    a window of one token; and without a window a key 600 places back among hundreds."""
    cases = [(36, 229, 35), (36, 229, 36), (36, 229, 1), (36, 100, 35), (36, 100, 36), (16, 127, 15), (16, 127, 16), (16, 128, 15), (16, 128, 16),
             (16, 143, 15), (16, 144, 16), (1, 77, 1), (2, 77, 1), (2, 77, 2), (None, 650, 600), (None, 229, 229)]
    page = 16
    folders = {}
    for window, ask_at, distance in cases:
        if window not in folders:
            folders[window] = planted_model(tmp_path / f"w{window}", window)
        folder = folders[window]
        ids = planted_sequence(ask_at + 6, ask_at, distance, seed=ask_at)
        truth = plain_logits(folder, ids)[ask_at]
        # the plain statement itself tells the two sides of the edge apart: without the key the logits are others
        without = plain_logits(folder, planted_sequence(ask_at + 6, ask_at, 0, seed=ask_at))[ask_at]
        seen = window is None or distance < window
        gap = float(np.abs(truth - without).max())
        assert (gap > 0.3 * float(np.abs(truth).max())) == seen, (window, ask_at, distance, gap)
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
            cut = max(1, ask_at - max(1, distance // 2))
            tb.step([("x", ids[:cut], list(range(cut)))])
            tb.step([("x", ids[cut: ask_at + 2], list(range(ask_at + 2 - cut)))])
            tb.step([("x", ids[ask_at + 2:], list(range(n - ask_at - 2)))], end=["x"])
        outputs, _, _ = run_trace(folder, tb, dtype, page)
        compare(folder, {"x": ids}, tb, outputs, dtype, f"{how} window {window} row {ask_at} distance {distance}")


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
    """Replays the trace in a pool of the trace's own peak demand plus one page (or `max_tokens`), cache and state slots
    filled with loud values first. -> ({step: logits}, how many pages had two owners or more, the replay)."""
    from research_2_b200.engine.replay import Replay

    live, round_to = traces.max_live(tb), 64
    if max_tokens is None:
        max_tokens, round_to = (traces.peak_pages(tb, page_size) + 1) * page_size, page_size
    replay = Replay(str(folder), dtype, max_tokens, block_size=page_size, max_live=max(live, 1), round_to=round_to, max_seq_len=max_seq_len)
    replay.step_fn.arena.fill_(64.0)
    for t in replay.step_fn.state_tensors:
        t.fill_(-9.0)
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
        assert traces.max_live(tb) == 4 and len(requests) > 4, "state slots are used again"
        if replay.model.cache_members:
            assert reused >= 4, f"only {reused} pages passed from one request to another"


def test_every_layer_after_every_layer(folders):
    """The stream after each layer (not only the logits), in float32: a layer that is wrong and then drowned shows here."""
    from research_2_b200.engine.replay import Replay

    for name in ("a", "d"):
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


@pytest.mark.parametrize("seed", range(100, 110))
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


def test_long_decoding_through_a_small_pool(folders):
    """400 tokens, 390 of them decoded one by one: the windows pass over decoded tokens, the window groups give their
    pages back (8 pages a group hold it all), the states are carried 390 times."""
    name = "a"
    folder, page = folders[name], CASES[name]["page_size"]
    ids = random_tokens(21, 400, CASES[name]["config"]["vocab"])
    tb = traces.prefill_then_decode({"x": ids}, n_decode=390)
    for dtype in ("float32", "bfloat16"):
        outputs, _, replay = run_trace(folder, tb, dtype, page, max_tokens=8 * page, max_seq_len=512)
        compare(folder, {"x": ids}, tb, outputs, dtype, f"long decoding in a small pool {dtype}")
        assert sorted(g.window for g in replay.cache.groups) == [7, 24]


def test_first_tokens(folders):
    for name in ("a", "b", "c"):
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
    folder, name = folders["d"], "d"
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
    """Prompts of unequal length through `generate` (scheduler, portions under a small token budget, state slots, CUDA
    graphs): float32 tokens equal the plain implementation's; bfloat16 tokens are (nearly) the best by the plain
    logits of the sequence so far."""
    import research_2_b200

    for name in ("a", "c"):
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
    """A preempted request is computed again from its first token: its state slot starts from zero."""
    import research_2_b200

    name = "d"
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
