"""Small Zudalorn configurations for the tests, model folders with random weights, and the plain implementation's
logits with an error budget.

The configurations differ from one another in every size and constant, and between them cover the values that one
model may happen to make equal or trivial: layers in every order (retention only: a model without any per-token
cache; latent attention only), one head and several, a latent smaller and larger than a head, value heads smaller
and larger than key heads, sizes that are no multiple of 16 or 8, a rotation of a part of the rotated dimensions, a
plain and a stretched one and none, a window of one token, of a few, one longer than any sequence and none, decays
of 0, 1 and between, layers without a feed-forward, experts in one group, in groups of one, two and more, of which
one, some or all groups are kept, with and without the expert that every token uses.
"""

from __future__ import annotations

import functools
from pathlib import Path

import numpy as np
import torch

from tests.plain import zudalorn_plain


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, window=None, rot=None):
    """rot: (dims, base) or (dims, base, (factor, original, fast, slow))."""
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if len(rot) > 2:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot[2]))
    return m


def retention(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp=None):
    return {"type": "latent_attention" if "kv_rank" in mixer else "retention", "mixer": mixer, "mlp": mlp}


def model(vocab, width, layers, eps=1e-6):
    return {"architecture": "Zudalorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


CASES = {
    # every kind of layer and of feed-forward, a layer without one; a stretched rotation; groups of two experts
    "a": {"config": model(211, 64, [
        layer(retention(2, 16, 24, (0.9, 0.99), rot=(8, 1000.0)), moe(8, 3, 16, groups=(4, 2), shared=24)),
        layer(latent(4, 16, 8, 24, 32, 0.2, window=24, rot=(8, 10000.0, (4.0, 64, 8.0, 2.0))), dense(96)),
        layer(retention(4, 8, 8, (0.5, 0.75, 0.97, 1.0))),
        layer(latent(2, 8, 16, 8, 12, 0.3, window=7, rot=(16, 500.0)), moe(6, 2, 8, groups=(3, 1))),
    ], eps=1e-6), "seed": 3, "std": 0.08, "page_size": 16},
    # latent attention only; sizes that are no multiple of 8; a window of one token; every expert used; groups of one expert
    "b": {"config": model(97, 40, [
        layer(latent(3, 12, 6, 20, 10, 0.25, window=9, rot=(4, 77.0)), moe(5, 5, 24)),
        layer(latent(1, 20, 4, 12, 44, 0.5, window=1, rot=(4, 30.0, (8.0, 16, 4.0, 1.0))), dense(56)),
        layer(latent(5, 4, 2, 4, 6, 0.7), moe(4, 1, 8, groups=(4, 2), shared=8)),
    ], eps=2e-5), "seed": 5, "std": 0.1, "page_size": 8},
    # retention only (no per-token cache at all); a state of 64 x 128; a full rotation and none; a head that forgets everything
    "c": {"config": model(300, 128, [
        layer(retention(1, 64, 128, (0.995,), rot=(64, 100000.0)), dense(160)),
        layer(retention(8, 16, 8, (0.0, 0.3, 0.6, 0.9, 0.95, 0.98, 0.99, 0.999)), moe(12, 4, 24, groups=(3, 2), shared=16)),
    ], eps=1e-5), "seed": 8, "std": 0.05, "page_size": 32},
    # heads and latents of 64 and more, no window in one layer and one beyond every sequence in the other, pages of 4
    "d": {"config": model(128, 96, [
        layer(latent(2, 64, 32, 64, 96, 0.1, rot=(32, 10000.0, (2.0, 128, 16.0, 1.0)))),
        layer(retention(3, 24, 40, (0.9, 0.96, 0.99), rot=(12, 50.0)), dense(72)),
        layer(latent(4, 32, 64, 16, 64, 0.11, window=100000, rot=(64, 1000000.0)), moe(2, 1, 40, groups=(2, 1), shared=8)),
    ], eps=1e-5), "seed": 13, "std": 0.07, "page_size": 4},
}


def _divisors(n: int) -> list[int]:
    return [d for d in range(1, n + 1) if n % d == 0]


def random_case(seed: int) -> dict:
    """A configuration drawn from a seed: one to five layers of either kind in any order, sizes that are and are not
    multiples of 16, every optional mechanism there or not."""
    import random

    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(1, 5)):
        if rng.random() < 0.5:
            heads, dim = rng.randint(1, 6), rng.choice([4, 8, 12, 16, 24, 32, 48, 64, 96])
            rot = None
            if rng.random() < 0.8:
                rot = (rng.choice(list(range(2, dim + 1, 2))) if rng.random() < 0.4 else dim, rng.choice([100.0, 10000.0, 1000000.0]))
            mixer = retention(heads, dim, rng.choice([dim, 4, 8, 16, 20, 32, 48, 64, 128]),
                              [rng.choice([0.5, 0.9, 0.97, 0.99, 0.999, 1.0 - 2.0 ** -rng.randint(3, 11)]) for _ in range(heads)], rot=rot)
        else:
            rot_dim = rng.choice([2, 4, 8, 16, 32, 64])
            rot = None
            if rng.random() < 0.85:
                dims = rng.choice(list(range(2, rot_dim + 1, 2))) if rng.random() < 0.3 else rot_dim
                rot = (dims, rng.choice([100.0, 10000.0, 50000.0]))
                if rng.random() < 0.6:
                    rot += ((rng.choice([2.0, 4.0, 16.0]), rng.choice([32, 128, 1024]), rng.choice([8.0, 32.0]), rng.choice([1.0, 2.0])),)
            dim = rng.choice([4, 8, 16, 24, 32, 64, 96, 128])
            mixer = latent(rng.randint(1, 8), dim, rot_dim, rng.choice([dim, 8, 16, 40, 64, 80]), rng.choice([8, 16, 24, 32, 64, 96, 128, 160]),
                           rng.choice([(dim + rot_dim) ** -0.5, 0.1, 0.3]), window=rng.choice([None, 1, 3, 16, 17, 40, 64, 100, 136, 1000]), rot=rot)
        r = rng.random()
        if r < 0.15:
            mlp = None
        elif r < 0.45:
            mlp = dense(rng.choice([16, 40, 64, 96, 200]))
        else:
            experts = rng.randint(2, 16)
            groups = None
            size = experts
            if rng.random() < 0.7:
                count = rng.choice(_divisors(experts))
                groups, size = (count, rng.randint(1, count)), experts // count
            most = size * (groups[1] if groups else 1)
            mlp = moe(experts, rng.randint(1, min(most, 5)), rng.choice([8, 16, 24, 32, 64]), groups=groups,
                      shared=rng.choice([8, 16, 48]) if rng.random() < 0.6 else None)
        layers.append(layer(mixer, mlp))
    config = model(rng.choice([50, 97, 256, 1000]), rng.choice([24, 40, 64, 72, 100, 128, 192, 320]), layers, eps=rng.choice([1e-6, 1e-5]))
    return {"config": config, "seed": seed, "std": 0.06, "page_size": rng.choice([4, 8, 16, 32]), "length": rng.choice([40, 150, 300])}


def make_model_dir(folder: Path, case: dict, store_dtype: str = "bfloat16") -> Path:
    from research_2_b200 import models  # noqa: F401  (registers the architectures)
    from research_2_b200.config.registry import architecture_of
    from research_2_b200.weights import write_model_folder

    arch = architecture_of(case["config"])
    return write_model_folder(folder, arch, arch.parse_config(case["config"]), case["seed"], store_dtype, std=case["std"])


def random_tokens(seed: int, n: int, vocab: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()


@functools.lru_cache(maxsize=64)
def _plain_cached(folder: str, ids: tuple) -> np.ndarray:
    cfg, w = zudalorn_plain.read_model(folder)
    return zudalorn_plain.forward(cfg, w, list(ids)).numpy()


def plain_logits(folder, ids) -> np.ndarray:
    return _plain_cached(str(folder), tuple(int(i) for i in ids))


@functools.lru_cache(maxsize=64)
def _movement_cached(folder: str, ids: tuple) -> np.ndarray:
    """Per position, how far the plain logits move when every normalised row is disturbed by relative noise of 2^-9
    (about bfloat16's rounding, which the engine applies in more places), the most over eight draws. A position at
    which a router's choice (of a group or of an expert) hangs on a score gap below 0.004 is excused altogether (infinity)."""
    cfg, w = zudalorn_plain.read_model(folder)
    truth = _plain_cached(folder, ids)
    worst = np.zeros(len(ids))
    zudalorn_plain.MARGINS = []
    try:
        zudalorn_plain.forward(cfg, w, list(ids))
        for margin in zudalorn_plain.MARGINS:
            worst[margin.numpy() < 0.01] = np.inf
        worst = np.maximum.accumulate(worst)
    finally:
        zudalorn_plain.MARGINS = None
    for seed in range(8):
        gen = torch.Generator().manual_seed(1000 + seed)
        zudalorn_plain.DISTURB = lambda x: x * (1 + 2.0 ** -9 * torch.randn(x.shape, generator=gen, dtype=torch.float64))
        try:
            moved = zudalorn_plain.forward(cfg, w, list(ids)).numpy()
        finally:
            zudalorn_plain.DISTURB = None
        worst = np.maximum(worst, np.abs(moved - truth).max(axis=1))
    return worst


FLOORS = {"float32": 1e-4, "bfloat16": 3e-2}


def assert_close_to_plain(got: np.ndarray, folder, ids, dtype_name: str, positions=None, what: str = "") -> None:
    """|logit - truth| <= floor * max |truth| with truth in float64; floors 1e-4 (float32) and 3e-2 (bfloat16). In
    bfloat16 a position may also be off by three times what disturbances of the size of its rounding do to the plain logits
    there; positions from a router's first close call on are excused, and only those."""
    truth = plain_logits(folder, ids)
    allowed = np.full(len(truth), FLOORS[dtype_name] * float(np.abs(truth).max()))
    if dtype_name == "bfloat16":
        allowed = np.maximum(allowed, 3.0 * _movement_cached(str(folder), tuple(int(i) for i in ids)))
    if positions is not None:
        truth, allowed = truth[list(positions)], allowed[list(positions)]
    assert got.shape == truth.shape, (got.shape, truth.shape, what)
    err = np.abs(got.astype(np.float64) - truth).max(axis=1)
    if not bool((err <= allowed).all()):
        first_bad = int(np.argmax(~(err <= allowed)))
        pos = list(positions)[first_bad] if positions is not None else first_bad
        raise AssertionError(f"{what}: |logit - truth| = {float(err[first_bad]):.3e} > allowed {float(allowed[first_bad]):.3e} at "
                             f"position {pos}, the first of {int((~(err <= allowed)).sum())} positions over their limit")
