"""Small Pidodra configurations for the tests, model folders with random weights, and the plain implementation's
logits with an error budget.

The configurations differ from one another in every size and constant, and between them cover the values that one
model may happen to make equal or trivial: layers in every order (latent attention only, grouped attention only), one
head and several, as many key/value heads as heads, one for all and groups of three, value heads smaller, equal and
larger than key heads, sizes that are no multiple of 16 or 8, queries through a latent and straight from the input, a
rotation of all of a head, of a part and none, plain and stretched frequencies in either mixer, layers that read the
keys of the layer just before them or of one further back (two readers of one layer), layers without a feed-forward,
experts in one group, in groups of one, two and more, of which one, some or all groups are kept, all experts chosen,
factors of one on the stream, the embedding and the routing weights.
"""

from __future__ import annotations

import functools
from pathlib import Path

import numpy as np
import torch

from tests.plain import pidodra_plain


def _rot(rot):
    """rot: (dims, base) or (dims, base, (factor, original, fast, slow))."""
    out = {"dims": rot[0], "base": rot[1]}
    if len(rot) > 2:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot[2]))
    return out


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, q_rank=None, rot=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if q_rank is not None:
        m["q_rank"] = q_rank
    if rot is not None:
        m["rot"] = _rot(rot)
    return m


def attention(heads, kv_heads, dim, vdim, scale, rot=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = _rot(rot)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(experts, top, ff, groups=None, scale=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    return {"kind": "moe", "router": router, "expert": {"ff": ff}}


def layer(mixer, mlp=None):
    return {"type": "latent_attention" if "kv_rank" in mixer else "attention", "mixer": mixer, "mlp": mlp}


def model(vocab, width, layers, eps=1e-6, alpha=None, embedding_scale=None):
    out = {"architecture": "Pidodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if alpha is not None:
        out["postln_alpha"] = alpha
    if embedding_scale is not None:
        out["embedding"] = {"scale": embedding_scale}
    return out


YARN = (4.0, 64, 8.0, 2.0)
CASES = {
    # both mixers, a reader right behind its lender and one two layers on, a layer without a feed-forward, queries with and without
    # a latent, stretched frequencies in both mixers
    "a": {"config": model(211, 64, [
        layer(latent(4, 16, 8, 24, 32, 0.2, q_rank=24, rot=(8, 10000.0)), moe(8, 3, 16, groups=(4, 2), scale=1.5)),
        layer(attention(4, 2, 16, 16, 0.25, rot=(16, 10000.0, YARN)), moe(6, 2, 8, groups=(3, 1), scale=2.5)),
        layer(attention(4, 2, 16, 16, 0.3, rot=(16, 10000.0, YARN), kv_from=1)),
        layer(latent(2, 8, 16, 8, 12, 0.3, rot=(16, 500.0, (2.0, 32, 4.0, 1.0))), moe(4, 4, 8)),
        layer(attention(4, 2, 16, 16, 0.2, rot=(16, 10000.0, YARN), kv_from=1), moe(5, 1, 24, groups=(5, 3))),
    ], eps=1e-6, alpha=2.0, embedding_scale=1.5), "seed": 3, "std": 0.08, "page_size": 16},
    # latent attention only; sizes that are no multiple of 8; one head; every expert used; groups of one expert; no rotation at all
    "b": {"config": model(97, 40, [
        layer(latent(3, 12, 6, 20, 10, 0.25, q_rank=7, rot=(6, 77.0)), moe(5, 5, 24, scale=0.5)),
        layer(latent(1, 20, 4, 12, 44, 0.5, q_rank=50, rot=(4, 30.0, (8.0, 16, 4.0, 1.0))), moe(4, 1, 8, groups=(4, 2))),
        layer(latent(5, 4, 2, 4, 6, 0.7)),
    ], eps=2e-5, alpha=0.5), "seed": 5, "std": 0.1, "page_size": 8},
    # grouped attention only: one head; heads of 24 of which 8 dimensions turn; values wider and narrower than keys; groups of three
    # and of eight; a layer without rotation; readers of two different layers; factors of one everywhere
    "c": {"config": model(300, 96, [
        layer(attention(1, 1, 24, 40, 0.2, rot=(8, 100000.0)), moe(12, 4, 24, groups=(3, 2))),
        layer(attention(6, 2, 16, 8, 0.3), moe(3, 2, 16, groups=(3, 3), scale=1.0)),
        layer(attention(1, 1, 24, 40, 0.25, rot=(8, 100000.0), kv_from=0), moe(2, 1, 40, groups=(2, 1))),
        layer(attention(8, 1, 32, 32, 0.18, rot=(32, 300.0, (16.0, 32, 4.0, 0.5)))),
        layer(attention(4, 2, 16, 8, 0.3, kv_from=1), moe(6, 3, 8, groups=(2, 1), scale=3.0)),
        layer(attention(8, 1, 32, 32, 0.2, rot=(32, 300.0, (16.0, 32, 4.0, 0.5)), kv_from=3)),
    ], eps=1e-5), "seed": 8, "std": 0.05, "page_size": 32},
    # heads and latents of 64 and more (the tensor-core kernels' shapes), pages of 4, a reader before and after a latent layer
    "d": {"config": model(128, 96, [
        layer(attention(4, 2, 64, 64, 0.125, rot=(64, 30000.0, (2.0, 128, 16.0, 1.0))), moe(4, 2, 40, groups=(2, 2), scale=2.0)),
        layer(latent(2, 64, 32, 64, 96, 0.1, q_rank=48, rot=(32, 10000.0))),
        layer(attention(2, 2, 64, 64, 0.11, rot=(64, 30000.0, (2.0, 128, 16.0, 1.0)), kv_from=0), moe(2, 1, 40, groups=(2, 1))),
    ], eps=1e-5, alpha=3.5, embedding_scale=0.7), "seed": 13, "std": 0.07, "page_size": 4},
}


def _divisors(n: int) -> list[int]:
    return [d for d in range(1, n + 1) if n % d == 0]


def random_case(seed: int) -> dict:
    """A configuration drawn from a seed: one to five layers of either kind in any order, sizes that are and are not
    multiples of 16, every optional mechanism there or not, readers of any earlier layer that has keys of its own."""
    import random

    rng = random.Random(seed)
    layers, lenders = [], []
    for i in range(rng.randint(1, 5)):
        if rng.random() < 0.5:
            rot_dim = rng.choice([2, 4, 8, 16, 32, 64])
            rot = None
            if rng.random() < 0.85:
                rot = (rot_dim, rng.choice([100.0, 10000.0, 250000.0]))
                if rng.random() < 0.4:
                    rot += ((rng.choice([2.0, 4.0, 16.0]), rng.choice([32, 128, 1024]), rng.choice([8.0, 32.0]), rng.choice([1.0, 2.0])),)
            dim = rng.choice([4, 8, 16, 24, 32, 64, 96, 128])
            mixer = latent(rng.randint(1, 8), dim, rot_dim, rng.choice([dim, 8, 16, 40, 64, 80]), rng.choice([8, 16, 24, 32, 64, 96, 128, 160]),
                           rng.choice([(dim + rot_dim) ** -0.5, 0.1, 0.3]), q_rank=rng.choice([None, 8, 24, 40, 96, 130]), rot=rot)
        elif lenders and rng.random() < 0.4:
            j = rng.choice(lenders)
            lender = layers[j]["mixer"]
            group = lender["heads"] // lender["kv_heads"]
            heads = lender["kv_heads"] * rng.choice([1, group, 2, 3])
            mixer = dict(lender, heads=heads, scale=rng.choice([0.1, 0.2, lender["dim"] ** -0.5]), kv_from=j)
        else:
            dim = rng.choice([8, 12, 16, 24, 32, 48, 64, 80, 128])
            kv_heads = rng.randint(1, 3)
            rot = None
            if rng.random() < 0.85:
                dims = rng.choice(list(range(2, dim + 1, 2))) if rng.random() < 0.4 else dim
                rot = (dims, rng.choice([100.0, 30000.0, 1000000.0]))
                if rng.random() < 0.6:
                    rot += ((rng.choice([2.0, 4.0, 16.0]), rng.choice([32, 128, 1024]), rng.choice([8.0, 32.0]), rng.choice([1.0, 2.0])),)
            mixer = attention(kv_heads * rng.choice([1, 1, 2, 3, 4, 8]), kv_heads, dim, rng.choice([dim, dim, 8, 16, 40, 64, 80]),
                              rng.choice([dim ** -0.5, 0.1, 0.3]), rot=rot)
            lenders.append(i)
        if rng.random() < 0.2:
            mlp = None
        else:
            experts = rng.randint(2, 16)
            groups, size = None, experts
            if rng.random() < 0.7:
                count = rng.choice(_divisors(experts))
                groups, size = (count, rng.randint(1, count)), experts // count
            most = size * (groups[1] if groups else 1)
            mlp = moe(experts, rng.randint(1, min(most, 5)), rng.choice([8, 16, 24, 32, 64]), groups=groups,
                      scale=rng.choice([None, 1.0, 2.0, 0.7]))
        layers.append(layer(mixer, mlp))
    config = model(rng.choice([50, 97, 256, 1000]), rng.choice([24, 40, 64, 72, 100, 128, 200, 320]), layers, eps=rng.choice([1e-6, 1e-5]),
                   alpha=rng.choice([None, 1.0, 2.0, 4.0]), embedding_scale=rng.choice([None, 1.0, 2.5]))
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
    cfg, w = pidodra_plain.read_model(folder)
    return pidodra_plain.forward(cfg, w, list(ids)).numpy()


def plain_logits(folder, ids) -> np.ndarray:
    return _plain_cached(str(folder), tuple(int(i) for i in ids))


@functools.lru_cache(maxsize=64)
def _movement_cached(folder: str, ids: tuple) -> np.ndarray:
    """Per position, how far the plain logits move when the rows that enter every sublayer are disturbed by relative
    noise of 2^-9 (about bfloat16's rounding, which the engine applies in more places), the most over eight draws. A
    position at which a router's choice (of a group or of an expert) hangs on a score gap below 0.01 is excused
    altogether (infinity), and so is every later one of the sequence."""
    cfg, w = pidodra_plain.read_model(folder)
    truth = _plain_cached(folder, ids)
    worst = np.zeros(len(ids))
    pidodra_plain.MARGINS = []
    try:
        pidodra_plain.forward(cfg, w, list(ids))
        for margin in pidodra_plain.MARGINS:
            worst[margin.numpy() < 0.01] = np.inf
        worst = np.maximum.accumulate(worst)
    finally:
        pidodra_plain.MARGINS = None
    for seed in range(8):
        gen = torch.Generator().manual_seed(1000 + seed)
        pidodra_plain.DISTURB = lambda x: x * (1 + 2.0 ** -9 * torch.randn(x.shape, generator=gen, dtype=torch.float64))
        try:
            moved = pidodra_plain.forward(cfg, w, list(ids)).numpy()
        finally:
            pidodra_plain.DISTURB = None
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
