"""Zudalorn without a GPU: configuration keys and their errors, the tensors a checkpoint must hold, the parts that a
configuration becomes, the cache and state members that they ask for, and the plain implementation's own mechanisms
against hand-made cases."""

from __future__ import annotations

import copy
import math

import pytest
import torch

from research_2_b200 import models  # noqa: F401  (registers the architectures)
from research_2_b200.config.registry import ConfigError, architecture_of
from research_2_b200.config.zudalorn import DenseMlp, ExpertsMlp, LatentAttentionMixer, RetentionMixer, Rotation, ZudalornConfig
from research_2_b200.models.zudalorn import model_spec, random_weights, weight_spec
from research_2_b200.weights.loader import WeightError, check_and_select
from tests.plain import zudalorn_plain as plain
from tests.zudalorn_cases import CASES, random_case

F64 = torch.float64


def test_every_case_parses_and_round_trips():
    for name, case in list(CASES.items()) + [(f"seed {s}", random_case(s)) for s in range(100, 130)]:
        arch = architecture_of(case["config"])
        cfg = arch.parse_config(case["config"])
        assert arch.name == "Zudalorn" and isinstance(cfg, ZudalornConfig)
        again = arch.parse_config(arch.config_to_json(cfg))
        assert again == cfg, name


def test_what_a_file_does_not_mention_is_not_there():
    cfg = ZudalornConfig.from_json(CASES["b"]["config"])
    last = cfg.layers[2].mixer
    assert isinstance(last, LatentAttentionMixer) and last.rot is None and last.window == 0
    assert cfg.layers[0].mixer.rot.scaling is None and cfg.layers[1].mixer.rot.scaling.factor == 8.0 and cfg.layers[1].mixer.window == 1
    first = cfg.layers[0].mlp
    assert isinstance(first, ExpertsMlp) and (first.groups, first.keep_groups, first.shared_ff) == (1, 1, 0)
    cfg = ZudalornConfig.from_json(CASES["a"]["config"])
    assert isinstance(cfg.layers[2].mixer, RetentionMixer) and cfg.layers[2].mixer.rot is None and cfg.layers[2].mlp is None
    assert isinstance(cfg.layers[1].mlp, DenseMlp) and cfg.layers[0].mlp.shared_ff == 24 and cfg.layers[3].mlp.shared_ff == 0
    assert cfg.eos_token_id is None


@pytest.mark.parametrize("path, value, text", [
    (("vocab",), None, "'vocab'"), (("width",), 0, "'width'"), (("norm", "eps"), None, "norm.'eps'"),
    (("layers", 0, "type"), "conv", "'type'"), (("layers", 1, "mixer", "heads"), None, "mixer.'heads'"),
    (("layers", 1, "mixer", "kv_rank"), None, "'kv_rank'"), (("layers", 1, "mixer", "rot", "dims"), 7, "even"),
    (("layers", 1, "mixer", "rot", "dims"), 10, "at most"), (("layers", 1, "mixer", "rot", "scaling", "fast"), None, "scaling.'fast'"),
    (("layers", 0, "mixer", "decay"), [0.5], "'decay'"), (("layers", 0, "mixer", "dim"), "x", "'dim'"),
    (("layers", 0, "mlp", "router", "top"), 5, "'top'"), (("layers", 0, "mlp", "router", "groups", "count"), 3, "groups"),
    (("layers", 0, "mlp", "kind"), "sparse", "'kind'"), (("layers", 1, "mlp", "ff"), None, "mlp.'ff'"),
    (("layers", 0, "mlp", "expert", "ff"), None, "expert.'ff'"),
])
def test_errors_name_the_key(path, value, text):
    data = copy.deepcopy(CASES["a"]["config"])
    at = data
    for key in path[:-1]:
        at = at[key]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError) as err:
        ZudalornConfig.from_json(data)
    assert text in str(err.value), str(err.value)


def test_weight_spec_and_loader_errors():
    cfg = ZudalornConfig.from_json(CASES["a"]["config"])
    spec = weight_spec(cfg)
    names = {t.name: t.shape for t in spec.tensors}
    assert names["l1.mix.q"] == (4 * 24, 64) and names["l1.mix.dkv"] == (40, 64) and names["l1.mix.dkv.norm"] == (32,)
    assert names["l1.mix.uk"] == (64, 32) and names["l1.mix.uv"] == (96, 32) and names["l1.mix.o"] == (64, 96)
    assert names["l0.mix.q"] == (32, 64) and names["l0.mix.v"] == (48, 64) and names["l0.mix.g"] == (48, 64) and names["l0.mix.o"] == (64, 48)
    assert names["l0.norm1"] == () and names["l0.norm2b"] == () and names["final.norm"] == ()
    assert names["l0.mlp.e7.down"] == (64, 16) and names["l0.mlp.shared.gate"] == (24, 64) and names["l0.mlp.shared.sg"] == (1, 64)
    assert names["l0.mlp.router"] == (8, 64) and names["l0.mlp.correction"] == (8,) and names["l1.mlp.act"] == (2,)
    assert "l2.norm2" not in names and "l2.norm2b" not in names and not any(n.startswith("l2.mlp.") for n in names), "a layer without a feed-forward"
    assert "l3.mlp.shared.up" not in names and names["l1.mlp.up"] == (96, 64) and names["head"] == (211, 64)
    weights = random_weights(cfg, 0)
    assert set(weights) == set(names) and all(tuple(weights[n].shape) == s for n, s in names.items())
    assert check_and_select(dict(weights), spec).keys() == names.keys()
    broken = dict(weights)
    del broken["l1.mix.dkv.norm"]
    broken["l0.mlp.correction"] = torch.zeros(5)
    broken["l9.extra"] = torch.zeros(1)
    with pytest.raises(WeightError) as err:
        check_and_select(broken, spec)
    assert err.value.missing == ["l1.mix.dkv.norm"] and err.value.unexpected == ["l9.extra"] and "l0.mlp.correction" in err.value.wrong[0]


def test_parts_and_members():
    from research_2_b200.cache.arena import MemberSpec, derive_groups

    cfg = ZudalornConfig.from_json(CASES["a"]["config"])
    spec = model_spec(cfg)
    assert [layer.mixer.kind for layer in spec.layers] == ["retention", "latent_attention", "retention", "latent_attention"]
    assert [None if layer.feed_forward is None else layer.feed_forward.kind for layer in spec.layers] == ["routed_experts", "act_mlp", None, "routed_experts"]
    assert all(layer.block == "sandwich" and layer.post_norm_1 is not None for layer in spec.layers)
    assert spec.layers[2].norm_2 is None and spec.layers[2].post_norm_2 is None and spec.layers[1].post_norm_2.params["width"] == 64
    first = spec.layers[0].feed_forward.params
    assert (first["scoring"], first["n_groups"], first["keep_groups"], first["top"], first["shared"]) == ("sigmoid", 4, 2, 3, True)
    assert spec.layers[3].feed_forward.params["shared"] is False
    att = spec.layers[1].mixer.params
    assert att["window"] == 24 and att["rot_dims"] == 8 and len(att["rot_freqs"]) == 4 and att["rot_magnitude"] == pytest.approx(0.1 * math.log(4.0) + 1.0)
    ret = spec.layers[0].mixer.params
    assert ret["decay"] == [0.9, 0.99] and ret["rot_dims"] == 8 and ret["rot_freqs"] == [1000.0 ** (-2.0 * i / 8) for i in range(4)]
    assert spec.layers[2].mixer.params["rot_dims"] == 0
    # one row of latent + rotated key part per token and no values; windows of 24 and 7: two cache groups
    groups, index = derive_groups([MemberSpec(1, 40, 24, 32, 0, values_in_keys=True), MemberSpec(1, 28, 7, 12, 0, values_in_keys=True)], 16, 10)
    assert [g.window for g in groups] == [24, 7] and index == [0, 1]
    assert MemberSpec(1, 40, 24, 32, 0, values_in_keys=True).stored_value_dim == 0 and MemberSpec(1, 40, 24, 32, 0).stored_value_dim == 32


def test_stretched_frequencies():
    """By hand: 8 dimensions, base 10000, original 64 positions, fast 8 turns, slow 2: the corner indices are
    4 ln(64 / (2 pi t)) / ln(10000) for t = 8 and 2, that is 0.10 and 0.71: lo = 0, hi = 1, so pair 0 keeps its frequency
    and every other pair's is divided by the factor."""
    rot = Rotation.from_json({"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}}, "", 8)
    freqs, magnitude = rot.frequencies()
    plain_f = [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    assert freqs == pytest.approx([plain_f[0], plain_f[1] / 4, plain_f[2] / 4, plain_f[3] / 4]) and magnitude == pytest.approx(0.1 * math.log(4.0) + 1)
    assert plain.yarn_frequencies(8, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0})[0] == pytest.approx(freqs)
    # corners that coincide (a ramp of width 0.001) and corners outside the pairs: all frequencies stay, or all are divided
    stay, _ = Rotation(8, 10000.0, Rotation.from_json({"dims": 8, "base": 10000.0, "scaling": {"factor": 2.0, "original": 10 ** 9, "fast": 1.0, "slow": 1.0}}, "", 8).scaling).frequencies()
    assert stay == pytest.approx(plain_f)
    cut, _ = Rotation.from_json({"dims": 8, "base": 10000.0, "scaling": {"factor": 2.0, "original": 1, "fast": 4.0, "slow": 2.0}}, "", 8).frequencies()
    assert cut[1:] == pytest.approx([f / 2 for f in plain_f[1:]]) and cut[0] == pytest.approx(plain_f[0])
    assert Rotation(8, 10000.0).frequencies() == (plain_f, 1.0)


def test_plain_router_by_hand():
    """Six experts in three groups of two, one group kept. Scores + corrections: group sums decide, not the best
    expert; the weights use the scores without the correction."""
    z = torch.tensor([[2.0, -2.0, 1.0, 1.0, -1.0, 3.0]], dtype=F64)
    s = torch.sigmoid(z)[0]
    none = torch.zeros(6, dtype=F64)
    chosen, weights = plain.route(z, none, 2, 3, 1)
    assert sorted(chosen[0]) == [2, 3], "the group with the largest sum of two, not the one with the best expert"
    assert torch.allclose(weights[0], torch.tensor([0.5, 0.5], dtype=F64))
    chosen, weights = plain.route(z, none, 2, 1, 1)
    assert chosen[0] == [5, 0] and torch.allclose(weights[0], torch.stack([s[5], s[0]]) / (s[5] + s[0]))
    correction = torch.tensor([0.0, 0.0, 0.0, 0.0, 2.0, 0.0], dtype=F64)
    chosen, weights = plain.route(z, correction, 1, 3, 1)
    assert chosen[0] == [4] and float(weights[0][0]) == pytest.approx(1.0), "chosen by the corrected score, weighted by the plain one"
    # negative choice scores: experts outside the kept groups never win, although their scores are larger than the kept ones'
    correction = torch.tensor([-5.0, -5.0, -9.0, -9.0, -9.0, -9.0], dtype=F64)
    chosen, _ = plain.route(z, correction, 2, 3, 1)
    assert sorted(chosen[0]) == [0, 1]
    # groups of one expert: a group's sum is its expert's score
    chosen, _ = plain.route(z, none, 2, 6, 2)
    assert chosen[0] == [5, 0]


def test_plain_retention_and_window_by_hand():
    # retention: o_t = sum_j decay^(t - j) (q_t . k_j) v_j
    gen = torch.Generator().manual_seed(0)
    q, k = torch.randn(6, 1, 4, generator=gen, dtype=F64), torch.randn(6, 1, 4, generator=gen, dtype=F64)
    v = torch.randn(6, 1, 3, generator=gen, dtype=F64)
    out = plain.retention_cells(q, k, v, torch.tensor([0.8], dtype=F64))
    want = sum(0.8 ** (5 - j) * float(q[5, 0] @ k[j, 0]) * v[j, 0] for j in range(6))
    assert torch.allclose(out[5, 0], want)
    # xIELU: continuous at zero with slope 1/2 on both sides, quadratic on the right
    z = torch.tensor([-1e-6, 0.0, 1e-6, 2.0, -30.0], dtype=F64)
    y = plain.xielu(z, 0.3, -0.2)
    sp, sq = math.log1p(math.exp(0.3)), math.log1p(math.exp(-0.2))
    assert float(y[1]) == 0.0 and float(y[2] - y[0]) == pytest.approx(1e-6, rel=1e-3)
    assert float(y[3]) == pytest.approx(sp * 4 + 1.0) and float(y[4]) == pytest.approx((0.5 + sq) * (math.exp(-30) - 1 + 30) - 15)
    # the interleaved and the half layout pair different dimensions
    x = torch.arange(8, dtype=F64).reshape(1, 8) + 1
    a = plain.rotate(x, [3], [0.5, 0.25], "interleaved")
    b = plain.rotate(x, [3], [0.5, 0.25], "half")
    c, s_ = math.cos(1.5), math.sin(1.5)
    assert float(a[0, 0]) == pytest.approx(1 * c - 2 * s_) and float(a[0, 1]) == pytest.approx(2 * c + 1 * s_)
    assert float(b[0, 0]) == pytest.approx(1 * c - 3 * s_) and float(b[0, 2]) == pytest.approx(3 * c + 1 * s_)
    assert torch.equal(a[0, 4:], x[0, 4:]) and torch.equal(b[0, 4:], x[0, 4:])
