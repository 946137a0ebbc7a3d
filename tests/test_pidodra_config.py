"""Pidodra without a GPU: configuration keys and their errors, the tensors a checkpoint must hold, the parts and the
schedule that a configuration becomes, the cache members that they ask for, and the plain implementation's own
mechanisms against hand-made cases."""

from __future__ import annotations

import copy
import math

import pytest
import torch

from research_2_b200 import models  # noqa: F401  (registers the architectures)
from research_2_b200.config.pidodra import AttentionMixer, ExpertsMlp, LatentAttentionMixer, PidodraConfig
from research_2_b200.config.registry import ConfigError, architecture_of
from research_2_b200.models.pidodra import model_spec, random_weights, weight_spec
from research_2_b200.weights.loader import WeightError, check_and_select
from tests.pidodra_cases import CASES, random_case
from tests.plain import pidodra_plain as plain

F64 = torch.float64


def test_every_case_parses_and_round_trips():
    for name, case in list(CASES.items()) + [(f"seed {s}", random_case(s)) for s in range(100, 140)]:
        arch = architecture_of(case["config"])
        cfg = arch.parse_config(case["config"])
        assert arch.name == "Pidodra" and isinstance(cfg, PidodraConfig)
        again = arch.parse_config(arch.config_to_json(cfg))
        assert again == cfg, name
        spec = model_spec(cfg)
        assert len(spec.schedule) == len(cfg.layers)


def test_what_a_file_does_not_mention_is_not_there():
    cfg = PidodraConfig.from_json(CASES["b"]["config"])
    last = cfg.layers[2].mixer
    assert isinstance(last, LatentAttentionMixer) and last.rot is None and last.q_rank == 0 and cfg.layers[2].mlp is None
    assert cfg.layers[0].mixer.rot.scaling is None and cfg.layers[1].mixer.rot.scaling.factor == 8.0 and cfg.layers[0].mixer.q_rank == 7
    first = cfg.layers[0].mlp
    assert isinstance(first, ExpertsMlp) and (first.groups, first.keep_groups, first.scale) == (1, 1, 0.5)
    assert cfg.embedding_scale == 1.0 and cfg.alpha == 0.5 and cfg.eos_token_id is None
    cfg = PidodraConfig.from_json(CASES["c"]["config"])
    assert cfg.alpha == 1.0 and cfg.layers[0].mlp.scale == 1.0
    second = cfg.layers[1].mixer
    assert isinstance(second, AttentionMixer) and second.rot is None and second.kv_from is None and cfg.layers[4].mixer.kv_from == 1
    data = copy.deepcopy(CASES["c"]["config"])
    del data["layers"][1]["mixer"]["kv_heads"], data["layers"][1]["mixer"]["vdim"], data["layers"][4]["mixer"]["kv_from"]
    loose = PidodraConfig.from_json(data).layers[1].mixer
    assert (loose.kv_heads, loose.vdim) == (6, 16)


@pytest.mark.parametrize("path, value, text", [
    (("vocab",), None, "'vocab'"), (("width",), 0, "'width'"), (("norm", "eps"), None, "norm.'eps'"), (("postln_alpha",), "x", "'postln_alpha'"),
    (("embedding", "scale"), -1.0, "embedding.'scale'"), (("layers", 0, "type"), "conv", "'type'"), (("layers", 0, "mixer", "heads"), None, "mixer.'heads'"),
    (("layers", 0, "mixer", "kv_rank"), None, "'kv_rank'"), (("layers", 0, "mixer", "rot", "dims"), 7, "even"),
    (("layers", 0, "mixer", "rot", "dims"), 10, "at most"), (("layers", 1, "mixer", "rot", "scaling", "fast"), None, "scaling.'fast'"),
    (("layers", 1, "mixer", "kv_heads"), 3, "multiple"), (("layers", 1, "mixer", "dim"), "x", "'dim'"),
    (("layers", 2, "mixer", "kv_from"), 0, "'kv_from'"), (("layers", 2, "mixer", "kv_from"), 2, "'kv_from'"), (("layers", 2, "mixer", "vdim"), 8, "equal"),
    (("layers", 4, "mixer", "kv_from"), 2, "'kv_from'"),
    (("layers", 0, "mlp", "router", "top"), 5, "'top'"), (("layers", 0, "mlp", "router", "groups", "count"), 3, "groups"),
    (("layers", 0, "mlp", "kind"), "dense", "'kind'"), (("layers", 0, "mlp", "expert", "ff"), None, "expert.'ff'"),
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
        PidodraConfig.from_json(data)
    assert text in str(err.value), str(err.value)


def test_weight_spec_and_loader_errors():
    cfg = PidodraConfig.from_json(CASES["a"]["config"])
    spec = weight_spec(cfg)
    names = {t.name: t.shape for t in spec.tensors}
    assert names["l0.mix.dq"] == (24, 64) and names["l0.mix.dq.norm"] == (24,) and names["l0.mix.uq"] == (4 * 24, 24) and "l0.mix.q" not in names
    assert names["l0.mix.dkv"] == (40, 64) and names["l0.mix.dkv.norm"] == (32,) and names["l0.mix.uk"] == (64, 32) and names["l0.mix.uv"] == (96, 32)
    assert names["l0.mix.sink"] == (4,) and names["l0.mix.g"] == (96, 64) and names["l0.mix.o"] == (64, 96)
    assert names["l3.mix.q"] == (2 * 24, 64) and "l3.mix.dq" not in names, "queries straight from the input"
    assert names["l1.mix.q"] == (64, 64) and names["l1.mix.k"] == (32, 64) and names["l1.mix.v"] == (32, 64) and names["l1.mix.g"] == (4, 64)
    assert names["l1.mix.q.norm"] == (16,) and names["l1.mix.k.norm"] == (16,) and names["l1.mix.o"] == (64, 64)
    assert names["l2.mix.q"] == (64, 64) and names["l2.mix.q.norm"] == (16,), "a reader has queries of its own"
    assert not any(n in names for n in ("l2.mix.k", "l2.mix.v", "l2.mix.k.norm", "l4.mix.k")), "and no keys or values"
    assert names["l0.norm1"] == (64,) and names["l0.norm2"] == (64,) and names["final.norm"] == (64,) and names["head"] == (211, 64)
    assert "l2.norm2" not in names and not any(n.startswith("l2.mlp.") for n in names), "a layer without a feed-forward"
    assert names["l0.mlp.e7.down"] == (64, 16) and names["l0.mlp.router"] == (8, 64) and names["l4.mlp.e4.gate"] == (24, 64)
    weights = random_weights(cfg, 0)
    assert set(weights) == set(names) and all(tuple(weights[n].shape) == s for n, s in names.items())
    assert check_and_select(dict(weights), spec).keys() == names.keys()
    broken = dict(weights)
    del broken["l0.mix.dq.norm"]
    broken["l0.mix.sink"] = torch.zeros(5)
    broken["l2.mix.k"] = torch.zeros(32, 64)
    with pytest.raises(WeightError) as err:
        check_and_select(broken, spec)
    assert err.value.missing == ["l0.mix.dq.norm"] and err.value.unexpected == ["l2.mix.k"] and "l0.mix.sink" in err.value.wrong[0]


def test_parts_schedule_and_members():
    from research_2_b200.cache.arena import MemberSpec, derive_groups

    cfg = PidodraConfig.from_json(CASES["a"]["config"])
    spec = model_spec(cfg)
    assert [layer.mixer.kind for layer in spec.layers] == ["latent_attention", "rotary_window_attention", "rotary_window_attention", "latent_attention",
                                                           "rotary_window_attention"]
    assert [None if layer.feed_forward is None else layer.feed_forward.kind for layer in spec.layers] == ["routed_experts"] * 2 + [None] + ["routed_experts"] * 2
    assert all(layer.block == "post_norm" and layer.block_params == {"alpha": 2.0} for layer in spec.layers) and spec.embedding_scale == 1.5
    assert spec.layers[2].norm_2 is None
    # layers with keys of their own get the members 0, 1, 2 in order; the readers name member 1 and do not write it
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 1, False), (3, 2, True), (4, 1, False)]
    first = spec.layers[0].feed_forward.params
    assert (first["scoring"], first["group_mark"], first["normalise"], first["route_scale"]) == ("softmax", "best", False, 1.5)
    assert (first["n_groups"], first["keep_groups"], first["top"], first["activation"]) == (4, 2, 3, "silu")
    att = spec.layers[1].mixer.params
    assert att["rot_dims"] == 16 and len(att["rot_freqs"]) == 8 and att["rot_magnitude"] == pytest.approx(0.1 * math.log(4.0) + 1.0) and att["qk_norm_eps"] == 1e-6
    assert "w_k" not in spec.layers[2].mixer.weights and "k_norm" not in spec.layers[2].mixer.weights and "w_k" in spec.layers[1].mixer.weights
    lat = spec.layers[0].mixer
    assert lat.params["rot_magnitude"] == 1.0 and lat.params["window"] == 0 and {"w_dq", "dq_norm", "w_uq", "sink", "w_gate"} <= set(lat.weights)
    assert "w_q" in spec.layers[3].mixer.weights and "w_dq" not in spec.layers[3].mixer.weights
    # no windows anywhere: one cache group for rows of latents and for keys and values alike
    groups, index = derive_groups([MemberSpec(1, 40, 0, 32, 0, values_in_keys=True), MemberSpec(2, 16, 0, 16, 0), MemberSpec(1, 28, 0, 12, 0, values_in_keys=True)], 16, 10)
    assert len(groups) == 1 and index == [0, 0, 0]


def test_plain_router_by_hand():
    """Six experts in three groups of two, two groups kept. The scores are a softmax over all six; a group counts by its
    best expert, not by a sum; the weights are the chosen scores times the factor and do not sum to one."""
    z = torch.tensor([[2.0, -2.0, 1.8, 1.8, -1.0, 3.0]], dtype=F64)
    s = torch.softmax(z, dim=-1)[0]
    chosen, weights = plain.route(z, 2, 3, 1, 2.0)
    assert chosen[0] == [5, 4], "only the group of the best expert is kept, so its weak neighbour is chosen too"
    assert torch.allclose(weights[0], torch.stack([s[5], s[4]]) * 2.0) and float(weights[0].sum()) < 2.0
    chosen, weights = plain.route(z, 3, 3, 2, 1.0)
    assert chosen[0] == [5, 0, 4], "groups 2 (best 3.0) and 0 (best 2.0) are kept; group 1, whose two scores sum to more than group 0's, is not"
    assert torch.allclose(weights[0], torch.stack([s[5], s[0], s[4]]))
    chosen, _ = plain.route(z, 2, 1, 1, 1.0)
    assert chosen[0] == [5, 0]
    chosen, weights = plain.route(z, 6, 6, 6, 0.5)
    assert sorted(chosen[0]) == list(range(6)) and float(weights[0].sum()) == pytest.approx(0.5), "all experts: the scores sum to one"
    # equal scores: the lower index wins, among groups and among experts
    chosen, _ = plain.route(torch.zeros(1, 6, dtype=F64), 2, 3, 1, 1.0)
    assert chosen[0] == [0, 1]


def test_plain_sink_rotations_and_sums_by_hand():
    # a sink takes its share of the softmax and gives nothing: two equal scores and a sink as large as them leave a third each
    weights = plain.softmax_with_sink(torch.tensor([[1.0, 1.0]], dtype=F64), torch.tensor([1.0], dtype=F64))
    assert torch.allclose(weights, torch.full((1, 2), 1.0 / 3, dtype=F64))
    weights = plain.softmax_with_sink(torch.tensor([[0.0]], dtype=F64), torch.tensor([-800.0], dtype=F64))
    assert float(weights[0, 0]) == 1.0
    weights = plain.softmax_with_sink(torch.tensor([[0.0]], dtype=F64), torch.tensor([800.0], dtype=F64))
    assert float(weights[0, 0]) == 0.0
    # the interleaved and the half layout pair different dimensions; a magnitude scales both parts
    x = torch.arange(8, dtype=F64).reshape(1, 8) + 1
    a = plain.rotate(x, [3], [0.5, 0.25], "interleaved", 1.2)
    b = plain.rotate(x, [3], [0.5, 0.25], "half")
    c, s_ = math.cos(1.5), math.sin(1.5)
    assert float(a[0, 0]) == pytest.approx(1.2 * (1 * c - 2 * s_)) and float(a[0, 1]) == pytest.approx(1.2 * (2 * c + 1 * s_))
    assert float(b[0, 0]) == pytest.approx(1 * c - 3 * s_) and float(b[0, 2]) == pytest.approx(3 * c + 1 * s_)
    assert torch.equal(a[0, 4:], x[0, 4:]) and torch.equal(b[0, 4:], x[0, 4:])
    # stretched frequencies by hand: 8 dimensions, base 10000, 64 positions, fast 8 turns, slow 2: corner indices 0.10 and 0.71, so
    # pair 0 keeps its frequency and every other pair's is divided by the factor
    freqs, magnitude = plain.frequencies({"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}})
    plain_f = [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    assert freqs == pytest.approx([plain_f[0], plain_f[1] / 4, plain_f[2] / 4, plain_f[3] / 4]) and magnitude == pytest.approx(0.1 * math.log(4.0) + 1)
    # a one-layer model by hand: x1 = norm(alpha x0 + mixer(x0)); with a mixer whose output matrix is zero the layer is a norm of x0
    case = {"architecture": "Pidodra", "vocab": 5, "width": 4, "norm": {"eps": 1e-12}, "postln_alpha": 3.0, "embedding": {"scale": 2.0},
            "layers": [{"type": "attention", "mixer": {"heads": 1, "dim": 2, "scale": 1.0}, "mlp": None}]}
    w = random_weights(PidodraConfig.from_json(case), 1)
    w = {n: t.to(F64) for n, t in w.items()}
    w["l0.mix.o"] = torch.zeros_like(w["l0.mix.o"])
    stream: list = []
    plain.forward(case, w, [1, 4], layers_out=stream)
    x0 = w["embed"][[1, 4]] * 2.0
    assert torch.allclose(stream[0], x0 / x0.pow(2).mean(-1, keepdim=True).sqrt() * w["l0.norm1"])
