"""Milivik without a GPU: the configuration reader, the builder's tensor list against the one the
tests derive on their own, cache groups, the table of slowed frequencies, and the plain
implementation against itself (token by token through its kept keys against whole prompts; a
window as long as the prompt is no window; a query that is aimed at one key)."""
import copy
import math

import pytest
import torch

import milivik_util as mu
import plain_milivik as plain
import replay_util as ru


def build(config):
    from dispec_b200.config.model_config import load_model_config
    from dispec_b200.weights.loader import build_model
    cfg = load_model_config(copy.deepcopy(config))
    return cfg, build_model(cfg)


@pytest.mark.parametrize("name", sorted(mu.CONFIGS))
def test_builder_asks_for_exactly_the_checkpoint_tensors(name):
    from dispec_b200.config.model_config import load_model_config
    config = mu.CONFIGS[name]["config"]
    cfg, m = build(config)
    assert load_model_config(cfg.to_dict()) == cfg
    req = m.tensor_requirements()
    want = plain.tensor_shapes(config)
    assert set(req) == set(want)
    for n, spec in req.items():
        assert tuple(spec.shape) == tuple(want[n]), n
    assert [c.layer for c in m.schedule] == list(range(len(config["layers"])))


def test_cache_groups_follow_the_mixers_and_their_windows():
    _, m = build(mu.CONFIGS["mix"]["config"])
    got = sorted((g.window, [(t.name, t.num_heads, t.width) for t in g.tensors], g.num_slots) for g in m.cache_groups)
    # the two maps' key parts lie side by side in one cached key of twice the width
    assert got == [(0, [("key", 2, 16), ("value", 2, 16)], 1), (0, [("key", 2, 32), ("value", 2, 8)], 1),
                   (0, [("latent", 1, 16), ("rotated_key", 1, 16)], 1), (20, [("latent", 1, 24), ("rotated_key", 1, 8)], 1)]
    assert m.state_needs == []


def test_the_norm_of_a_missing_feed_forward_may_be_present():
    _, m = build(mu.CONFIGS["mix"]["config"])  # its third layer has no feed-forward
    assert m.spec.optional_tensors == {"l2.norm2"}


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="conv"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "at most"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "not implemented"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "ff"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_errors_name_the_key(change, word):
    from dispec_b200.config.model_config import ConfigError, load_model_config
    c = copy.deepcopy(mu.CONFIGS["mix"]["config"])
    change(c)
    with pytest.raises(ConfigError) as e:
        load_model_config(c)
    assert word in str(e.value)


def test_part_constructors_refuse_what_cannot_run():
    from dispec_b200.parts.attention import DifferentialAttention
    from dispec_b200.parts.latent_attention import LatentAttention
    from dispec_b200.parts.moe import GatedMoE
    from dispec_b200.parts.rotary import RotaryEncoding
    with pytest.raises(ValueError):
        DifferentialAttention(16, 4, 3, 8, 8, 0.5, 0.3, 1e-6, None)
    with pytest.raises(ValueError):
        DifferentialAttention(16, 4, 2, 8, 8, 0.5, 0.3, 1e-6, None, q_temp=(0.5, 0))
    with pytest.raises(ValueError):
        LatentAttention(16, 2, 8, 4, 8, 8, 8, 0.5, 1e-6, None, gate="row")
    with pytest.raises(ValueError):
        GatedMoE(16, 8, 6, top=2, limit=None, group_score="mean")
    with pytest.raises(ValueError):
        GatedMoE(16, 8, 6, top=2, limit=None, shared_gate=True)
    with pytest.raises(ValueError):
        RotaryEncoding(16, 10000.0, slowed=(0.0, 64, 16, 1))


@pytest.mark.parametrize("dims,base,slowed", [(8, 10000.0, (4.0, 64, 16.0, 2.0)), (6, 300.0, (1.5, 20, 4.0, 1.0)),
                                              (32, 1e6, (8.0, 4096, 32.0, 1.0)), (64, 20000.0, (40.0, 512, 1.0, 1.0)),
                                              (16, 50.0, None)])
def test_slowed_frequencies_of_the_rotary_part_are_the_plain_ones(dims, base, slowed):
    from dispec_b200.parts.rotary import RotaryEncoding
    enc = RotaryEncoding(dims, base, layout="halves", exact_table=True, slowed=slowed)
    enc.prepare("cpu")
    rot = {"dims": dims, "base": base}
    if slowed:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), slowed))
    freq, mag = plain.yarn_table(rot)
    got = enc.rotation()
    assert got.layout == "halves" and got.rotary_dim == dims
    assert abs(got.magnitude - mag) < 1e-12 and (got.magnitude > 1.0) == bool(slowed and slowed[0] > 1)
    assert (got.inv_freq.double() - freq).abs().max() <= 1e-7 * freq.abs().max()
    if slowed:  # the fastest pair keeps its frequency or is blended, the slowest is divided by the factor or blended
        plainf = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        assert ((freq <= plainf * (1 + 1e-12)) & (freq >= plainf / slowed[0] * (1 - 1e-12))).all()


# ------------------------------------------------------------------ the plain implementation against itself
@pytest.mark.parametrize("name", ["mix", "odd"])
def test_plain_token_by_token_equals_plain_whole_prompt(name):
    config = mu.CONFIGS[name]["config"]
    weights = mu.random_weights(config, mu.CONFIGS[name]["seed"])
    ids = ru.random_ids(45, config["vocab"], 3)
    whole, _ = plain.forward(config, weights, ids)
    past, rows, start = None, [], 0
    for stop in (17, 18, 30, 45):  # a portion, a single token, portions again
        logits, past = plain.forward(config, weights, ids[start:stop], pos=torch.arange(start, stop), past=past)
        rows.append(logits)
        start = stop
    assert (torch.cat(rows) - whole).abs().max() < 1e-9


def test_plain_window_as_long_as_the_prompt_is_no_window():
    config = copy.deepcopy(mu.CONFIGS["mix"]["config"])
    weights = mu.random_weights(config, 5)
    ids = ru.random_ids(30, config["vocab"], 4)
    base, _ = plain.forward(config, weights, ids)
    for e in config["layers"]:
        e["mixer"]["mask"] = {"size": 30}
    same, _ = plain.forward(config, weights, ids)
    config["layers"][2]["mixer"]["mask"] = {"size": 29}  # the last position loses its first key
    less, _ = plain.forward(config, weights, ids)
    wide = copy.deepcopy(mu.CONFIGS["mix"]["config"])
    for e in wide["layers"]:
        e["mixer"].pop("mask", None)
    assert (plain.forward(wide, weights, ids)[0][:7] - base[:7]).abs().max() < 1e-12  # up to the shortest window
    for e in wide["layers"]:
        e["mixer"]["mask"] = {"size": 30}
    assert (plain.forward(wide, weights, ids)[0] - same).abs().max() < 1e-12
    assert (less[:29] - same[:29]).abs().max() < 1e-12 and (less[29] - same[29]).abs().max() > 1e-9


def test_plain_softmax_attention_sees_exactly_the_window():
    q = torch.zeros(1, 1, 4, dtype=plain.F)
    q[0, 0, 0] = 50.0
    k = torch.zeros(10, 1, 4, dtype=plain.F)
    v = torch.arange(10, dtype=plain.F).view(10, 1, 1)
    pos_k = torch.arange(10)
    for aimed in range(10):
        kk = k.clone()
        kk[aimed, 0, 0] = 1.0
        out = plain.softmax_attention(q, kk, v, torch.tensor([7]), pos_k, 1.0, 4)  # position 7 sees 4..7
        if 4 <= aimed <= 7:
            assert abs(float(out) - aimed) < 1e-6
        else:
            assert abs(float(out) - 5.5) < 1e-9  # no score stands out: the mean of the visible values


def test_plain_router_keeps_groups_by_the_sum_of_their_two_best():
    W = {"r.router": torch.eye(6, dtype=plain.F)}
    # scores rise with the logits; group 0 = experts 0-1, group 1 = 2-3, group 2 = 4-5
    h = torch.tensor([[3.0, -9.0, 1.0, 0.9, 0.5, 0.4]], dtype=plain.F)  # the best expert sits in a group with a poor second
    ids, w = plain.route(h, W, "r.", {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}})
    assert sorted(ids[0].tolist()) == [2, 3] and abs(float(w.sum()) - 2.0) < 1e-9
    ids, w = plain.route(h, W, "r.", {"experts": 6, "top": 2, "scale": 1.0, "groups": {"count": 3, "keep": 2}})
    assert sorted(ids[0].tolist()) == [2, 3]  # groups 1 and 2 stay open: 1.44 and 1.22 against 0.95
    h[0, 4:] = -2.0
    ids, w = plain.route(h, W, "r.", {"experts": 6, "top": 2, "scale": 1.0, "groups": {"count": 3, "keep": 2}})
    assert sorted(ids[0].tolist()) == [0, 2]
    s = torch.sigmoid(torch.tensor([3.0, 1.0], dtype=plain.F))
    assert (w[0].sort().values - (s / s.sum()).sort().values).abs().max() < 1e-12
    ids, _ = plain.route(h, W, "r.", {"experts": 6, "top": 3, "scale": 1.0})
    assert sorted(ids[0].tolist()) == [0, 2, 3]


def test_plain_query_temperature_and_lambda():
    t = plain.query_temperature(torch.tensor([0, 1, 2, 3, 7, 8]), {"coef": 0.5, "every": 4})
    want = [1.0, 1.0, 1.0, 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(3), 1 + 0.5 * math.log(3)]
    assert (t - torch.tensor(want, dtype=plain.F)).abs().max() < 1e-12
    W = {"x.lq1": torch.tensor([1.0, 2.0]), "x.lk1": torch.tensor([0.5, 0.25]), "x.lq2": torch.tensor([0.0, 1.0]),
         "x.lk2": torch.tensor([3.0, -1.0])}
    assert abs(plain.diff_lambda(W, "x.", 0.2) - (math.e - math.exp(-1.0) + 0.2)) < 1e-12
