"""Desalix without a GPU: the configuration reader, the builder's tensor list against the one the
tests derive on their own, the order of the layer runs with their caches, and the plain
implementation against itself (a chunk as long as the prompt is no chunk; values enter the sum
turned by the distance; the sink; the order of the runs)."""
import copy
import math

import pytest
import torch

import desalix_util as du
import plain_desalix as plain
import replay_util as ru


def build(config):
    from dispec_b200.config.model_config import load_model_config
    from dispec_b200.weights.loader import build_model
    cfg = load_model_config(copy.deepcopy(config))
    return cfg, build_model(cfg)


@pytest.mark.parametrize("name", sorted(du.CONFIGS))
def test_builder_asks_for_exactly_the_checkpoint_tensors(name):
    from dispec_b200.config.model_config import load_model_config
    config = du.CONFIGS[name]["config"]
    cfg, m = build(config)
    assert load_model_config(cfg.to_dict()) == cfg
    req = m.tensor_requirements()
    want = du.tensor_shapes(config)
    assert set(req) == set(want)
    for n, spec in req.items():
        assert tuple(spec.shape) == tuple(want[n]), n


@pytest.mark.parametrize("name", sorted(du.CONFIGS))
def test_schedule_follows_the_plain_order_of_runs_and_every_run_has_a_cache_of_its_own(name):
    config = du.CONFIGS[name]["config"]
    cfg, m = build(config)
    assert [(c.layer, c.entry) for c in m.schedule] == plain.layer_runs(config)
    labels = [m.call_cache[i] for i in range(len(m.schedule))]
    assert len(set(labels)) == len(labels) and all(c.write for c in m.schedule)
    assert sum(g.num_slots for g in m.cache_groups) == len(m.schedule)
    assert (m.pass_entry is not None) == bool(config.get("loop"))


def test_cache_groups_follow_the_mixers_and_their_chunks():
    _, m = build(du.CONFIGS["mix"]["config"])
    got = sorted((g.window, [(t.name, t.num_heads, t.width) for t in g.tensors], g.num_slots) for g in m.cache_groups)
    assert got == [(0, [("key", 2, 8), ("value", 2, 12)], 3), (7, [("key", 2, 16), ("value", 2, 8)], 3),
                   (20, [("key", 2, 16), ("value", 2, 8)], 1), (40, [("key", 1, 24), ("value", 1, 8)], 3)]
    assert m.state_needs == []


def test_an_empty_or_missing_loop_repeats_nothing():
    c = copy.deepcopy(du.CONFIGS["mix"]["config"])
    c["loop"] = {"start": 2, "stop": 2, "times": 5}
    cfg, m = build(c)
    assert [x.layer for x in m.schedule] == [0, 1, 2, 3] and m.pass_entry is None
    c["loop"] = {"start": 0, "stop": 4, "times": 2}
    assert [(x.layer, x.entry) for x in build(c)[1].schedule] == [(0, 0), (1, None), (2, None), (3, None),
                                                                  (0, 1), (1, None), (2, None), (3, None)]


def test_tensors_of_pieces_a_model_lacks_may_be_present():
    c = copy.deepcopy(du.CONFIGS["mix"]["config"])  # its third layer has no feed-forward
    _, m = build(c)
    assert m.spec.optional_tensors == {"l2.norm2", "l2.norm2b", "l2.ls2"}
    c["loop"] = {"start": 2, "stop": 2, "times": 5}
    assert "loop.step" in build(c)[1].spec.optional_tensors


def test_a_single_number_may_be_stored_with_dimensions():
    from dispec_b200.weights.loader import check_source

    config = du.CONFIGS["flat"]["config"]
    _, m = build(config)
    shapes = du.tensor_shapes(config)
    shapes["final.norm"], shapes["l0.norm1"] = (1,), (1, 1)

    class Source:
        names = lambda self: list(shapes)
        shape = lambda self, n: shapes[n]
        dtype = lambda self, n: torch.bfloat16

    check_source(m, Source(), "test")
    shapes["l1.norm2b"] = (2,)
    with pytest.raises(Exception, match="l1.norm2b"):
        check_source(m, Source(), "test")


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="conv"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "at most"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=7), "odd"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not implemented"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_errors_name_the_key(change, word):
    from dispec_b200.config.model_config import ConfigError, load_model_config
    c = copy.deepcopy(du.CONFIGS["mix"]["config"])
    change(c)
    with pytest.raises(ConfigError) as e:
        load_model_config(c)
    assert word in str(e.value)


def test_part_constructors_refuse_what_cannot_run():
    from dispec_b200.parts.attention import SinkAttention
    from dispec_b200.parts.block import PassEntry
    from dispec_b200.parts.moe import GatedMoE
    with pytest.raises(ValueError):
        GatedMoE(16, 8, 6, top=7, limit=1.0)
    with pytest.raises(ValueError):
        GatedMoE(16, 8, 6, top=2, limit=0.0)
    with pytest.raises(ValueError):
        GatedMoE(16, 8, 6, top=2, limit=1.0, score="tanh")
    with pytest.raises(ValueError):
        SinkAttention(16, 4, 2, 8, 8, 0.3, None, sink="maybe")
    with pytest.raises(ValueError):
        SinkAttention(16, 4, 2, 8, 8, 0.3, None, mask="stripes")
    with pytest.raises(ValueError):
        SinkAttention(16, 4, 2, 8, 7, 0.3, None, value_theta=100.0)
    with pytest.raises(ValueError):
        SinkAttention(16, 4, 2, 8, 8, 0.3, None, value_norm=True, value_mix=("source", "v"))
    with pytest.raises(ValueError):
        PassEntry(16, 0)


# ------------------------------------------------------------- the plain implementation itself
def _qkv(T, H, G, d, dv, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(T, H, d, generator=g).double(), torch.randn(T, G, d, generator=g).double(),
            torch.randn(T, G, dv, generator=g).double())


def test_plain_chunk_as_long_as_the_prompt_is_no_chunk_and_the_sink_takes_its_share():
    q, k, v = _qkv(9, 4, 2, 6, 5, 1)
    pos = torch.arange(9)
    sink = torch.tensor([0.3, -1.0, 2.0, 0.0]).double()
    a = plain.sink_softmax_attention(q, k, v, pos, pos, 0.4, 0, sink)
    b = plain.sink_softmax_attention(q, k, v, pos, pos, 0.4, 9, sink)
    c = plain.sink_softmax_attention(q, k, v, pos, pos, 0.4, 4, sink)
    assert torch.allclose(a, b) and not torch.allclose(a, c)
    # the first token of every chunk sees itself and the sink: its weight is exp(s) / (exp(sink) + exp(s))
    for t in (0, 4, 8):
        for h in range(4):
            s = (q[t, h] @ k[t, h // 2]) * 0.4
            assert torch.allclose(c[t, h], v[t, h // 2] * math.exp(s) / (math.exp(sink[h]) + math.exp(s)))
    # position 3 and position 4 are neighbours in different chunks
    assert torch.allclose(c[3], a[3]) and not torch.allclose(c[4], a[4])


def test_plain_values_enter_the_sum_turned_by_the_distance():
    """Turning every value by its position and the sum back by the query's is the same as adding up
    values turned by (key position - query position)."""
    g = torch.Generator().manual_seed(3)
    T, dv, base = 7, 8, 50.0
    v = torch.randn(T, 1, dv, generator=g).double()
    w = torch.softmax(torch.randn(T, T, generator=g).double().tril() - 1e9 * torch.ones(T, T).triu(1), -1)
    pos = torch.arange(T)
    turned = plain.turn_halves(v, pos, base, dv)
    out = plain.turn_halves((w @ turned[:, 0])[:, None], pos, base, dv, sign=-1.0)[:, 0]
    for i in range(T):
        want = sum(w[i, j] * plain.turn_halves(v[j:j + 1], torch.tensor([j - i]), base, dv)[0, 0] for j in range(i + 1))
        assert torch.allclose(out[i], want)
    # a sum that holds one value alone gives that value back whatever the positions
    one = plain.turn_halves(plain.turn_halves(v, pos, base, dv), pos, base, dv, sign=-1.0)
    assert torch.allclose(one, v)


def test_plain_turn_keeps_the_dimensions_behind_the_turned_ones_and_pairs_halves():
    x = torch.arange(12.0).double().view(1, 1, 12)
    y = plain.turn_halves(x, torch.tensor([1]), 1.0, 4)  # every frequency 1: a turn by one radian
    assert torch.equal(y[..., 4:], x[..., 4:])
    c, s = math.cos(1.0), math.sin(1.0)
    assert torch.allclose(y[0, 0, :4], torch.tensor([0 * c - 2 * s, 1 * c - 3 * s, 2 * c + 0 * s, 3 * c + 1 * s]).double())


def test_plain_router_takes_the_largest_sigmoids_without_renormalising():
    z = torch.tensor([0.1, 2.0, -1.0, 2.0, 0.5]).double()
    chosen, s = plain.route(z, 3)
    assert chosen == [1, 3, 4] and torch.allclose(s, torch.sigmoid(z))


def test_plain_expert_weight_is_on_the_input():
    g = torch.Generator().manual_seed(5)
    W = {"x.router": torch.randn(3, 6, generator=g).double()}
    for e in range(3):
        W.update({f"x.e{e}.gate": torch.randn(4, 6, generator=g).double(), f"x.e{e}.up": torch.randn(4, 6, generator=g).double(),
                  f"x.e{e}.down": torch.randn(6, 4, generator=g).double()})
    h = torch.randn(1, 6, generator=g).double()
    mlp = {"expert": {"ff": 4, "limit": 0.5}, "router": {"experts": 3, "top": 1}}
    chosen, s = plain.route(W["x.router"] @ h[0], 1)
    want = plain.clamped_glu(s[chosen[0]] * h, W, f"x.e{chosen[0]}.", 0.5)
    assert torch.allclose(plain.moe(h, W, "x.", mlp), want)
    assert not torch.allclose(want, s[chosen[0]] * plain.clamped_glu(h, W, f"x.e{chosen[0]}.", 0.5))


def test_plain_passes_take_the_embedding_in_again_and_their_own_vector():
    spec = du.CONFIGS["all_looped"]
    config, w = spec["config"], du.random_weights(spec["config"], spec["seed"])
    ids = ru.random_ids(5, config["vocab"], 2)
    trace = []
    plain.forward(config, w, ids, trace)
    assert len(trace) == 4
    # the same with the loop unrolled by hand into four layers that share their tensors' values
    flat = copy.deepcopy(config)
    flat.pop("loop")
    one = copy.deepcopy(flat)
    one["layers"] = one["layers"][:1]
    x0 = w["embed"].double()[torch.tensor(ids)] * config["embedding"]["scale"]
    x = x0.clone()
    for t in range(4):
        x = x + (x0 if t else 0) + w["loop.step"].double()[t]
        p, e = "l0.", config["layers"][0]
        W = {k: v.double() for k, v in w.items()}
        a = plain.attention(plain.scalar_norm(x, W[p + "norm1"], 1e-6), W, p + "mix.", e["mixer"], 1e-6)
        x = x + plain.scalar_norm(a, W[p + "norm1b"], 1e-6) * W[p + "ls1"]
        f = plain.moe(plain.scalar_norm(x, W[p + "norm2"], 1e-6), W, p + "mlp.", e["mlp"])
        x = x + plain.scalar_norm(f, W[p + "norm2b"], 1e-6) * W[p + "ls2"]
        assert torch.allclose(x, trace[t])
