"""Milivik through the engine against the plain implementation.

Replays through bin/trace_run: the same requests whole, with their last tokens one by one, in
portions of changing size down to two tokens, and mixed (up to four live, portions beside single
tokens, few pages and four state slots so that both are used again, freed pages filled with NaN),
in float32 and bfloat16, also from captured CUDA graphs.  "Sharp" variants scale the queries so
that a lost far key or a key on the wrong side of a window's edge shows.  The stream after every
layer.  Generation through LLMEngine, ContinuousBatchingEngine and the command line.  The kernels
and parts one by one, with queries aimed at single keys."""
import copy
import math
from types import SimpleNamespace

import pytest
import torch

import milivik_util as mu
import plain_milivik as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

LENGTHS = {"mix": [1, 9, 40, 131, 260], "odd": [2, 17, 64, 150], "wide": [3, 33, 97, 230], "long": [4, 299, 340, 705]}
LENGTHS.update({k + suffix: v for k, v in LENGTHS.items() for suffix in ("_one_expert", "_every_expert")})

# difference of router scores (or of groups' sums) below which the engine's arithmetic may route a token otherwise
CLOSE_CALL = {"bfloat16": 0.02, "float32": 3e-6}


def first_close_call(config, weights, ids, dtype):
    """(logits, first position at which the plain router's choice hangs on less than CLOSE_CALL)."""
    plain.ROUTING_MARGINS = []
    try:
        logits = plain.forward(config, weights, ids)[0].float()
        close = [t for t, m in plain.ROUTING_MARGINS if m < CLOSE_CALL[dtype]]
    finally:
        plain.ROUTING_MARGINS = None
    return logits, (min(close) if close else len(ids))


def replay(name, dtype, tmp_path, cuda_graph=False, sharp=False):
    """float32: every position within 2e-4 (sharp weights, whose softmax magnifies the rounding of a
    score: 1.5e-3).  bfloat16: within rounding.  Both up to the first position of a
    request at which the plain router's choice (of groups or of experts) is a close call.  From there
    on the engine may have sent a token to another expert: that token gets another addend of the same
    size (the norm after the experts makes it so), and the tokens after it see it through the caches.
    Those positions are held to be finite and of the logits' size only; the same configurations with
    every expert chosen, or with one expert, leave the router no choice and are held to the rounding
    bound everywhere (tests below)."""
    spec = mu.CONFIGS[name]
    model_dir = str(tmp_path / "model")
    config, weights = mu.make_folder(model_dir, name, sharp=sharp)
    prompts = {f"p{n}": ru.random_ids(n, config["vocab"], 100 + n) for n in LENGTHS[name]}
    trace, peak = ru.build_four_mode_trace(prompts, spec["page_size"])
    got = ru.run_trace(model_dir, dtype, trace, peak, str(tmp_path / "out"), page_size=spec["page_size"],
                       cuda_graph=cuda_graph, max_requests=4)
    refs = {n: first_close_call(config, weights, ids, dtype) for n, ids in prompts.items()}
    modes, strict = set(), 0
    for (step, rid, pos), row in got.items():
        mode, pname = rid.split("/")
        modes.add(mode.rstrip("01"))
        ref = refs[pname][0][pos]
        assert torch.isfinite(row).all(), (step, rid, pos)
        err = (row - ref).abs().max().item()
        scale = max(ref.abs().max().item(), 1e-3)
        if pos < refs[pname][1]:
            strict += 1
            # (bfloat16: every sublayer's result is divided by its own root mean square, which turns the
            # relative rounding of a small result into an absolute one)
            bound = (1.5e-3 if sharp else 2e-4) * max(scale, 1.0) if dtype == "float32" else 0.06 * scale + 0.03
            assert err <= bound, f"first wrong place: step {step} request {rid} position {pos}: {err}"
        else:
            assert err <= 2.0 * scale + 0.5, (step, rid, pos, err)
    assert modes == {"whole", "tail", "portions", "mixed"}
    assert dtype != "float32" or strict >= 0.5 * len(got)  # in 32-bit, close calls are the exception
    return strict / max(len(got), 1)


def with_one_expert(name):
    """The configuration with one expert in every mixture (and that one chosen): no routing decision,
    so bfloat16 is held to the strict bound everywhere."""
    spec = copy.deepcopy(mu.CONFIGS[name])
    for e in spec["config"]["layers"]:
        if e.get("mlp") and e["mlp"]["kind"] == "moe":
            e["mlp"]["router"] = {"experts": 1, "top": 1, "scale": e["mlp"]["router"].get("scale", 1.0)}
    mu.CONFIGS[name + "_one_expert"] = spec
    return name + "_one_expert"


def with_every_expert_chosen(name):
    """Every group stays open and ``top`` equals the number of experts: scores, group sums, weights,
    the experts' products and their sum all run, and no score decides anything."""
    spec = copy.deepcopy(mu.CONFIGS[name])
    for e in spec["config"]["layers"]:
        if e.get("mlp") and e["mlp"]["kind"] == "moe":
            r = e["mlp"]["router"]
            r["top"] = r["experts"]
            if r.get("groups"):
                r["groups"]["keep"] = r["groups"]["count"]
    mu.CONFIGS[name + "_every_expert"] = spec
    return name + "_every_expert"


@pytest.mark.parametrize("name", sorted(mu.CONFIGS))
def test_replay_float32(name, tmp_path):
    replay(name, "float32", tmp_path)


@pytest.mark.parametrize("name", ["mix", "odd", "wide"])
def test_replay_bfloat16(name, tmp_path):
    replay(name, "bfloat16", tmp_path)


@pytest.mark.parametrize("name", ["mix", "odd", "wide", "long"])
@pytest.mark.parametrize("variant", [with_one_expert, with_every_expert_chosen])
def test_replay_bfloat16_without_routing_is_within_rounding_everywhere(name, variant, tmp_path):
    assert replay(variant(name), "bfloat16", tmp_path) == 1.0


@pytest.mark.parametrize("name", ["mix", "wide"])
def test_replay_bfloat16_single_token_steps_from_captured_graphs(name, tmp_path):
    replay(name, "bfloat16", tmp_path, cuda_graph=True)


@pytest.mark.parametrize("name", ["mix", "odd", "long"])
def test_replay_float32_sharp_window_edges_and_far_keys(name, tmp_path):
    replay(name, "float32", tmp_path, sharp=True)


# ------------------------------------------------------------------ the stream after every layer
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    # bfloat16 generation runs on configurations whose routers have no choice (see ``replay``)
    for name in ("mix", "wide", "odd", with_every_expert_chosen("mix"), with_every_expert_chosen("wide")):
        d = str(tmp_path_factory.mktemp(f"milivik_{name}"))
        out[name] = (d,) + mu.make_folder(d, name)
    return out


def load(folder, dtype):
    from dispec_b200 import load_model
    return load_model(folder, dtype, "cuda:0")


@pytest.mark.parametrize("name", ["mix", "odd", "wide"])
def test_stream_after_every_layer_float32(folders, name):
    from dispec_b200.engine import ModelRunner, SeqEntry
    from dispec_b200.engine.batch import build_context
    folder, config, weights = folders[name]
    model = load(folder, "float32")
    r = ModelRunner(model, page_size=mu.CONFIGS[name]["page_size"], num_pages=16, max_num_seqs=2)
    ids = ru.random_ids(37, config["vocab"], 7)
    r.admit("a")
    r.cache.extend("a", len(ids))
    ctx, _ = build_context([SeqEntry("a", ids, 0, [])], r.cache, r.storage, r.states, r.staging, r.dtype, r.device,
                           model.attention_tile_tokens, r.vocab_size)
    ctx.layer_trace = []
    with torch.inference_mode():
        model.forward(ctx)
    want = []
    plain.forward(config, weights, ids, layer_trace=want)
    assert len(ctx.layer_trace) == len(want) == len(config["layers"])
    for i, (got, ref) in enumerate(zip(ctx.layer_trace, want)):
        assert (got.cpu().double() - ref).abs().max() < 1e-4 * max(1.0, ref.abs().max().item()), f"layer {i}"


# ------------------------------------------------------------------ generation entry points
def assert_greedy(weights, config, prompt, got, dtype):
    """Teacher-forced on the engine's tokens: each equals the plain argmax, or the plain top-2 gap
    there is below what the type can resolve."""
    logits = plain.forward(config, weights, list(prompt) + list(got))[0].float()
    for i, tok in enumerate(got):
        row = logits[len(prompt) - 1 + i]
        top2 = torch.topk(row, 2)
        reach = 1e-4 if dtype == "float32" else 2 * (0.03 * row.abs().max().item() + 0.02)
        assert tok == int(top2.indices[0]) or float(top2.values[0] - top2.values[1]) < reach, (i, tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_llm_engine(folders, dtype):
    from dispec_b200 import LLMEngine, SamplingParams
    folder, config, weights = folders["mix" if dtype == "float32" else "mix_every_expert"]
    engine = LLMEngine(load(folder, dtype), num_blocks=32, cuda_graph=dtype == "bfloat16")
    for n in (1, 9, 40):  # the same engine: pages are used again
        prompt = ru.random_ids(n, config["vocab"], 300 + n)
        got = engine.generate(prompt, 10, SamplingParams(temperature=0.0))
        assert len(got) == 10
        assert_greedy(weights, config, prompt, got, dtype)
    cache = engine.runner.cache
    assert all(cache.num_free_pages(g) == 32 for g in range(len(cache.groups)))


def test_long_decoding_float32_past_every_window(folders):
    from dispec_b200 import LLMEngine, SamplingParams
    folder, config, weights = folders["mix"]
    engine = LLMEngine(load(folder, "float32"), num_blocks=32)
    prompt = ru.random_ids(3, config["vocab"], 1)
    got = engine.generate(prompt, 150, SamplingParams())
    assert len(got) == 150
    assert_greedy(weights, config, prompt, got, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_continuous_batching_more_requests_than_slots(folders, dtype):
    """Seven requests through three slots and a small pool: portions of prompts beside decoded
    tokens; slots and pages of finished requests go to waiting ones."""
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams
    folder, config, weights = folders["wide" if dtype == "float32" else "wide_every_expert"]
    engine = ContinuousBatchingEngine(load(folder, dtype), KVConfig(block_size=32), num_blocks=12,
                                      max_batch_tokens=48, chunk_size=20, max_num_seqs=3)
    reqs = []
    for i, n in enumerate([1, 9, 40, 64, 9, 70, 2]):
        prompt = ru.random_ids(n, config["vocab"], 400 + i)
        reqs.append((engine.add_request(prompt, 9, SamplingParams(temperature=0.0)), prompt))
    engine.run_until_done()
    out = engine.collect_outputs()
    for rid, prompt in reqs:
        assert len(out[rid]) == 9
        assert_greedy(weights, config, prompt, out[rid], dtype)
    assert engine.runner.cache.free_slots() == 3


def test_command_line_serves_a_folder_and_a_configuration_with_random_weights(tmp_path):
    """`python -m dispec_b200 generate` on a Milivik folder: greedy tokens equal the plain ones (up
    to the first position whose two best logits are closer than the type resolves); `random` writes
    a folder for the same configuration that `generate` serves too."""
    import json
    import os
    import subprocess
    import sys
    folder = str(tmp_path / "model")
    config, weights = mu.make_folder(folder, "odd")
    env = dict(os.environ, PYTHONPATH=ru.ROOT)
    prompts = [[5, 17, 3, 90], [7, 8, 9, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23]]
    cmd = [sys.executable, "-m", "dispec_b200", "generate", "--dtype", "float32", "--max-new", "8", "--block-size", "8",
           "--num-blocks", "32", "--max-batch-tokens", "16", "--chunk-size", "6"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    proc = subprocess.run(cmd + ["--model", folder], check=True, env=env, cwd=ru.ROOT, capture_output=True, text=True)
    lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert [ln["prompt_tokens"] for ln in lines] == [len(p) for p in prompts]
    for ln, prompt in zip(lines, prompts):
        assert len(ln["output_ids"]) == 8
        assert_greedy(weights, config, prompt, ln["output_ids"], "float32")
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(config))
    made = str(tmp_path / "made")
    subprocess.run([sys.executable, "-m", "dispec_b200", "random", "--config", str(cfg_path), "--out", made, "--seed", "5",
                    "--std", "0.08"], check=True, env=env, cwd=ru.ROOT)
    from safetensors.torch import load_file
    made_weights = {k: v.float() for k, v in load_file(os.path.join(made, "model.safetensors")).items()}
    assert {k: tuple(v.shape) for k, v in made_weights.items()} == plain.tensor_shapes(config)
    proc = subprocess.run(cmd + ["--model", made], check=True, env=env, cwd=ru.ROOT, capture_output=True, text=True)
    lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
    for ln, prompt in zip(lines, prompts):
        assert_greedy(made_weights, config, prompt, ln["output_ids"], "float32")


# ----------------------------------------------------------------------- kernels one by one
def dev(t, dtype=torch.float32):
    return t.to(device="cuda:0", dtype=dtype).contiguous()


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda:0")


@pytest.mark.parametrize("width,copies", [(52, False), (256, True), (1000, True)])
def test_output_norm_block_sums_and_hands_on_a_copy(width, copies):
    """The block with stand-in sublayers: x + N1(f(x)) + N2(g(x + N1(f(x)))), gains stored around zero."""
    from dispec_b200.parts.base import WideStream
    from dispec_b200.parts.block import OutputNormBlock
    from dispec_b200.parts.norms import RMSNorm32
    g = torch.Generator().manual_seed(width)
    x = torch.randn(6, width, generator=g) * 3
    w1, w2 = 0.2 * torch.randn(width, generator=g), 0.2 * torch.randn(width, generator=g)
    dtype = torch.bfloat16 if copies else torch.float32
    seen = []

    class Sub:
        def __init__(self, f):
            self.f = f

        def forward(self, ctx, h, *rest):
            seen.append(h)
            return self.f(h.float())

    norms = []
    for w in (w1, w2):
        n = RMSNorm32(width, 1e-5, unit_offset=True)
        n.load({"weight": dev(w)})
        norms.append(n)
    block = OutputNormBlock(width, Sub(lambda h: h * 0.5 + 1.0), norms[0], Sub(lambda h: torch.tanh(h)), norms[1])
    s = WideStream(dev(x), None)
    ctx = SimpleNamespace(dtype=dtype)
    out, nxt = block.forward(ctx, s, None, None, None, then_norm=block.first_norm_after_product())
    rnd = (lambda t: t.to(dtype).double())
    h0 = rnd(x)
    x1 = x.double() + plain.norm_one_plus(h0 * 0.5 + 1.0, w1.double(), 1e-5)
    x2 = x1 + plain.norm_one_plus(torch.tanh(rnd(x1.float())), w2.double(), 1e-5)
    assert out is s and (s.full.cpu().double() - x2).abs().max() < 1e-4
    assert all(h.dtype == dtype for h in seen)
    if copies:
        assert nxt.dtype == dtype and (nxt.float().cpu().double() - x2).abs().max() < 0.02 * x2.abs().max()
        assert block.forward(ctx, s, nxt, None, None)[1] is None  # the last block keeps nothing pending
    else:
        assert nxt is None and seen[0] is s.full  # the 32-bit path reads the stream's own rows


def test_scaled_logits_head():
    from dispec_b200.parts.embedding import LinearHead
    g = torch.Generator().manual_seed(3)
    w, h = torch.randn(37, 24, generator=g), torch.randn(5, 24, generator=g)
    head = LinearHead(37, 24, scale=0.3)
    head.load({"weight": dev(w)})
    got = head.forward(SimpleNamespace(dtype=torch.float32), dev(h))
    assert (got.cpu().double() - h.double() @ w.double().T * 0.3).abs().max() < 1e-5


@pytest.mark.parametrize("H,G,dk,dv,page", [(4, 2, 16, 8, 4), (5, 5, 6, 10, 8), (8, 2, 64, 128, 16)])
def test_two_map_store_norms_parts_scales_queries_and_lays_keys_side_by_side(H, G, dk, dv, page):
    from dispec_b200.ops import attention as AO
    g = torch.Generator().manual_seed(H * dk)
    pos = torch.tensor([0, 1, 2, 3, 4, 5, 6, 11, -1, 12], dtype=torch.int32)
    T = pos.shape[0]
    n_qkv = (H + G) * 2 * dk + G * dv
    z = torch.randn(T, n_qkv + H, generator=g)  # the gates' columns follow and must not be touched
    qw, kw = torch.rand(dk, generator=g) + 0.5, torch.rand(dk, generator=g) + 0.5
    n_pages = 5
    table = torch.tensor([[3, 0, 4, 1]], dtype=torch.int32)
    k_pool = torch.full((n_pages, G, page, 2 * dk), float("nan"), device="cuda:0")
    v_pool = torch.full((n_pages, G, page, dv), float("nan"), device="cuda:0")
    cache = SimpleNamespace(key_pool=k_pool, value_pool=v_pool, page_table=table.cuda(), write=True)
    zd = dev(z)
    q = AO.qkv_rotate_store(zd[:, :n_qkv], pos.cuda(), torch.zeros(T, dtype=torch.int32, device="cuda:0"), cache, None, 0,
                            H, G, dk, dv, torch.float32, q_norm=dev(qw), k_norm=dev(kw), norm_eps=1e-5, maps=2,
                            q_temp=(0.7, 3))
    q = q.cpu().double().view(T, H, 2, 2, dk)
    zq = z[:, :H * 2 * dk].double().view(T, H, 2, dk)
    zk = z[:, H * 2 * dk:(H + G) * 2 * dk].double().view(T, G, 2, dk)
    zv = z[:, (H + G) * 2 * dk:n_qkv].double().view(T, G, dv)
    temp = plain.query_temperature(pos.clamp(min=0), {"coef": 0.7, "every": 3})
    for t in range(T):
        if pos[t] < 0:
            continue
        want_q = plain.norm_plain(zq[t], qw.double(), 1e-5) * temp[t]
        for m in range(2):
            assert (q[t, :, m, m] - want_q[:, m]).abs().max() < 1e-5
            assert q[t, :, m, 1 - m].abs().max() == 0.0  # zero outside the map's own part
        pg, off = int(table[0, pos[t] // page]), int(pos[t] % page)
        want_k = plain.norm_plain(zk[t], kw.double(), 1e-5).reshape(G, 2 * dk)
        assert (k_pool[pg, :, off].cpu().double() - want_k).abs().max() < 1e-5
        assert (v_pool[pg, :, off].cpu().double() - zv[t]).abs().max() < 1e-6
    assert int(torch.isfinite(k_pool[:, 0, :, 0]).sum()) == int((pos >= 0).sum())


@pytest.mark.parametrize("H,dv,a_dtype", [(3, 10, torch.float32), (8, 128, torch.bfloat16), (1, 40, torch.float32)])
def test_diff_heads_kernel(H, dv, a_dtype):
    from dispec_b200.ops import norm32
    g = torch.Generator().manual_seed(dv)
    T = 9
    a = torch.randn(T, 2 * H * dv, generator=g).to(a_dtype)
    gate = torch.randn(T, H + 2, generator=g)
    lam, diff = 0.83, 0.2
    for use_gate in (True, False):
        got = norm32.diff_heads(a.cuda(), H, lam, 1 - diff, 1e-5, torch.float32,
                                gate=dev(gate)[:, 1:H + 1] if use_gate else None)
        av = a.double().view(T, H, 2, dv)
        want = plain.rms(av[:, :, 0] - lam * av[:, :, 1], 1e-5) * (1 - diff)
        if use_gate:
            want = want * torch.sigmoid(gate[:, 1:H + 1].double())[:, :, None]
        assert (got.cpu().double().view(T, H, dv) - want).abs().max() < 1e-5


@pytest.mark.parametrize("cols,gates", [(24, 24), (24, 3), (130, 1)])
def test_sigmoid_gate_kernel_per_element_and_per_head(cols, gates):
    from dispec_b200.ops import norm32
    g = torch.Generator().manual_seed(cols + gates)
    x, gate = torch.randn(7, cols, generator=g), torch.randn(7, gates + 5, generator=g)
    got = norm32.sigmoid_gate(dev(x, torch.bfloat16), dev(gate)[:, 5:], torch.float32)
    want = x.bfloat16().double() * torch.sigmoid(gate[:, 5:].double()).repeat_interleave(cols // gates, dim=1)
    assert (got.cpu().double() - want).abs().max() < 1e-6


@pytest.mark.parametrize("E,top,groups,keep", [(6, 3, 3, 2), (9, 2, 3, 1), (16, 4, 4, 2), (8, 2, 2, 1), (4, 4, 1, 1),
                                               (5, 2, 5, 3), (40, 8, 8, 4), (1, 1, 1, 1)])
def test_router_kernel_with_group_sums_normalised_weights_and_a_gate_row(E, top, groups, keep):
    from dispec_b200.ops import moe
    g = torch.Generator().manual_seed(E + top)
    T, W = 41, 29
    h, w = torch.randn(T, W, generator=g), torch.randn(E + 1, W, generator=g)
    ids, wts, gate = moe.route(dev(h), dev(w), groups, keep, top, score="sigmoid", group_score="top2_sum",
                               normalize=True, weight_scale=1.7, extra_rows=1)
    r = {"experts": E, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}
    want_ids, want_w = plain.route(h.double(), {"r.router": w[:E].double()}, "r.", r)
    assert (gate.cpu().double()[:, 0] - torch.sigmoid(h.double() @ w[E].double())).abs().max() < 1e-6
    for t in range(T):
        got = ids[t].tolist()
        assert sorted(got) == sorted(want_ids[t].tolist()), t
        by_id = dict(zip(want_ids[t].tolist(), want_w[t].tolist()))
        assert max(abs(float(wts[t, k]) - by_id[e]) for k, e in enumerate(got)) < 1e-5
        assert abs(float(wts[t].sum()) - 1.7) < 1e-5


def test_router_kernel_tells_apart_groups_whose_sums_round_to_two():
    """Logits of 18 and more have a 32-bit sigmoid of exactly 1: the groups' sums are still ranked as
    exact arithmetic would, and the experts by their logits."""
    from dispec_b200.ops import moe
    w = torch.eye(8)
    h = torch.tensor([[20.0, 21.0, 24.0, 19.0, 22.0, 22.5, 30.0, 18.0]])  # deficits e^-20 + e^-21, e^-24 + e^-19, ...
    ids, wts = moe.route(dev(h), dev(w), 4, 1, 2, score="sigmoid", group_score="top2_sum", normalize=True)
    assert sorted(ids[0].tolist()) == [4, 5]
    ids, _ = moe.route(dev(h), dev(w), 4, 2, 3, score="sigmoid", group_score="top2_sum", normalize=True)
    assert sorted(ids[0].tolist()) == [1, 4, 5]  # groups 2 and 0 stay open; the largest logits among their experts
    assert abs(float(wts.sum()) - 1.0) < 1e-6


def test_router_kernel_ranks_groups_by_two_scores_not_by_the_best():
    from dispec_b200.ops import moe
    w = torch.eye(6)
    h = torch.tensor([[3.0, -9.0, 1.0, 0.9, 0.5, 0.4], [3.0, 2.5, 1.0, 0.9, 4.0, -9.0]])
    ids, _ = moe.route(dev(h), dev(w), 3, 1, 2, score="sigmoid", group_score="top2_sum", normalize=True)
    assert sorted(ids[0].tolist()) == [2, 3] and sorted(ids[1].tolist()) == [0, 1]
    ids, _ = moe.route(dev(h), dev(w), 3, 1, 2, score="sigmoid")  # by the best score: the other answer
    assert sorted(ids[0].tolist()) == [0, 1] and sorted(ids[1].tolist()) == [4, 5]


@pytest.mark.parametrize("dtype,W,ff", [(torch.float32, 52, 14), (torch.bfloat16, 64, 24), (torch.bfloat16, 256, 128)])
def test_mixture_part_with_silu_units_and_a_gated_shared_unit(dtype, W, ff):
    """The whole feed-forward part on equal inputs against the plain mixture (choices included)."""
    from dispec_b200.parts.moe import GatedMoE
    from dispec_b200.parts.swiglu import SwiGLUFeedForward
    g = torch.Generator().manual_seed(W)
    E, top, T = 6, 3, 45
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top, "scale": 1.3,
                                                           "groups": {"count": 3, "keep": 2}}, "shared": {"ff": ff + 8}}
    P = {}
    for name, shape in [("router", (E, W)), ("shared.sg", (1, W)), ("shared.gate", (ff + 8, W)), ("shared.up", (ff + 8, W)),
                        ("shared.down", (W, ff + 8))] + [(f"e{e}.{n}", (W, ff) if n == "down" else (ff, W))
                                                         for e in range(E) for n in ("gate", "up", "down")]:
        P["m." + name] = (torch.randn(shape, generator=g) * (3.0 if name == "router" else 1.0) / shape[-1] ** 0.5).bfloat16().float()
    h = torch.randn(T, W, generator=g).bfloat16().float()
    shared = SwiGLUFeedForward(W, ff + 8, out_float32=True)
    shared.load({n + "_proj.weight": dev(P["m.shared." + n], dtype) for n in ("gate", "up", "down")})
    part = GatedMoE(W, ff, E, top, None, alpha=1.0, up_shift=0.0, score="sigmoid", weight_on="output", num_groups=3,
                    keep_groups=2, group_score="top2_sum", normalize=True, weight_scale=1.3, shared=shared, shared_gate=True)
    tensors = {"router.weight": dev(P["m.router"]), "shared_gate.weight": dev(P["m.shared.sg"])}
    for e in range(E):
        for n in ("gate", "up", "down"):
            tensors[f"experts.{e}.{n}.weight"] = dev(P[f"m.e{e}.{n}"], dtype)
    part.load(tensors)
    got = part.forward(SimpleNamespace(dtype=dtype), dev(h, dtype)).cpu().double()
    want = plain.moe(h.double(), {k: v.double() for k, v in P.items()}, "m.", mlp)
    tol = 1e-4 if dtype == torch.float32 else 0.03
    assert (got - want).abs().max() < tol * max(1.0, want.abs().max().item())


# ----------------------------------------------------------------------- latent attention kernels
def scattered_pools(lens, page, widths, g, dtype=torch.float32):
    """Rows of random values for requests of the given lengths, laid out in pools of scattered pages
    (NaN everywhere else).  Returns (page tables, per width: per request rows, per width: pool)."""
    n_pages = sum(-(-n // page) for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // page) for n in lens)
    pools = [torch.full((n_pages, 1, page, max(w, 1)), float("nan"))[..., :w] for w in widths]
    tables, rows = [], [[] for _ in widths]
    for n in lens:
        need = -(-n // page)
        tables.append([perm.pop() for _ in range(need)] + [-1] * (width - need))
        for i, w in enumerate(widths):
            r = torch.randn(n, w, generator=g).to(dtype).float()
            rows[i].append(r)
            for j in range(n):
                pools[i][tables[-1][j // page], 0, j % page] = r[j]
    return tables, rows, pools


def release_before(tables, lens, page, window):
    """Page ids of the pages a window has passed for good become -1, as the cache manager leaves them."""
    out = [list(t) for t in tables]
    for t, n in zip(out, lens):
        for p in range(max(0, n - window) // page):
            t[p] = -1
    return out


def latent_reference(qa, q_rot, lat, rk, p, window, scale, freq, mag):
    qr = plain.turn_halves(q_rot.double()[None], torch.tensor([p]), freq, mag)[0] if freq is not None else q_rot.double()
    lo = max(0, p - window + 1) if window else 0
    s = (qa.double() @ lat[lo:p + 1].double().T + qr @ rk[lo:p + 1].double().T) * scale
    w = torch.softmax(s, dim=-1)
    return w @ lat[lo:p + 1].double(), w, lo


@pytest.mark.parametrize("pool_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,r,page,window", [(3, 20, 6, 8, 13), (10, 192, 16, 16, 40), (2, 520, 64, 64, 0), (4, 24, 8, 4, 4)])
def test_latent_attention_kernel_sees_exactly_the_window(H, R, r, page, window, pool_dtype):
    """One key's score stands out by far: the first key inside the window and the one before it, keys
    on both sides of a page border, the query's own position and the one after it (stored already,
    invisible), the sequence's first token.  Pages the window has passed are gone from the table."""
    from dispec_b200.ops import latent as LO
    g = torch.Generator().manual_seed(R + window)
    n = 5 * page + 3
    tables, (lat, rk), (c_pool, r_pool) = scattered_pools([n], page, [R, r], g, pool_dtype)
    lat, rk = lat[0], rk[0]
    p = n - 2
    first = max(0, p - window + 1) if window else 0
    qpos = [p] * 7
    star = [first, max(first - 1, 0), (first // page + 1) * page - 1, (first // page + 1) * page, p, p + 1, 0]
    if window:
        tables = release_before(tables, [p + 1], page, window)
    else:  # the first tokens of a sequence
        qpos, star = qpos + [page, 0], star + [page, 0]
    T = len(qpos)
    slowed = {"dims": r, "base": 50.0, "scaling": {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    freq, mag = plain.yarn_table(slowed)
    qa = torch.randn(T, H, R, generator=g) * 0.05
    q_rot = torch.randn(T, H, r, generator=g) * 0.05
    for t in range(T):
        qa[t] += 6.0 * lat[star[t]] / lat[star[t]].norm() ** 2 * math.sqrt(R)
    qraw = torch.zeros(T, H * (5 + r))
    for a in range(H):
        qraw[:, a * (5 + r) + 5:(a + 1) * (5 + r)] = q_rot[:, a]
    scale = 0.37
    out = LO.latent_attention(dev(qa.reshape(T, -1)), dev(qraw), 5 + r, 5, dev(freq), r, dev(c_pool, pool_dtype),
                              dev(r_pool, pool_dtype), i32(tables).expand(T, -1).contiguous(), i32(qpos),
                              torch.zeros(T, dtype=torch.int32, device="cuda:0"), H, scale, torch.float32,
                              layout="halves", magnitude=mag, window=window)
    out = out.cpu().double().view(T, H, R)
    from dispec_b200.ops import library
    assert library.device_error() == 0  # no page behind the window was looked up
    for t in range(T):
        want, w, lo = latent_reference(qa[t], q_rot[t], lat, rk, qpos[t], window, scale, freq, mag)
        assert (out[t] - want).abs().max() < 2e-4, (t, star[t])
        if lo <= star[t] <= qpos[t]:
            assert w[:, star[t] - lo].min() > 0.5  # the aimed-at key does carry the result
        elif w.shape[1] >= 12:
            assert w.max() < 0.9  # a key outside the window or after the query: nothing stands out


def test_latent_store_kernel_turns_halves_with_a_magnitude_and_norms_the_query_latent():
    from dispec_b200.ops import latent as LO
    g = torch.Generator().manual_seed(2)
    R, r, page, Q = 20, 8, 4, 3
    down = torch.randn(6, Q + R + r + 7, generator=g)  # gate columns follow
    gain = torch.rand(R, generator=g) + 0.5
    pos = torch.tensor([3, 4, 5, 0, -1, 9], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 1, 1, 1], dtype=torch.int32)
    table = torch.tensor([[2, 0, -1], [1, 3, 4]], dtype=torch.int32)
    rot = {"dims": 6, "base": 20.0, "scaling": {"factor": 2.5, "original": 8, "fast": 2.0, "slow": 0.5}}
    freq, mag = plain.yarn_table(rot)
    c_pool = torch.full((5, 1, page, R), float("nan"), device="cuda:0")
    r_pool = torch.full((5, 1, page, r), float("nan"), device="cuda:0")
    q_gain = torch.rand(Q, generator=g) + 0.5
    cq = LO.latent_store(dev(down), Q, Q + R, dev(gain), 1e-6, dev(freq), 6, pos.cuda(), seq.cuda(), table.cuda(),
                         c_pool, r_pool, layout="halves", magnitude=mag, query_latent=(0, Q, dev(q_gain), torch.float32))
    # the query latent's norm comes out of the same launch, for padding rows too
    assert (cq.cpu().double() - plain.norm_plain(down[:, :Q].double(), q_gain.double(), 1e-6)).abs().max() < 1e-5
    for t in range(6):
        if pos[t] < 0:
            continue
        pg, off = int(table[seq[t], pos[t] // page]), int(pos[t] % page)
        c = plain.norm_plain(down[t, Q:Q + R].double(), gain.double(), 1e-6)
        k = plain.turn_halves(down[t, Q + R:Q + R + r].double()[None], pos[t:t + 1], freq, mag)[0]
        assert (c_pool[pg, 0, off].cpu().double() - c).abs().max() < 1e-5
        assert (r_pool[pg, 0, off].cpu().double() - k).abs().max() < 1e-5
        assert (k[6:] - down[t, Q + R + 6:Q + R + r].double()).abs().max() == 0  # dimensions beyond ``dims`` pass


@pytest.mark.parametrize("H,R,r,page,window", [(10, 192, 16, 16, 40), (12, 512, 64, 16, 100), (70, 64, 32, 8, 33),
                                               (4, 128, 32, 16, 32), (6, 64, 16, 16, 300), (8, 128, 32, 32, 0)])
def test_latent_attention_on_tensor_cores_with_a_window(H, R, r, page, window):
    """The tensor-core kernel over a step of two single tokens (keys cut into ranges and merged) and
    a portion of a prompt whose window starts in the middle of key tiles and pages; every query is
    aimed at one key: the first of its window, the one before it, both sides of a page border, its
    own position, the next one (stored, invisible), a far one.  Pages behind the windows are gone."""
    from dispec_b200.ops import latent as LO
    from dispec_b200.ops import library
    g = torch.Generator().manual_seed(H + R)
    lens = [3 * page + 5, 420, 9 * page + 7]
    portion = 45
    tables, (lat, rk), (c_pool, r_pool) = scattered_pools(lens, page, [R, r], g, torch.bfloat16)
    q_lens = [1, 1, portion]
    if window:
        tables = release_before(tables, [n - ql + 1 for n, ql in zip(lens, q_lens)], page, window)
    seq_of, pos = [], []
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        seq_of += [s] * ql
        pos += list(range(n - ql, n))
    T = len(pos)
    star = []
    for t in range(T):
        p, n = pos[t], lens[seq_of[t]]
        first = max(0, p - window + 1) if window else 0
        star.append([first, max(first - 1, 0), (first // page + 1) * page - 1, (first // page + 1) * page, p,
                     min(p + 1, n - 1), first // 2][t % 7])
    rot = {"dims": r, "base": 50.0, "scaling": {"factor": 3.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    freq, mag = plain.yarn_table(rot)
    qa = torch.randn(T, H, R, generator=g) * 0.05
    q_rot = torch.randn(T, H, r, generator=g) * 0.05
    for t in range(T):
        c = lat[seq_of[t]][star[t]]
        qa[t] += 8.0 * c / c.norm() ** 2 * math.sqrt(R)
    qraw = torch.zeros(T, H * (8 + r))
    for a in range(H):
        qraw[:, a * (8 + r) + 8:(a + 1) * (8 + r)] = q_rot[:, a]
    qraw = qraw.bfloat16()
    tpt = LO.mma_tokens_per_tile(H)
    tiles = [(s, a) for s, ql in enumerate(q_lens) for a in range(0, ql, tpt)]
    ctx = SimpleNamespace(attention_tiles={tpt: (i32([s for s, _ in tiles]), i32([a for _, a in tiles]), len(tiles))},
                          q_start=i32([0, 1, 2, 2 + portion]), ctx_len=i32(lens), num_decode_seqs=2, max_ctx_len=max(lens))
    assert LO.mma_supported(R, r, torch.bfloat16)
    scale = 0.21
    out = LO.latent_attention_tiles(ctx, dev(qa.reshape(T, -1)), dev(qraw, torch.bfloat16), 8 + r, 8, dev(freq), r,
                                    dev(c_pool, torch.bfloat16), dev(r_pool, torch.bfloat16), i32(tables), H, scale,
                                    layout="halves", magnitude=mag, window=window)
    out = out.float().cpu().double().view(T, H, R)
    assert torch.isfinite(out).all() and library.device_error() == 0
    for t in range(T):
        s_ = seq_of[t]
        want, w, lo = latent_reference(qa[t], q_rot[t].bfloat16(), lat[s_], rk[s_], pos[t], window, scale, freq, mag)
        assert (out[t] - want).abs().max() < 0.05 * max(1.0, want.abs().max().item()), (t, star[t], pos[t])


def test_head_products_kernel_with_an_output_gate():
    from dispec_b200.ops import latent as LO
    g = torch.Generator().manual_seed(9)
    M, H, N, K = 70, 5, 48, 64
    x = torch.randn(M, H * K, generator=g).bfloat16()
    w = (torch.randn(H, N, K, generator=g) / K ** 0.5).bfloat16()
    gate = torch.randn(M, 7 + H * N, generator=g)
    out = torch.full((M, H * N), float("nan"), dtype=torch.float32, device="cuda:0")
    LO.head_products(x.cuda(), K, w.cuda(), out, N, gate=dev(gate)[:, 7:])
    want = torch.einsum("mhk,hnk->mhn", x.double().view(M, H, K), w.double()).reshape(M, H * N) * torch.sigmoid(gate[:, 7:].double())
    assert (out.cpu().double() - want).abs().max() < 1e-4 * max(1.0, want.abs().max().item())


# ----------------------------------------------------------------------- the two-map attention part
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page,window", [(4, 2, 16, 32, 16, 0), (5, 5, 6, 10, 8, 21), (8, 2, 64, 128, 16, 0),
                                                   (6, 1, 32, 16, 4, 64)])
def test_differential_attention_part_against_the_plain_mixer(H, G, dk, dv, page, window, dtype):
    """The mixer alone through a runner-like context: a long prompt, then portions and single tokens,
    with weights that make the maps sharp (so that a lost far key or a mixed-up map shows)."""
    from dispec_b200.engine.batch import LayerCacheView
    from dispec_b200.ops import attention as AO
    from dispec_b200.parts.attention import DifferentialAttention
    from dispec_b200.parts.rotary import NoPositionEncoding
    g = torch.Generator().manual_seed(H * dk + window)
    W, n = 48, 300
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "diff": 0.35, "scale": 0.8, "q_temp": {"coef": 0.6, "every": 128}}
    shapes = {"q": (H * 2 * dk, W), "k": (G * 2 * dk, W), "v": (G * dv, W), "g": (H, W), "o": (W, H * dv), "q.norm": (dk,),
              "k.norm": (dk,), "lq1": (dk,), "lk1": (dk,), "lq2": (dk,), "lk2": (dk,)}
    P = {}
    for name, shape in shapes.items():
        t = torch.randn(shape, generator=g)
        t = 3.0 + 0.3 * t if name == "q.norm" else 1.0 + 0.2 * t if name == "k.norm" else 0.3 * t if name[0] == "l" else t / shape[-1] ** 0.5
        P["x." + name] = t.bfloat16().float()
    part = DifferentialAttention(W, H, G, dk, dv, m["scale"], m["diff"], 1e-6, NoPositionEncoding(), window=window,
                                 q_temp=(0.6, 128))
    model_t = {n_ + ".weight": dev(P["x." + n_], dtype) for n_ in ("q", "k", "v", "g", "o")}
    model_t.update({n_ + ".weight": dev(P["x." + n_]) for n_ in ("q.norm", "k.norm")})
    model_t.update({n_: dev(P["x." + n_]) for n_ in ("lq1", "lk1", "lq2", "lk2")})
    part.load(model_t)
    assert abs(part.lam - plain.diff_lambda({k: v.double() for k, v in P.items()}, "x.", 0.35)) < 1e-9
    x = torch.randn(n, W, generator=g).bfloat16().float()
    want, _ = plain.diff_attention(x.double(), {k: v.double() for k, v in P.items()}, "x.", m, 1e-6, torch.arange(n),
                                   window=window)
    n_pages = -(-n // page) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = i32([perm[:-(-n // page)]])
    k_pool = torch.full((n_pages, G, page, 2 * dk), float("nan"), dtype=dtype, device="cuda:0")
    v_pool = torch.full((n_pages, G, page, dv), float("nan"), dtype=dtype, device="cuda:0")
    cache = LayerCacheView({"key": k_pool, "value": v_pool}, table, 0, True, page, n_pages, window)
    tpt = part.tokens_per_attention_tile()
    got, start = [], 0
    for stop in (200, 201, 202, 260, 262, 299, 300):  # a long portion, single tokens, portions down to two tokens
        ql = stop - start
        tiles = [(0, a) for a in range(0, ql, tpt)] if tpt else []
        ctx = SimpleNamespace(dtype=dtype, positions=i32(list(range(start, stop))), seq_of_token=i32([0] * ql),
                              q_start=i32([0, ql]), ctx_len=i32([stop]), num_decode_seqs=1 if ql == 1 else 0,
                              max_ctx_len=stop, attention_tiles={tpt: (i32([s for s, _ in tiles]), i32([a for _, a in tiles]),
                                                                       len(tiles))} if tpt else {})
        got.append(part.forward(ctx, dev(x[start:stop], dtype), cache, None).cpu().double())
        start = stop
    got = torch.cat(got)
    tol = 2e-4 if dtype == torch.float32 else 0.06
    assert (got - want).abs().max() < tol * max(1.0, want.abs().max().item())
