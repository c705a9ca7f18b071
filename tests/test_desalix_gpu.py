"""Desalix through the engine against the plain implementation.

Replays through bin/trace_run: the same requests whole, with their last tokens one by one, in
portions of changing size down to two tokens, and mixed (up to four live, portions beside single
tokens, few pages and four state slots so that both are used again, freed pages filled with NaN),
in float32 and bfloat16, also from captured CUDA graphs.  "Sharp" variants scale the queries so
that a lost far key of a chunk or a key on the wrong side of a chunk's edge shows.  The stream
after every layer run.  Generation through LLMEngine and ContinuousBatchingEngine.  The kernels
and parts one by one."""
import copy
import math
from types import SimpleNamespace

import pytest
import torch

import desalix_util as du
import plain_desalix as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

LENGTHS = {"mix": [1, 9, 40, 131, 260], "odd": [2, 17, 64, 150], "wide": [3, 33, 97, 230],
           "flat": [1, 23, 24, 25, 70], "all_looped": [1, 2, 45, 100], "long": [4, 299, 340, 705]}
LENGTHS.update({k + suffix: v for k, v in LENGTHS.items() for suffix in ("_one_expert", "_every_expert")})

CLOSE_CALL = 0.02  # difference of router scores below which bfloat16 activations may route a token otherwise


def first_close_call(config, weights, ids):
    """(logits, first position at which the plain router's choice hangs on less than CLOSE_CALL)."""
    plain.ROUTING_MARGINS = []
    try:
        logits = plain.forward(config, weights, ids).float()
        close = [t for t, m in plain.ROUTING_MARGINS if m < CLOSE_CALL]
    finally:
        plain.ROUTING_MARGINS = None
    return logits, (min(close) if close else len(ids))


def replay(name, dtype, tmp_path, cuda_graph=False, sharp=False):
    """float32: every position within 2e-4.  bfloat16: within rounding up to the first position of
    a request at which the plain router's choice is a close call.  From there on the engine may have
    sent a token to another expert: that token gets another addend of the same size (the norm after
    the experts makes it so), and the tokens after it see it through the caches, with chunks of a
    few keys undiluted.  Those positions are held to be finite and of the logits' size only; the
    same configurations with every expert chosen, or with one expert, leave the router no choice
    and are held to the rounding bound everywhere (tests below)."""
    spec = du.CONFIGS[name]
    model_dir = str(tmp_path / "model")
    config, weights = du.make_folder(model_dir, name, sharp=sharp)
    prompts = {f"p{n}": ru.random_ids(n, config["vocab"], 100 + n) for n in LENGTHS[name]}
    trace, peak = ru.build_four_mode_trace(prompts, spec["page_size"])
    got = ru.run_trace(model_dir, dtype, trace, peak, str(tmp_path / "out"), page_size=spec["page_size"],
                       cuda_graph=cuda_graph, max_requests=4)
    refs = {n: first_close_call(config, weights, ids) for n, ids in prompts.items()}
    modes, strict = set(), 0
    for (step, rid, pos), row in got.items():
        mode, pname = rid.split("/")
        modes.add(mode.rstrip("01"))
        ref = refs[pname][0][pos]
        assert torch.isfinite(row).all(), (step, rid, pos)
        err = (row - ref).abs().max().item()
        scale = max(ref.abs().max().item(), 1e-3)
        if dtype == "float32":
            assert err <= 2e-4 * max(scale, 1.0), f"first wrong place: step {step} request {rid} position {pos}: {err}"
        elif pos < refs[pname][1]:
            strict += 1
            assert err <= 0.04 * scale + 0.03, f"first wrong place: step {step} request {rid} position {pos}: {err}"
        else:
            assert err <= 2.0 * scale + 0.5, (step, rid, pos, err)
    assert modes == {"whole", "tail", "portions", "mixed"}
    return strict / max(len(got), 1)


def with_one_expert(name):
    """The configuration with one expert in every mixture (and that one chosen): no routing decision,
    so bfloat16 is held to the strict bound everywhere."""
    spec = copy.deepcopy(du.CONFIGS[name])
    for e in spec["config"]["layers"]:
        if e.get("mlp"):
            e["mlp"]["router"] = {"experts": 1, "top": 1}
    du.CONFIGS[name + "_one_expert"] = spec
    return name + "_one_expert"


@pytest.mark.parametrize("name", sorted(du.CONFIGS))
def test_replay_float32(name, tmp_path):
    replay(name, "float32", tmp_path)


@pytest.mark.parametrize("name", ["mix", "odd", "wide"])
def test_replay_bfloat16(name, tmp_path):
    replay(name, "bfloat16", tmp_path)


def with_every_expert_chosen(name):
    """The configuration with ``top`` equal to the number of experts: scores, weighted inputs, the
    experts' products and their sum all run, and no score decides anything."""
    spec = copy.deepcopy(du.CONFIGS[name])
    for e in spec["config"]["layers"]:
        if e.get("mlp"):
            e["mlp"]["router"]["top"] = e["mlp"]["router"]["experts"]
    du.CONFIGS[name + "_every_expert"] = spec
    return name + "_every_expert"


@pytest.mark.parametrize("name", ["mix", "odd", "wide", "long"])
@pytest.mark.parametrize("variant", [with_one_expert, with_every_expert_chosen])
def test_replay_bfloat16_without_routing_is_within_rounding_everywhere(name, variant, tmp_path):
    assert replay(variant(name), "bfloat16", tmp_path) == 1.0


@pytest.mark.parametrize("name", ["mix", "wide"])
def test_replay_bfloat16_single_token_steps_from_captured_graphs(name, tmp_path):
    replay(name, "bfloat16", tmp_path, cuda_graph=True)


@pytest.mark.parametrize("name", ["mix", "odd", "flat", "all_looped", "long"])
def test_replay_float32_sharp_chunk_edges_and_far_keys(name, tmp_path):
    replay(name, "float32", tmp_path, sharp=True)


# ------------------------------------------------------------------ the stream after every run
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    # bfloat16 generation runs on configurations whose routers have no choice (see ``replay``)
    for name in ("mix", "wide", "odd", with_every_expert_chosen("mix"), with_every_expert_chosen("wide")):
        d = str(tmp_path_factory.mktemp(f"desalix_{name}"))
        out[name] = (d,) + du.make_folder(d, name)
    return out


def load(folder, dtype):
    from dispec_b200 import load_model
    return load_model(folder, dtype, "cuda:0")


@pytest.mark.parametrize("name", ["mix", "odd", "wide"])
def test_stream_after_every_layer_run_float32(folders, name):
    from dispec_b200.engine import ModelRunner, SeqEntry
    from dispec_b200.engine.batch import build_context
    folder, config, weights = folders[name]
    model = load(folder, "float32")
    r = ModelRunner(model, page_size=du.CONFIGS[name]["page_size"], num_pages=16, max_num_seqs=2)
    ids = ru.random_ids(37, config["vocab"], 7)
    r.admit("a")
    r.cache.extend("a", len(ids))
    ctx, _ = build_context([SeqEntry("a", ids, 0, [])], r.cache, r.storage, r.states, r.staging, r.dtype, r.device,
                           model.attention_tile_tokens, r.vocab_size)
    ctx.layer_trace = []
    with torch.inference_mode():
        model.forward(ctx)
    want = []
    plain.forward(config, weights, ids, want)
    assert len(ctx.layer_trace) == len(want) == len(plain.layer_runs(config))
    for i, (got, ref) in enumerate(zip(ctx.layer_trace, want)):
        assert (got.cpu().double() - ref).abs().max() < 1e-4 * max(1.0, ref.abs().max().item()), f"layer run {i}"


# ------------------------------------------------------------------ generation entry points
def assert_greedy(weights, config, prompt, got, dtype):
    """Teacher-forced on the engine's tokens: each equals the plain argmax, or the plain top-2 gap
    there is below what the type can resolve."""
    logits = plain.forward(config, weights, list(prompt) + list(got)).float()
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


def test_long_decoding_float32_past_many_chunks(folders):
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
    """`python -m dispec_b200 generate` on a Desalix folder: greedy tokens equal the plain ones (up
    to the first position whose two best logits are closer than the type resolves); `random` writes
    a folder for the same configuration that `generate` serves too."""
    import json
    import os
    import subprocess
    import sys
    folder = str(tmp_path / "model")
    config, weights = du.make_folder(folder, "flat")
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
    assert {k: tuple(v.shape) for k, v in made_weights.items()} == du.tensor_shapes(config)
    proc = subprocess.run(cmd + ["--model", made], check=True, env=env, cwd=ru.ROOT, capture_output=True, text=True)
    lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
    for ln, prompt in zip(lines, prompts):
        assert_greedy(made_weights, config, prompt, ln["output_ids"], "float32")


# ----------------------------------------------------------------------- kernels one by one
def dev(t, dtype=torch.float32):
    return t.to(device="cuda:0", dtype=dtype).contiguous()


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda:0")


@pytest.mark.parametrize("width", [52, 256, 1000])
def test_stream_update_with_rms_norms_and_a_row_added_to_all(width):
    from dispec_b200.ops import norm32
    g = torch.Generator().manual_seed(width)
    x = torch.randn(7, width, generator=g) * 3 + 1.5
    y, bias = torch.randn(7, width, generator=g), torch.randn(width, generator=g)
    rw, nw = (1 + 0.1 * torch.randn(width, generator=g) for _ in range(2))
    xs = dev(x)
    h = norm32.stream_update(xs, dev(y), rms_weight=dev(rw), rms_eps=1e-6, norm_weight=dev(nw), norm_eps=1e-5,
                             norm_kind="rms", out_dtype=torch.float32)
    want = x.double() + plain.rms(y.double(), 1e-6) * rw.double()
    assert (xs.cpu().double() - want).abs().max() < 1e-5
    assert (h.cpu().double() - plain.rms(want, 1e-5) * nw.double()).abs().max() < 1e-5
    # the start of a pass: another stream's rows and one row for all, then the norm; then the row alone
    h = norm32.stream_update(xs, dev(y), bias=dev(bias), norm_weight=dev(nw), norm_eps=1e-5, norm_kind="rms",
                             out_dtype=torch.bfloat16)
    want = want + y.double() + bias.double()
    assert (xs.cpu().double() - want).abs().max() < 1e-5
    assert (h.float().cpu().double() - plain.rms(want, 1e-5) * nw.double()).abs().max() < 0.03
    assert norm32.stream_update(xs, None, bias=dev(bias)) is None
    assert (xs.cpu().double() - (want + bias.double())).abs().max() < 1e-5


def test_pass_entry_adds_the_embedding_only_after_the_first_pass():
    from dispec_b200.parts.base import WideStream
    from dispec_b200.parts.block import PassEntry
    g = torch.Generator().manual_seed(4)
    x, x0, step = torch.randn(5, 24, generator=g), torch.randn(5, 24, generator=g), torch.randn(3, 24, generator=g)
    gain = 1 + 0.1 * torch.randn(24, generator=g)
    part = PassEntry(24, 3)
    part.load({"step": dev(step)})
    assert part.needs_embedding and not PassEntry(24, 1).needs_embedding
    ctx = SimpleNamespace(dtype=torch.float32)
    want = x.double()
    s = WideStream(dev(x), None)
    for t in range(3):
        h = part.forward(ctx, s, dev(x0), t, then_norm=(dev(gain), 1e-6))
        want = want + (x0.double() if t else 0) + step[t].double()
        assert (s.full.cpu().double() - want).abs().max() < 1e-5
        assert (h.cpu().double() - plain.rms(want, 1e-6) * gain.double()).abs().max() < 1e-5
    assert part.forward(ctx, s, dev(x0), 0) is None
    with pytest.raises(ValueError):
        part.forward(ctx, s, dev(x0), 3)


@pytest.mark.parametrize("E,top", [(6, 2), (9, 4), (4, 1), (40, 8), (3, 3), (1, 1)])
def test_router_kernel_with_sigmoid_scores(E, top):
    from dispec_b200.ops import moe
    g = torch.Generator().manual_seed(E)
    T, W = 37, 29
    h, w = torch.randn(T, W, generator=g), torch.randn(E, W, generator=g)
    ids, wts = moe.route(dev(h), dev(w), 1, 1, top, score="sigmoid")
    for t in range(T):
        want, s = plain.route(w.double() @ h[t].double(), top)
        got = ids[t].tolist()
        assert sorted(got) == sorted(want), t
        assert (wts[t].cpu().double() - s[got]).abs().max() < 1e-6


def test_router_kernel_tells_apart_logits_whose_sigmoids_round_to_one():
    """Logits of 18 to 40 all have a 32-bit sigmoid of exactly 1: the largest logits are chosen all the
    same, not the first experts among the equal scores; very negative ones (scores near 0) likewise."""
    from dispec_b200.ops import moe
    E, W = 7, 16
    w = torch.zeros(E, W)
    h = torch.zeros(3, W)
    h[:, 0] = 1.0
    w[:, 0] = torch.tensor([18.0, 30.0, 22.0, 40.0, 19.0, 35.0, 21.0])
    h[1, 0] = -1.0  # logits -18 ... -40: the largest are experts 0, 4, 6
    h[2, 0] = 0.0   # all logits 0: the first experts win the ties
    ids, wts = moe.route(dev(h), dev(w), 1, 1, 3, score="sigmoid")
    assert sorted(ids[0].tolist()) == [1, 3, 5] and (wts[0] == 1.0).all()
    assert sorted(ids[1].tolist()) == [0, 4, 6] and (wts[1] < 1e-7).all() and (wts[1] > 0).all()
    assert sorted(ids[2].tolist()) == [0, 1, 2] and (wts[2] == 0.5).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,ff,E,top,shared,weight_on", [
    (1, 20, 6, 4, 1, None, "input"), (45, 52, 14, 9, 4, (10, 0.7), "input"), (150, 64, 40, 6, 2, (24, 1.5), "input"),
    (70, 128, 96, 16, 3, None, "input"), (300, 64, 64, 2, 1, (128, 1.0), "input"), (33, 64, 24, 5, 2, None, "output")])
def test_gated_mixture_of_experts_feed_forward(dtype, T, W, ff, E, top, shared, weight_on):
    """The part itself: router, rows sorted by expert on the device, the gated unit in the first
    product's epilogue with the score on the sums, the second product, the sum with the shared
    expert.  More than one tile of rows per expert, experts that nobody chooses, sums on both sides
    of the clamps."""
    from dispec_b200.parts.clamped_glu import ClampedGLU
    from dispec_b200.parts.moe import GatedMoE
    g = torch.Generator().manual_seed(T)
    limit = 0.9
    mat = lambda n, k, f=1.0: (f * torch.randn(n, k, generator=g) / k ** 0.5).bfloat16().float()
    w = {"x.router": 3 * torch.randn(E, W, generator=g) / W ** 0.5}
    units = [(f"e{e}", ff) for e in range(E)] + ([("shared", shared[0])] if shared else [])
    for n, f in units:
        w.update({f"x.{n}.gate": mat(f, W, 2.0), f"x.{n}.up": mat(f, W, 2.0), f"x.{n}.down": mat(W, f)})
    sh = None
    if shared:
        sh = ClampedGLU(W, shared[0], shared[1])
        sh.load({k + ".weight": dev(w[f"x.shared.{k}"], dtype) for k in ("gate", "up", "down")})
    part = GatedMoE(W, ff, E, top, limit, weight_on=weight_on, shared=sh)
    tensors = {"router.weight": dev(w["x.router"])}
    for e in range(E):
        for k in ("gate", "up", "down"):
            tensors[f"experts.{e}.{k}.weight"] = dev(w[f"x.e{e}.{k}"], dtype)
    part.load(tensors)
    h = torch.randn(T, W, generator=g).bfloat16().float()
    got = part.forward(SimpleNamespace(dtype=dtype), dev(h, dtype)).cpu().double()
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    wd = {k: v.double() for k, v in w.items()}
    if weight_on == "input":
        want = plain.moe(h.double(), wd, "x.", mlp)
    else:
        want = torch.zeros(T, W, dtype=torch.float64)
        for t in range(T):
            chosen, s = plain.route(wd["x.router"] @ h[t].double(), top)
            for e in chosen:
                want[t] += s[e] * plain.clamped_glu(h[t].double(), wd, f"x.e{e}.", limit)
    # the clamps did something, on both sides
    gates = h.double() @ wd["x.e0.gate"].T
    assert (gates > limit).any() and (gates < -limit).any()
    tol = 1e-4 if dtype == torch.float32 else 0.03
    assert (got - want).abs().max() < tol * max(1.0, want.abs().max().item())


def _cache(k_pool, v_pool, table, write=True):
    return SimpleNamespace(key_pool=k_pool, value_pool=v_pool, page_table=table, write=write,
                           tensors={"key": k_pool, "value": v_pool})


@pytest.mark.parametrize("pool_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,rot", [(3, 2, 10, 6, 6), (6, 2, 64, 64, 48), (2, 2, 8, 12, 0), (4, 4, 16, 8, 16)])
def test_norm_rotate_and_store_kernel(pool_dtype, H, G, dk, dv, rot):
    """Head norms with their weights before the turn, values normed without a weight and turned over
    all their dimensions; rows with a negative position are skipped and nothing else is touched."""
    from dispec_b200.ops import attention as A
    g = torch.Generator().manual_seed(H * dk)
    page, base, eps = 4, 20.0, 1e-3
    cols = (H + G) * dk + G * dv
    qkv = torch.randn(6, cols, generator=g) * 2
    qw, kw = 1 + 0.3 * torch.randn(dk, generator=g), 1 + 0.3 * torch.randn(dk, generator=g)
    pos = torch.tensor([3, 4, 5, 0, -1, 9], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 1, 1, 1], dtype=torch.int32)
    table = torch.tensor([[2, 0, -1], [1, 3, 4]], dtype=torch.int32)
    inv_freq = (base ** (-torch.arange(0, rot, 2).double() / rot)).float() if rot else None
    v_freq = (base ** (-torch.arange(0, dv, 2).double() / dv)).float()
    k_pool = torch.full((5, G, page, dk), float("nan"), device="cuda:0", dtype=pool_dtype)
    v_pool = torch.full((5, G, page, dv), float("nan"), device="cuda:0", dtype=pool_dtype)
    q = A.qkv_rotate_store(dev(qkv), pos.cuda(), seq.cuda(), _cache(k_pool, v_pool, table.cuda()),
                           dev(inv_freq) if rot else None, rot, H, G, dk, dv, pool_dtype, q_norm=dev(qw), k_norm=dev(kw),
                           norm_eps=eps, v_norm=True, v_inv_freq=dev(v_freq))
    tol = 1e-5 if pool_dtype == torch.float32 else 0.03
    written = 0
    for t in range(6):
        if pos[t] < 0:
            continue
        p1 = pos[t:t + 1]
        want_q = plain.scalar_free_head_norm(qkv[t, :H * dk].double().view(1, H, dk), qw.double(), eps)
        want_k = plain.scalar_free_head_norm(qkv[t, H * dk:(H + G) * dk].double().view(1, G, dk), kw.double(), eps)
        if rot:
            want_q, want_k = plain.turn_halves(want_q, p1, base, rot), plain.turn_halves(want_k, p1, base, rot)
        want_v = plain.turn_halves(plain.rms(qkv[t, (H + G) * dk:].double().view(1, G, dv), eps), p1, base, dv)
        pg, off = int(table[seq[t], pos[t] // page]), int(pos[t] % page)
        assert (q[t].float().cpu().double().view(H, dk) - want_q[0]).abs().max() < tol
        assert (k_pool[pg, :, off].float().cpu().double() - want_k[0]).abs().max() < tol
        assert (v_pool[pg, :, off].float().cpu().double() - want_v[0]).abs().max() < tol
        written += 1
    assert int(torch.isfinite(k_pool[:, 0, :, 0].float()).sum()) == written
    assert int(torch.isfinite(v_pool[:, 0, :, 0].float()).sum()) == written


AIMS = ["first", "border-", "border+", "chunk_first", "chunk_before", "self", "next", None]


def _aimed_requests(H, G, dk, dv, page, size, lens, q_lens, seed, base):
    """Requests on scattered pages (NaN elsewhere) whose last ``q_lens`` tokens are queries, each
    aimed at one stored key by a large score: the first of the request, both sides of a page
    border, the first key of the query's chunk and the one before it (outside), its own position,
    the next one (stored already, invisible), or nothing (the sink takes the weight).  Values are
    stored turned by their positions."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // page) for n in lens)
    k_pool = torch.full((n_pages, G, page, dk), float("nan"))
    v_pool = torch.full((n_pages, G, page, dv), float("nan"))
    out = dict(tables=[], keys=[], vals=[], qs=[], stars=[])
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        need = -(-n // page)
        out["tables"].append([perm.pop() for _ in range(need)] + [-1] * (width - need))
        kk = torch.randn(n, G, dk, generator=g).bfloat16().float()
        vv = torch.randn(n, G, dv, generator=g).bfloat16().float()
        qq = torch.randn(ql, H, dk, generator=g) * 0.05
        star = []
        for i in range(ql):
            p = n - ql + i
            lo = (p // size) * size if size else 0
            a = AIMS[(i + s) % len(AIMS)]
            star.append({"first": 0, "border-": min(page - 1, n - 1), "border+": min(page, n - 1), "chunk_first": lo,
                         "chunk_before": max(lo - 1, 0), "self": p, "next": min(p + 1, n - 1), None: None}[a])
        for j in {j for j in star if j is not None}:
            kk[j] = (kk[j] * 3.0).bfloat16().float()
        for i, j in enumerate(star):
            for h in range(H):
                if j is None:
                    qq[i, h] -= 0.5 * kk[:, h // (H // G)].mean(0)
                else:
                    kj = kk[j, h // (H // G)]
                    qq[i, h] += 40.0 * kj / kj.norm() ** 2
        turned = plain.turn_halves(vv.double(), torch.arange(n), base, dv).float().bfloat16().float() if base else vv
        for j in range(n):
            k_pool[out["tables"][-1][j // page], :, j % page] = kk[j]
            v_pool[out["tables"][-1][j // page], :, j % page] = turned[j]
        out["keys"].append(kk); out["vals"].append(turned); out["qs"].append(qq.bfloat16().float()); out["stars"].append(star)
    out.update(k_pool=k_pool, v_pool=v_pool)
    return out


def _plain_chunk_attention(c, s, n, ql, scale, size, sink, base, dv):
    pos_q, pos_k = torch.arange(n - ql, n), torch.arange(n)
    o = plain.sink_softmax_attention(c["qs"][s].double(), c["keys"][s].double(), c["vals"][s].double(), pos_q, pos_k, scale,
                                     size, sink)
    return plain.turn_halves(o, pos_q, base, dv, sign=-1.0) if base else o


@pytest.mark.parametrize("pool_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page,size,base", [(4, 2, 16, 8, 16, 20, 100.0), (5, 5, 6, 10, 8, 8, 300.0),
                                                      (18, 2, 64, 128, 32, 64, 1e6), (2, 1, 24, 16, 16, 0, 50.0),
                                                      (6, 2, 16, 8, 16, 7, None), (8, 1, 128, 64, 16, 96, 1e4),
                                                      (3, 1, 10, 6, 4, 1, 10.0), (10, 1, 8, 260, 16, 33, 77.0)])
def test_chunked_attention_with_a_learned_sink_sees_exactly_its_chunk(H, G, dk, dv, page, size, base, pool_dtype):
    """The 32-bit kernel: single tokens and a portion of a prompt, every query aimed (see
    ``_aimed_requests``); chunks of one token, shorter than a page, no multiple of it, none; more
    than eight query heads a key head; the result turned back by the query's position."""
    from dispec_b200.ops import attention as A
    lens, q_lens = [3 * page + 5, 200, max(9 * page + 7, 61)], [1, 1, 45]
    c = _aimed_requests(H, G, dk, dv, page, size, lens, q_lens, H * dk, base)
    T = sum(q_lens)
    sink = torch.randn(H, generator=torch.Generator().manual_seed(9)) * 2
    pos = [n - ql + i for n, ql in zip(lens, q_lens) for i in range(ql)]
    seq = [s for s, ql in enumerate(q_lens) for _ in range(ql)]
    freq = dev((base ** (-torch.arange(0, dv, 2).double() / dv)).float()) if base else None
    out = torch.full((T, H * dv), float("nan"), dtype=pool_dtype, device="cuda:0")
    scale = 0.4
    A.paged_attention_generic(dev(torch.cat(c["qs"]).reshape(T, -1), pool_dtype), H * dk, dev(c["k_pool"], pool_dtype),
                              dev(c["v_pool"], pool_dtype), i32(c["tables"]), i32(pos), i32(seq), out, H, G, dk, size, scale,
                              sink=True, chunked=True, sink_values=dev(sink), turn_freq=freq)
    out = out.float().cpu().double().view(T, H, dv)
    assert torch.isfinite(out).all()
    at = 0
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        want = _plain_chunk_attention(c, s, n, ql, scale, size, sink.double(), base, dv)
        err = (out[at:at + ql] - want).abs().amax(dim=(1, 2))
        tol = 2e-4 if pool_dtype == torch.float32 else 0.02
        assert err.max() < tol * max(1.0, want.abs().max().item()), (s, int(err.argmax()), c["stars"][s][int(err.argmax())])
        # the aims do what they are for: an aimed-at key inside the chunk carries the result
        for i, j in enumerate(c["stars"][s]):
            p = n - ql + i
            if j is not None and plain.visible(p, j, size):
                only = plain.turn_halves(c["vals"][s][j:j + 1].double(), torch.tensor([p]), base, dv, sign=-1.0)[0] if base \
                    else c["vals"][s][j].double()
                assert (want[i] - only.repeat_interleave(H // G, 0)).abs().max() < 0.2 * only.abs().max(), (s, i, j)
        at += ql


@pytest.mark.parametrize("H,G,dk,dv,page,size,base", [(4, 2, 16, 16, 16, 20, 100.0), (18, 2, 64, 128, 32, 64, 1e6),
                                                      (8, 1, 128, 64, 16, 100, 1e4), (12, 2, 128, 128, 16, 0, 5e5),
                                                      (6, 2, 32, 16, 8, 7, None), (5, 5, 48, 32, 16, 33, 10.0),
                                                      (6, 2, 64, 64, 16, 48, 250.0), (2, 2, 16, 16, 16, 1, 30.0)])
@pytest.mark.parametrize("splits", [1, 3, 16])
def test_chunked_attention_on_tensor_cores_matches_the_plain_softmax(H, G, dk, dv, page, size, base, splits):
    """The tensor-core kernel on the same aimed step; tiles of a portion cross chunk edges, so rows
    of one tile start at different keys.  With ``splits`` the single tokens' keys are cut into shares
    (more shares than key tiles too) and merged; the sink must count once and the merged result is
    turned back."""
    from dispec_b200.ops import attention as A
    lens, q_lens = [3 * page + 5, 200, max(9 * page + 7, 61)], [1, 1, 45]
    c = _aimed_requests(H, G, dk, dv, page, size, lens, q_lens, H + dk, base)
    group = H // G
    assert A.sink_mma_supported(group, dk, dv)
    tpt = A.sink_tokens_per_tile(group, dk, dv)
    tiles = [(s, a) for s, ql in enumerate(q_lens) for a in range(0, ql, tpt)]
    T = sum(q_lens)
    sink = torch.randn(H, generator=torch.Generator().manual_seed(9)) * 2
    pos = [n - ql + i for n, ql in zip(lens, q_lens) for i in range(ql)]
    freq = dev((base ** (-torch.arange(0, dv, 2).double() / dv)).float()) if base else None
    out = torch.full((T, H * dv), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    scale = 0.4
    A.sink_attention_tiles(dev(torch.cat(c["qs"]).reshape(T, -1), torch.bfloat16), dev(c["k_pool"], torch.bfloat16),
                           dev(c["v_pool"], torch.bfloat16), i32(c["tables"]), i32([0, 1, 2, 2 + q_lens[2]]), i32(lens),
                           i32([s for s, _ in tiles]), i32([a for _, a in tiles]), len(tiles), out, H, G, size, scale, True,
                           num_single=2, splits=splits, chunked=True, sink_values=dev(sink), turn_freq=freq, positions=i32(pos))
    out = out.float().cpu().double().view(T, H, dv)
    assert torch.isfinite(out).all()
    at = 0
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        want = _plain_chunk_attention(c, s, n, ql, scale, size, sink.double(), base, dv)
        err = (out[at:at + ql] - want).abs().amax(dim=(1, 2))
        assert err.max() < 0.03 * max(1.0, want.abs().max().item()), (s, int(err.argmax()), c["stars"][s][int(err.argmax())])
        at += ql
