"""Tiny Desalix configurations, weights and model folders for the tests.  The list of tensors is
derived here from the configuration (not from the package's builder), the weights are drawn with
torch's generator and written with the package's safetensors writer."""
import copy
import json
import os

import torch


def attention(heads, kv_heads, dim, vdim, chunk=None, rot=None, base=10000.0, scale=None, mlp=None, turn=True):
    """``rot``: rotated dimensions of queries and keys (0: none of them, values still turn);
    ``turn`` False: no ``rot`` entry at all (nothing turns)."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if turn:
        m["rot"] = {"base": base, "dims": rot or 0}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def moe(experts, top, ff, limit=1.0, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared[0], "limit": shared[1]}
    return d


def model(width, vocab, layers, loop=None, eps=1e-6, scale=0.7):
    d = {"architecture": "Desalix", "vocab": vocab, "width": width, "embedding": {"scale": scale},
         "norm": {"eps": eps}, "layers": layers}
    if loop:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


CONFIGS = {
    # several key heads, keys and values of unlike sizes, chunks shorter than a page and no multiple
    # of it, a layer without chunks, one without a feed-forward, one or several experts a token,
    # with and without a shared expert; all layers but the first run three times
    "mix": dict(config=model(64, 160, [
        attention(4, 2, 16, 8, chunk=20, rot=8, mlp=moe(6, 2, 24, limit=0.8, shared=(40, 1.5))),
        attention(6, 2, 16, 8, chunk=7, rot=16, base=50.0, mlp=moe(4, 1, 16)),
        attention(2, 2, 8, 12, rot=4, mlp=None),
        attention(2, 1, 24, 8, chunk=40, rot=12, mlp=moe(5, 3, 16, limit=2.0, shared=(16, 0.5))),
    ], loop=(1, 4, 3)), seed=31, page_size=16),
    # nothing a multiple of 8, one query head per key head, the run of repeated layers at the start,
    # passed twice, a chunk of one page, every expert chosen
    "odd": dict(config=model(52, 211, [
        attention(5, 5, 6, 10, chunk=8, rot=4, base=300.0, scale=0.5, mlp=moe(3, 3, 14, limit=1.2)),
        attention(3, 1, 10, 6, chunk=33, rot=10, mlp=None),
        attention(5, 5, 10, 10, chunk=9, rot=0, mlp=moe(9, 4, 14, shared=(10, 1.0))),
    ], loop=(0, 2, 2), eps=3e-6, scale=1.5), seed=32, page_size=8),
    # sizes the tensor-core kernels take: nine query heads per key head, values wider than keys and
    # the other way round, a chunk of exactly two pages, the run of repeated layers at the end, passed once
    "wide": dict(config=model(256, 384, [
        attention(18, 2, 64, 128, chunk=64, rot=32, base=1e6, mlp=moe(16, 3, 128, shared=(256, 1.5))),
        attention(8, 2, 32, 64, chunk=100, rot=16, mlp=moe(8, 2, 64, limit=0.6)),
        attention(8, 1, 128, 64, chunk=48, rot=128, mlp=moe(4, 1, 192, shared=(64, 1.0))),
    ], loop=(1, 3, 1)), seed=33, page_size=32),
    # no run of layers is repeated; a layer in which nothing turns
    "flat": dict(config=model(48, 96, [
        attention(4, 2, 8, 12, chunk=24, rot=8, mlp=moe(4, 2, 32, shared=(24, 1.0))),
        attention(4, 4, 12, 8, chunk=5, turn=False, mlp=moe(2, 1, 16)),
    ]), seed=34, page_size=16),
    # chunks of hundreds of positions (many pages and key tiles; single tokens' keys cut into shares),
    # one of them no multiple of a page, a layer that sees everything; sizes the tensor-core kernels take
    "long": dict(config=model(128, 200, [
        attention(4, 2, 32, 32, chunk=512, rot=16, mlp=moe(4, 2, 32, shared=(32, 1.0))),
        attention(6, 1, 16, 48, chunk=300, rot=16, base=1e5, scale=0.3, mlp=moe(3, 1, 48, limit=2.0)),
        attention(2, 2, 64, 16, rot=32, base=500.0, mlp=None),
    ], loop=(0, 2, 2)), seed=36, page_size=16),
    # every layer runs four times
    "all_looped": dict(config=model(40, 70, [attention(2, 1, 16, 16, chunk=16, rot=16, mlp=moe(3, 1, 24))],
                                    loop=(0, 1, 4)), seed=35, page_size=16),
}


def tensor_shapes(config):
    """name -> shape of every tensor a checkpoint of this configuration holds."""
    W, V = config["width"], config["vocab"]
    shapes = {"embed": (V, W), "head": (V, W), "final.norm": ()}
    loop = config.get("loop")
    if loop:
        shapes["loop.step"] = (loop["times"], W)
    for i, e in enumerate(config["layers"]):
        p, m = f"l{i}.", e["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        shapes.update({p + "norm1": (), p + "norm1b": (), p + "ls1": (W,), p + "mix.q": (H * d, W), p + "mix.k": (G * d, W),
                       p + "mix.v": (G * dv, W), p + "mix.o": (W, H * dv), p + "mix.q.norm": (d,), p + "mix.k.norm": (d,),
                       p + "mix.sink": (H,)})
        mlp = e.get("mlp")
        if mlp is not None:
            shapes.update({p + "norm2": (), p + "norm2b": (), p + "ls2": (W,), p + "mlp.router": (mlp["router"]["experts"], W)})
            units = [(f"e{x}", mlp["expert"]["ff"]) for x in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                units.append(("shared", mlp["shared"]["ff"]))
            for name, ff in units:
                shapes.update({f"{p}mlp.{name}.gate": (ff, W), f"{p}mlp.{name}.up": (ff, W), f"{p}mlp.{name}.down": (W, ff)})
    return shapes


def random_weights(config, seed):
    """Weights as float32 tensors holding bfloat16 values."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.split(".")[-1]
        if last in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm" or name.endswith((".q.norm", ".k.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last in ("ls1", "ls2"):
            t = 0.3 + 0.5 * torch.rand(shape, generator=g)
        elif last == "sink":
            t = torch.randn(shape, generator=g)
        elif name == "loop.step":
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif last == "router":
            t = 3.0 * torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif last in ("gate", "up"):
            t = 2.0 * torch.randn(shape, generator=g) / shape[-1] ** 0.5  # some sums reach the clamps
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16).float()
    return out


def sharpen(config, weights):
    """Makes far keys of a chunk and its edges matter: the weights on normed query heads grow so that
    every softmax falls on one or two keys of the chunk (and beats the sink)."""
    out = dict(weights)
    for i in range(len(config["layers"])):
        out[f"l{i}.mix.q.norm"] = (weights[f"l{i}.mix.q.norm"] * 12.0).to(torch.bfloat16).float()
    return out


def make_folder(folder, name, sharp=False):
    """Writes config.json and model.safetensors (bfloat16); returns (config, weights as float32)."""
    from dispec_b200.weights import write_safetensors

    spec = CONFIGS[name]
    config = copy.deepcopy(spec["config"])
    weights = random_weights(config, spec["seed"])
    if sharp:
        weights = sharpen(config, weights)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return config, weights
