"""Tiny Milivik configurations, weights and model folders for the tests.  The list of tensors
comes from the plain implementation (not from the package's builder), the weights are drawn with
torch's generator and written with the package's safetensors writer."""
import copy
import json
import os

import torch

import plain_milivik as plain


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window=None, rot=None, base=10000.0, slowed=None, scale=None,
           mlp=None):
    """``rot``: rotated dimensions of the shared key part (None: no rotation at all); ``slowed`` =
    (factor, original, fast, slow)."""
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"dims": rot, "base": base}
        if slowed:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), slowed))
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def diff(heads, kv_heads, dim, vdim, lam0, q_temp=None, scale=None, mlp=None):
    """The two-map attention (it sees every earlier key: the design gives it no window)."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": lam0,
         "scale": scale if scale is not None else dim ** -0.5}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, scale=1.0, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if groups:
        d["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def model(width, vocab, layers, eps=1e-6, scale=0.7, logit_scale=0.5):
    return {"architecture": "Milivik", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "logit_scale": logit_scale, "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # both mixers and both feed-forwards, windows shorter than a page and no multiple of it, a layer
    # without window / with a partly turned key part / without feed-forward, groups of which some or
    # all stay open, with and without a shared expert
    "mix": dict(config=model(64, 160, [
        latent(4, 16, 8, 8, 24, 40, window=20, rot=8, slowed=(4.0, 64, 16.0, 2.0), mlp=dense(96)),
        diff(4, 2, 16, 8, 0.25, q_temp=(0.4, 16), mlp=moe(6, 3, 24, groups=(3, 2), scale=1.7, shared=40)),
        latent(2, 8, 16, 12, 16, 24, rot=8, base=50.0, mlp=None),
        diff(6, 2, 8, 16, 0.6, mlp=moe(4, 1, 16)),
    ]), seed=41, page_size=16),
    # nothing a multiple of 8, one query head per key head, a mixer in which nothing turns, a
    # temperature that changes every third position, one group kept of three
    "odd": dict(config=model(52, 211, [
        diff(5, 5, 6, 10, 0.1, q_temp=(0.3, 3), scale=0.5, mlp=moe(9, 2, 14, groups=(3, 1), scale=0.8, shared=10)),
        latent(3, 10, 6, 6, 20, 12, window=9, rot=6, base=300.0, slowed=(1.5, 20, 4.0, 1.0), mlp=None),
        latent(5, 6, 4, 10, 12, 20, window=33, mlp=dense(30)),
    ], eps=3e-6, scale=1.5, logit_scale=1.0), seed=42, page_size=8),
    # sizes the tensor-core kernels take: latents of 64 and 128, eighteen heads, a window of exactly two
    # pages, four query heads per key head with values wider than keys, every expert chosen in one layer
    "wide": dict(config=model(256, 384, [
        latent(8, 64, 32, 64, 128, 192, window=64, rot=32, slowed=(8.0, 128, 32.0, 1.0),
               mlp=moe(16, 4, 128, groups=(4, 2), scale=2.5, shared=256)),
        diff(8, 2, 64, 128, 0.35, q_temp=(0.45, 64), mlp=dense(512)),
        latent(18, 32, 16, 32, 64, 64, window=100, rot=16, mlp=moe(8, 2, 64, groups=(4, 1), shared=64)),
        diff(4, 1, 16, 32, 0.5, mlp=moe(4, 4, 32)),
    ], scale=4.0, logit_scale=0.2), seed=43, page_size=32),
    # windows of hundreds of positions (many pages and key tiles; single tokens' keys cut into shares),
    # one of them no multiple of a page, a temperature that first changes far into the sequence
    "long": dict(config=model(128, 200, [
        latent(4, 16, 32, 32, 64, 64, window=300, rot=32, slowed=(2.5, 256, 24.0, 1.0), mlp=dense(128)),
        diff(2, 1, 32, 48, 0.25, q_temp=(0.4, 128), mlp=moe(4, 2, 32, groups=(2, 1), scale=1.5, shared=32)),
        latent(6, 16, 16, 48, 128, 32, window=512, rot=16, mlp=None),
    ]), seed=44, page_size=16),
}


def random_weights(config, seed):
    """Weights as float32 tensors holding bfloat16 values."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in plain.tensor_shapes(config).items():
        last = name.split(".")[-1]
        if last in ("norm1", "norm2") or name == "final.norm":
            t = 0.2 * torch.randn(shape, generator=g)  # gains stored around zero
        elif name.endswith((".q.norm", ".k.norm", ".dq.norm", ".dkv.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.4 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif last == "router":  # the feed-forwards read the stream itself, whose size follows the embedding's scale
            t = 0.5 / float((config.get("embedding") or {}).get("scale", 1.0)) * torch.randn(shape, generator=g) / shape[1] ** 0.5
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16).float()
    return out


def sharpen(config, weights):
    """Makes far keys and the edges of windows matter: queries grow so that every softmax falls on one
    or two of the visible keys (through the gain of the normed query latent, or of the query heads)."""
    out = dict(weights)
    for i, e in enumerate(config["layers"]):
        name = f"l{i}.mix.dq.norm" if e["type"] == "latent_attention" else f"l{i}.mix.q.norm"
        out[name] = (weights[name] * 12.0).to(torch.bfloat16).float()
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
