"""Milivik: a decoder whose layers are listed one by one in config.json, each with a mixer and an
optional feed-forward, a norm on every sublayer's result only (x <- x + N(sublayer(x)), gains
stored around zero), a scaled embedding, and logits from the embedding matrix times a constant.

Mixers: ``latent_attention`` (queries through a normed latent, keys and values as linear maps
of a cached normed latent plus one rotated key part shared by the heads, half-split rotation
with slowed frequencies, a sliding window, an output gate per element) and ``attention``
(grouped-query differential attention: two softmax maps per head over the same values, head
norms on queries and keys, a query temperature that grows with the position, no rotation, a
gate per head).  Feed-forwards: ``dense`` (silu(W_gate h) * (W_up h), then W_down) and ``moe``
(sigmoid scores, groups of experts ranked by the sum of their two best scores, weights divided
by their sum and scaled, a shared expert gated per token).

config.json: ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``logit_scale`` and ``layers``: a list of {``type``, ``mixer``, ``mlp`` or null}.
``latent_attention``: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``q_rank``, ``scale``,
``mask.size`` (optional), ``rot``: {``dims``, ``base``, ``scaling``: {``factor``, ``original``,
``fast``, ``slow``} (optional)} (optional).  ``attention``: ``heads``, ``kv_heads``, ``dim``,
``vdim``, ``scale``, ``diff``, ``q_temp``: {``coef``, ``every``} (optional); it sees every
earlier key.  ``mlp``: {``kind``: "dense", ``ff``} or {``kind``: "moe", ``expert``: {``ff``},
``router``: {``experts``, ``top``, ``scale``, ``groups``: {``count``, ``keep``} (optional)},
``shared``: {``ff``} (optional)}.  Tensors: ``embed``, ``final.norm`` and, for layer i,
``l<i>.norm1|norm2``, ``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o`` or
``l<i>.mix.q|k|v|q.norm|k.norm|lq1|lk1|lq2|lk2|g|o``, ``l<i>.mlp.gate|up|down`` or
``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.shared.gate|up|down|sg``;
matrices are stored [out, in].
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import ClassVar

from dispec_b200.config.model_config import ConfigError, ModelConfig, _require
from dispec_b200.models.spec import ModelSpec
from dispec_b200.parts.base import PartSpec
from dispec_b200.registry import register_architecture

MIXERS = ("latent_attention", "attention")


def _window(m: dict) -> int:
    return int((m.get("mask") or {}).get("size") or 0)


def _check_mixer(kind: str, m: dict, at: str) -> None:
    if kind == "latent_attention":
        _require(m, ["heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale"], at + " mixer")
        rot = m.get("rot")
        if rot:
            _require(rot, ["dims", "base"], at + " mixer.rot")
            if rot["dims"] % 2 or not 0 <= rot["dims"] <= m["rot_dim"] or not rot["base"] > 0:
                raise ConfigError(f"{at}: rot.dims={rot['dims']} must be even and at most rot_dim={m['rot_dim']}, "
                                  f"rot.base positive")
            if rot.get("scaling"):
                _require(rot["scaling"], ["factor", "original", "fast", "slow"], at + " mixer.rot.scaling")
    else:
        _require(m, ["heads", "kv_heads", "dim", "vdim", "scale", "diff"], at + " mixer")
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{at}: heads={m['heads']} is not a multiple of kv_heads={m['kv_heads']}")
        if m.get("q_temp"):
            _require(m["q_temp"], ["coef", "every"], at + " mixer.q_temp")
            if int(m["q_temp"]["every"]) < 1:
                raise ConfigError(f"{at}: q_temp.every must be at least 1")
    if kind == "latent_attention" and _window(m) < 0:
        raise ConfigError(f"{at}: mask.size must not be negative")


def _check_mlp(mlp: dict, at: str) -> None:
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        _require(mlp, ["ff"], at + " mlp")
    elif kind == "moe":
        _require(mlp, ["expert", "router"], at + " mlp")
        _require(mlp["expert"], ["ff"], at + " mlp.expert")
        r = mlp["router"]
        _require(r, ["experts", "top"], at + " mlp.router")
        g = r.get("groups") or {"count": 1, "keep": 1}
        _require(g, ["count", "keep"], at + " mlp.router.groups")
        if r["experts"] % g["count"] or not 0 < g["keep"] <= g["count"]:
            raise ConfigError(f"{at}: {r['experts']} experts in {g['count']} groups of which {g['keep']} stay open")
        if not 0 < r["top"] <= g["keep"] * (r["experts"] // g["count"]):
            raise ConfigError(f"{at}: top={r['top']} experts cannot come from {g['keep']} groups of "
                              f"{r['experts'] // g['count']}")
        if mlp.get("shared"):
            _require(mlp["shared"], ["ff"], at + " mlp.shared")
    else:
        raise ConfigError(f"{at}: mlp.kind={kind!r} is not implemented (known: dense, moe)")


@dataclass(frozen=True)
class MilivikConfig(ModelConfig):
    architecture: ClassVar[str] = "Milivik"

    vocab_size: int
    hidden_size: int
    embedding_scale: float
    logit_scale: float
    eps: float
    layers: tuple  # of dict, as in config.json (deep copies; never mutated)
    max_position_embeddings: int = 0  # 0: no limit of the model's own

    @classmethod
    def from_dict(cls, d: dict) -> "MilivikConfig":
        where = cls.architecture
        _require(d, ["vocab", "width", "norm", "layers"], where)
        _require(d["norm"], ["eps"], where + " norm")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(d["layers"]):
            at = f"{where} layers[{i}]"
            _require(e, ["type", "mixer"], at)
            if e["type"] not in MIXERS:
                raise ConfigError(f"{at}: mixer type {e['type']!r} is not implemented (known: {', '.join(MIXERS)})")
            _check_mixer(e["type"], e["mixer"], at)
            if e.get("mlp") is not None:
                _check_mlp(e["mlp"], at)
            layers.append(copy.deepcopy(e))
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   logit_scale=float(d.get("logit_scale", 1.0)), eps=float(d["norm"]["eps"]), layers=tuple(layers),
                   max_position_embeddings=int(d.get("max_position_embeddings", 0)))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale, "norm": {"eps": self.eps},
             "layers": copy.deepcopy(list(self.layers))}
        if self.max_position_embeddings:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d

    def flat(self) -> dict:
        out = super().flat()
        out["num_layers"] = len(self.layers)
        out["layer_types"] = ",".join(e["type"] for e in self.layers)
        return out


def _mixer_spec(cfg: MilivikConfig, kind: str, m: dict, prefix: str) -> PartSpec:
    h = cfg.hidden_size
    if kind == "latent_attention":
        rot = m.get("rot")
        rotary = PartSpec("position_encoding", "none")
        if rot and rot["dims"]:
            sc = rot.get("scaling")
            slowed = (sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None
            rotary = PartSpec("position_encoding", "rotary",
                              {"head_dim": m["rot_dim"], "theta": rot["base"], "rotary_dim": rot["dims"],
                               "layout": "halves", "exact_table": True, "slowed": slowed})
        names = {f"{n}.weight": prefix + n for n in ("dq", "uq", "dkv", "uk", "uv", "g", "o")}
        names.update({"dq.norm": prefix + "dq.norm", "dkv.norm": prefix + "dkv.norm"})
        return PartSpec("mixer", "latent_attention",
                        {"hidden_size": h, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
                         "vdim": m["vdim"], "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"],
                         "eps": cfg.eps, "position_encoding": rotary, "window": _window(m), "gate": "element"}, names)
    qt = m.get("q_temp")
    names = {n + ".weight": prefix + n for n in ("q", "k", "v", "g", "o", "q.norm", "k.norm")}
    names.update({n: prefix + n for n in ("lq1", "lk1", "lq2", "lk2")})
    return PartSpec("mixer", "differential_attention",
                    {"hidden_size": h, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "key_dim": m["dim"],
                     "value_dim": m["vdim"], "scale": m["scale"], "diff": m["diff"], "norm_eps": cfg.eps,
                     "position_encoding": PartSpec("position_encoding", "none"), "q_temp": (qt["coef"], qt["every"]) if qt else None}, names)


def _glu_spec(h: int, ff: int, prefix: str) -> PartSpec:
    return PartSpec("feed_forward", "swiglu", {"hidden_size": h, "intermediate_size": int(ff), "out_float32": True},
                    {n + "_proj.weight": prefix + n for n in ("gate", "up", "down")})


def _ffn_spec(cfg: MilivikConfig, mlp: dict, prefix: str) -> PartSpec:
    h = cfg.hidden_size
    if mlp.get("kind", "dense") == "dense":
        return _glu_spec(h, mlp["ff"], prefix)
    r = mlp["router"]
    E = int(r["experts"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    tensors = {"router.weight": prefix + "router"}
    for i in range(E):
        for n in ("gate", "up", "down"):
            tensors[f"experts.{i}.{n}.weight"] = f"{prefix}e{i}.{n}"
    shared = None
    if mlp.get("shared"):
        shared = _glu_spec(h, mlp["shared"]["ff"], prefix + "shared.")
        tensors["shared_gate.weight"] = prefix + "shared.sg"
    return PartSpec("feed_forward", "glu_moe",
                    {"hidden_size": h, "intermediate_size": int(mlp["expert"]["ff"]), "num_experts": E,
                     "top": int(r["top"]), "limit": None, "alpha": 1.0, "up_shift": 0.0, "score": "sigmoid",
                     "weight_on": "output", "num_groups": int(groups["count"]), "keep_groups": int(groups["keep"]),
                     "group_score": "top2_sum", "normalize": True, "weight_scale": float(r.get("scale", 1.0)),
                     "shared": shared, "shared_gate": shared is not None}, tensors)


def build_milivik(cfg: MilivikConfig) -> ModelSpec:
    h = cfg.hidden_size
    norm = lambda name: PartSpec("norm", "rms_norm_f32", {"hidden_size": h, "eps": cfg.eps, "unit_offset": True},
                                 {"weight": name})
    blocks, spare = [], set()
    for i, e in enumerate(cfg.layers):
        p = f"l{i}."
        params = {"hidden_size": h, "mixer": _mixer_spec(cfg, e["type"], e["mixer"], p + "mix."),
                  "mixer_out_norm": norm(p + "norm1")}
        if e.get("mlp") is not None:
            params.update(feed_forward=_ffn_spec(cfg, e["mlp"], p + "mlp."), ffn_out_norm=norm(p + "norm2"))
        else:
            spare.add(p + "norm2")  # a checkpoint may carry the norm of a feed-forward the layer does not have
        blocks.append(PartSpec("block", "output_norm", params))
    return ModelSpec(
        architecture=cfg.architecture,
        embedding=PartSpec("embedding", "scaled_embedding",
                           {"vocab_size": cfg.vocab_size, "hidden_size": h, "scale": cfg.embedding_scale},
                           {"weight": "embed"}),
        layers=blocks, final_norm=norm("final.norm"),
        head=PartSpec("head", "linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": h, "scale": cfg.logit_scale},
                      {"weight": "embed"}),
        vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings, optional_tensors=frozenset(spare))


register_architecture(MilivikConfig.architecture, MilivikConfig, build_milivik)
