"""Desalix: a decoder whose layers are listed one by one in config.json, each with an ``attention``
mixer (grouped-query attention over the keys of the query's own chunk of positions, a learned
sink per head in the softmax, RMS norms on query and key heads, partial rotation, and values
that are normed and cached turned by their position, the result turned back by the query's) and
an optional mixture-of-experts feed-forward (experts that are clamped gated units, sigmoid
scores, the score on the expert's input, a shared expert).  Every sublayer has an RMS norm with
one number as gain before and after it, and a scale per channel on its normed result before
the 32-bit residual sum.  A run of layers may be passed over several times with the same
weights (each pass with caches of its own): before a pass after the first the embedding output
is added to the stream again, and before every pass a vector of that pass.

config.json: ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``loop``
(optional: ``start``, ``stop``, ``times``) and ``layers``: a list of {``type``, ``mixer``: {``heads``,
``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (optional), ``rot.dims`` / ``rot.base``
(optional)}, ``mlp``: {``kind``: "moe", ``expert``: {``ff``, ``limit``}, ``router``: {``experts``, ``top``},
``shared``: {``ff``, ``limit``} (optional)} or null}.  Tensors: ``embed``, ``head``, ``final.norm``,
``loop.step`` and, for layer i, ``l<i>.norm1|norm1b|norm2|norm2b`` (single numbers), ``l<i>.ls1|2``,
``l<i>.mix.q|k|v|o``, ``l<i>.mix.q.norm|k.norm``, ``l<i>.mix.sink``, ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.shared.gate|up|down``; matrices are stored [out, in].
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import ClassVar

from dispec_b200.config.model_config import ConfigError, ModelConfig, _require
from dispec_b200.models.spec import LayerCall, ModelSpec
from dispec_b200.parts.base import PartSpec
from dispec_b200.registry import register_architecture

GLU_ALPHA = 1.702  # the design's constant in g * sigmoid(alpha * g)


def _chunk(m: dict) -> int:
    return int((m.get("mask") or {}).get("size") or 0)


def _rot(m: dict):
    """(rotated dimensions of queries and keys, base) or None for a mixer without rotation."""
    rot = m.get("rot")
    if not rot:
        return None
    return int(rot.get("dims") or 0), float(rot["base"])


@dataclass(frozen=True)
class DesalixConfig(ModelConfig):
    architecture: ClassVar[str] = "Desalix"

    vocab_size: int
    hidden_size: int
    embedding_scale: float
    eps: float
    layers: tuple  # of dict, as in config.json (deep copies; never mutated)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0  # 0: no run of layers is repeated and nothing enters the stream between layers
    max_position_embeddings: int = 0  # 0: no limit of the model's own

    @classmethod
    def from_dict(cls, d: dict) -> "DesalixConfig":
        where = cls.architecture
        _require(d, ["vocab", "width", "norm", "layers"], where)
        _require(d["norm"], ["eps"], where + " norm")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(d["layers"]):
            at = f"{where} layers[{i}]"
            _require(e, ["type", "mixer"], at)
            if e["type"] != "attention":
                raise ConfigError(f"{at}: mixer type {e['type']!r} is not implemented (known: attention)")
            m = e["mixer"]
            _require(m, ["heads", "kv_heads", "dim", "vdim", "scale"], at + " mixer")
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{at}: heads={m['heads']} is not a multiple of kv_heads={m['kv_heads']}")
            rot = m.get("rot")
            if rot:
                _require(rot, ["base"], at + " mixer.rot")
                dims, base = _rot(m)
                if dims % 2 or dims > m["dim"] or not base > 0:
                    raise ConfigError(f"{at}: rot.dims={dims} must be even and at most dim={m['dim']}, rot.base positive")
                if m["vdim"] % 2:
                    raise ConfigError(f"{at}: values of an odd size vdim={m['vdim']} cannot be turned")
            if _chunk(m) < 0:
                raise ConfigError(f"{at}: mask.size must not be negative")
            mlp = e.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"{at}: mlp.kind={mlp['kind']!r} is not implemented (known: moe)")
                _require(mlp, ["expert", "router"], at + " mlp")
                _require(mlp["expert"], ["ff", "limit"], at + " mlp.expert")
                _require(mlp["router"], ["experts", "top"], at + " mlp.router")
                if not 0 < mlp["router"]["top"] <= mlp["router"]["experts"]:
                    raise ConfigError(f"{at}: top={mlp['router']['top']} of {mlp['router']['experts']} experts")
                if mlp.get("shared"):
                    _require(mlp["shared"], ["ff", "limit"], at + " mlp.shared")
            layers.append(copy.deepcopy(e))
        loop = d.get("loop") or {}
        start = stop = times = 0
        if loop:
            _require(loop, ["start", "stop", "times"], where + " loop")
            start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"{where}: loop start={start} stop={stop} times={times} does not fit "
                                  f"{len(layers)} layers")
            if start == stop:  # an empty run has no first layer for anything to enter before
                start = stop = times = 0
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   eps=float(d["norm"]["eps"]), layers=tuple(layers), loop_start=start, loop_stop=stop,
                   loop_times=times, max_position_embeddings=int(d.get("max_position_embeddings", 0)))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps},
             "layers": copy.deepcopy(list(self.layers))}
        if self.loop_times:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_position_embeddings:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d

    def flat(self) -> dict:
        out = super().flat()
        out["num_layers"] = len(self.layers)
        return out

    def layer_runs(self) -> list:
        """The order in which the layers run: (layer, t) with t the number of the pass that begins
        at this run, or None."""
        L = len(self.layers)
        if not self.loop_times:
            return [(i, None) for i in range(L)]
        runs = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            runs += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, None) for i in range(self.loop_stop, L)]


def _mixer_spec(cfg: DesalixConfig, m: dict, prefix: str) -> PartSpec:
    rot = _rot(m)
    rotary = PartSpec("position_encoding", "none")
    if rot is not None and rot[0]:
        rotary = PartSpec("position_encoding", "rotary", {"head_dim": m["dim"], "theta": rot[1], "rotary_dim": rot[0],
                                                          "layout": "halves", "exact_table": True})
    tensors = {n + ".weight": prefix + n for n in ("q", "k", "v", "o", "q.norm", "k.norm")}
    tensors["sink"] = prefix + "sink"
    return PartSpec("mixer", "sink_attention",
                    {"hidden_size": cfg.hidden_size, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                     "key_dim": m["dim"], "value_dim": m["vdim"], "scale": m["scale"], "window": _chunk(m),
                     "mask": "chunk", "sink": "learned", "head_norm": True, "value_norm": True, "norm_eps": cfg.eps,
                     "value_theta": rot[1] if rot is not None else None, "position_encoding": rotary}, tensors)


def _glu_names(prefix: str) -> dict:
    return {n + ".weight": prefix + n for n in ("gate", "up", "down")}


def _ffn_spec(cfg: DesalixConfig, mlp: dict, prefix: str) -> PartSpec:
    h, r = cfg.hidden_size, mlp["router"]
    E = int(r["experts"])
    tensors = {"router.weight": prefix + "router"}
    for i in range(E):
        for n in ("gate", "up", "down"):
            tensors[f"experts.{i}.{n}.weight"] = f"{prefix}e{i}.{n}"
    shared = None
    if mlp.get("shared"):
        shared = PartSpec("feed_forward", "clamped_glu",
                          {"hidden_size": h, "intermediate_size": int(mlp["shared"]["ff"]),
                           "limit": float(mlp["shared"]["limit"]), "alpha": GLU_ALPHA}, _glu_names(prefix + "shared."))
    return PartSpec("feed_forward", "glu_moe",
                    {"hidden_size": h, "intermediate_size": int(mlp["expert"]["ff"]), "num_experts": E,
                     "top": int(r["top"]), "limit": float(mlp["expert"]["limit"]), "alpha": GLU_ALPHA,
                     "score": "sigmoid", "weight_on": "input", "shared": shared}, tensors)


def build_desalix(cfg: DesalixConfig) -> ModelSpec:
    h = cfg.hidden_size
    norm = lambda name: PartSpec("norm", "rms_norm_scalar_f32", {"hidden_size": h, "eps": cfg.eps}, {"weight": name})
    blocks = []
    # a checkpoint may carry the stream norms and channel scale of a feed-forward that a layer does
    # not have, and the pass vectors of a run that is empty: they are ignored
    spare = set() if cfg.loop_times else {"loop.step"}
    for i, e in enumerate(cfg.layers):
        p = f"l{i}."
        params = {"hidden_size": h, "mixer_norm": norm(p + "norm1"), "mixer": _mixer_spec(cfg, e["mixer"], p + "mix."),
                  "mixer_out_norm": norm(p + "norm1b")}
        tensors = {"scale1": p + "ls1"}
        if e.get("mlp") is not None:
            params.update(ffn_norm=norm(p + "norm2"), feed_forward=_ffn_spec(cfg, e["mlp"], p + "mlp."),
                          ffn_out_norm=norm(p + "norm2b"))
            tensors["scale2"] = p + "ls2"
        else:
            spare.update({p + "norm2", p + "norm2b", p + "ls2"})
        blocks.append(PartSpec("block", "sandwich_norm", params, tensors))
    # every run of a layer has a cache of its own (its label is its place in the schedule)
    schedule = [LayerCall(layer, None, True, entry) for layer, entry in cfg.layer_runs()]
    pass_entry = None
    if cfg.loop_times:
        pass_entry = PartSpec("stream_input", "pass_entry", {"hidden_size": h, "times": cfg.loop_times, "reinject": True},
                              {"step": "loop.step"})
    return ModelSpec(
        architecture=cfg.architecture,
        embedding=PartSpec("embedding", "scaled_embedding",
                           {"vocab_size": cfg.vocab_size, "hidden_size": h, "scale": cfg.embedding_scale},
                           {"weight": "embed"}),
        layers=blocks, final_norm=norm("final.norm"),
        head=PartSpec("head", "linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": h}, {"weight": "head"}),
        schedule=schedule, pass_entry=pass_entry, vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings,
        optional_tensors=frozenset(spare))


register_architecture(DesalixConfig.architecture, DesalixConfig, build_desalix)
