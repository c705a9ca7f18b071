"""Grouped-query attention over the paged cache: ``gqa_attention`` (keys and values of one
width, plain softmax) and ``sink_attention`` (widths of their own, a window or a chunked mask,
an optional sink in the softmax, optional norms of the heads, values optionally blended with
another layer's or turned by their positions; at the end of this file).

q, k, v = h W^T + b (one fused product, rows ordered q, k, v: puneethgv/DiSpec
dispec/engine/model_runner.py:104-118,131-136); rotation of q and k and the write of k, v
into the pages (:145-148); scores scaled by ``scale`` (default head_dim**-0.5, :72), key b
visible to the query at position p iff b <= p (and b > p - window for a window layer), softmax
and weighted sum in 32-bit (:160-183 and dispec/engine/triton_attn.py:59-95); output
projection without bias (:158,185).
"""
from __future__ import annotations

import math

import torch

from dispec_b200 import ops
from dispec_b200.ops import attention as attn_ops
from dispec_b200.ops import norm32 as norm32_ops
from dispec_b200.cache.manager import CacheTensor
from dispec_b200.parts.base import CacheNeed, Mixer, TensorSpec
from dispec_b200.registry import register_part


@register_part("mixer", "gqa_attention")
class GQAAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool, position_encoding, window: int = 0, scale: float | None = None,
                 out_bias: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.qkv_bias = qkv_bias
        self.out_bias = out_bias
        self.window = window
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        if not self.scale > 0.0:
            raise ValueError(f"the attention scale must be positive, got {self.scale}")
        self.position_encoding = position_encoding
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def tensor_specs(self):
        h, d = self.hidden_size, self.head_dim
        specs = {
            "q_proj.weight": TensorSpec((self.num_heads * d, h)),
            "k_proj.weight": TensorSpec((self.num_kv_heads * d, h)),
            "v_proj.weight": TensorSpec((self.num_kv_heads * d, h)),
            "o_proj.weight": TensorSpec((h, self.num_heads * d)),
        }
        if self.qkv_bias:
            specs["q_proj.bias"] = TensorSpec((self.num_heads * d,))
            specs["k_proj.bias"] = TensorSpec((self.num_kv_heads * d,))
            specs["v_proj.bias"] = TensorSpec((self.num_kv_heads * d,))
        if self.out_bias:
            specs["o_proj.bias"] = TensorSpec((h,))
        return specs

    def load(self, tensors):
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                tensors["v_proj.weight"]], dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"],
                                    tensors["v_proj.bias"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        self.b_o = tensors.get("o_proj.bias")

    def cache_need(self):
        return CacheNeed.key_value(self.num_kv_heads, self.head_dim, self.window)

    def tokens_per_attention_tile(self):
        group = self.num_heads // self.num_kv_heads
        small = attn_ops.tokens_per_tile(group)
        if small and self.head_dim in (64, 128):
            return (small, attn_ops.prefill_tokens_per_tile(group))  # portions of prompts: 128-row tiles
        return small

    adds_residual = True
    takes_deferred_norm = True

    def forward(self, ctx, x, cache, state, residual=None, then_norm=None):
        """``residual``: added by the last product (32-bit sum, rounded once), so that the sum
        comes back.  ``x`` may be a norm still to be applied (``NormedRows``), and ``then_norm``
        the (weight, eps) of the norm that reads the result: then (result, NormedRows) comes back."""
        H, KVH, D = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = ops.linear(x, self.w_qkv, self.b_qkv)
        rot = self.position_encoding.rotation()
        if rot is not None and rot.layout != "halves":
            raise ValueError(f"gqa_attention turns pairs (i, i + rotary_dim/2) only, not the {rot.layout!r} layout")
        if rot is not None and rot.magnitude != 1.0:
            raise ValueError("gqa_attention applies pure rotations only (the encoding has a magnitude)")
        inv_freq, rotary_dim = (rot.inv_freq, rot.rotary_dim) if rot is not None else (None, 0)
        scale = self.scale * self.position_encoding.score_scale()
        # single tokens come first in the batch: when their attention kernel rotates q and k itself and
        # stores the new key and value, the rotation kernel runs on the portions of prompts only
        n_dec = ctx.num_decode_seqs
        fused = None
        if attn_ops.decode_rope_fusable(ctx, H, KVH, D, rotary_dim, qkv.dtype):
            fused = (inv_freq, rotary_dim, cache.write)
        first = n_dec if fused else 0
        if qkv.shape[0] > first:
            ops.rope_kv_store(qkv[first:], ctx.positions[first:], ctx.seq_of_token[first:], cache.page_table,
                              cache.key_pool if cache.write else None,
                              cache.value_pool if cache.write else None,
                              inv_freq, H, KVH, D, rotary_dim, write_kv=cache.write)
        out = torch.empty((qkv.shape[0], H * D), dtype=qkv.dtype, device=qkv.device)
        attn_ops.paged_attention(ctx, qkv, qkv.stride(0), cache, out, H, KVH, D, self.window,
                                 scale, fused_rope=fused)
        return ops.linear(out, self.w_o, self.b_o, residual=residual, out=residual, then_norm=then_norm)


@register_part("mixer", "sink_attention")
class SinkAttention(Mixer):
    """Grouped-query attention whose keys (``key_dim``) and values (``value_dim``) have widths of
    their own:

        q = W_q h, k = W_k h, v = W_v h (no biases); q and k turned by the position encoding;
        s_j = (q . k_j) * scale over the keys j the window lets position p see (p - window < j <= p;
        window 0: every j <= p);
        sink:     weights exp(s_j) / (1 + sum_j exp(s_j))   (one more key of score 0 and no value)
        no sink:  the plain softmax;
        output projection W_o on the concatenated heads.

    ``value_mix``: None, or a pair (role, key).  The mixer with role "source" publishes its values
    of the step's tokens under ``key``; one with role "blend" replaces its own by
    (1 - m) v + m v_source, m being its tensor ``value_mix`` (a scalar), before they are cached and
    used.  A source owns the tensor too (unused), so that checkpoints list it for every such layer.

    ``mask``: "window" (above) or "chunk": position p sees the keys j <= p of its own chunk,
    floor(j / window) = floor(p / window), chunks counted from position 0 of the sequence.
    ``sink``: True (above), False, or "learned": the extra key's score is the head's number z_h
    (tensor ``sink`` [H], unscaled): weights exp(s_j) / (exp(z_h) + sum_j exp(s_j)).
    ``head_norm``: every query and key head is divided by its root mean square (``norm_eps`` inside
    the root) and multiplied by ``q.norm.weight`` / ``k.norm.weight`` ([key_dim], one for all heads)
    before it is turned.  ``value_norm``: every value head is divided by its root mean square (no
    weight).  ``value_theta``: the value of position j is cached turned, pair (m, m + value_dim/2)
    by the angle j * value_theta^(-2m / value_dim), after its norm; every head's result at position
    p is turned back by -p times the same angles, so that a value enters the sum turned by p - j.
    Scores, softmax, angles, norms and the blend are 32-bit; the projections return 32-bit rows,
    which are rounded once, after norm, rotation and blend, when they enter the cache."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, position_encoding, window: int = 0, sink=True, value_mix=None,
                 mask: str = "window", head_norm: bool = False, value_norm: bool = False, norm_eps: float = 0.0,
                 value_theta: float | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if not float(scale) > 0.0:
            raise ValueError(f"the attention scale must be positive, got {scale}")
        if value_mix is not None and (len(value_mix) != 2 or value_mix[0] not in ("source", "blend")):
            raise ValueError(f"value_mix must be None or ('source' | 'blend', key), got {value_mix!r}")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        if sink not in (True, False, "learned"):
            raise ValueError(f"sink must be True, False or 'learned', got {sink!r}")
        if mask not in ("window", "chunk"):
            raise ValueError(f"mask must be 'window' or 'chunk', got {mask!r}")
        if value_theta is not None and (value_dim % 2 or not float(value_theta) > 0):
            raise ValueError(f"values of width {value_dim} cannot be turned with base {value_theta}")
        if value_mix is not None and value_norm:
            raise ValueError("sink_attention: values are blended or normed, not both")
        self.scale, self.window, self.sink = float(scale), int(window), sink
        self.mask, self.head_norm, self.value_norm = mask, bool(head_norm), bool(value_norm)
        self.norm_eps = float(norm_eps)
        self.value_theta = float(value_theta) if value_theta is not None else None
        self.position_encoding = position_encoding
        self.value_mix = tuple(value_mix) if value_mix is not None else None
        self.w_qkv = self.w_o = self.blend = self.q_norm = self.k_norm = self.sink_values = self.value_freq = None

    def tensor_specs(self):
        h, H, G, dk, dv = self.hidden_size, self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        specs = {"q.weight": TensorSpec((H * dk, h)), "k.weight": TensorSpec((G * dk, h)),
                 "v.weight": TensorSpec((G * dv, h)), "o.weight": TensorSpec((h, H * dv))}
        if self.value_mix is not None:
            specs["value_mix"] = TensorSpec((), dtype="float32")
        if self.head_norm:
            specs["q.norm.weight"] = TensorSpec((dk,), dtype="float32", init="one_plus_normal")
            specs["k.norm.weight"] = TensorSpec((dk,), dtype="float32", init="one_plus_normal")
        if self.sink == "learned":
            specs["sink"] = TensorSpec((H,), dtype="float32")
        return specs

    def load(self, tensors):
        self.w_qkv = torch.cat([tensors["q.weight"], tensors["k.weight"], tensors["v.weight"]], dim=0).contiguous()
        self.w_o = tensors["o.weight"]
        self.blend = tensors.get("value_mix")
        self.q_norm, self.k_norm = tensors.get("q.norm.weight"), tensors.get("k.norm.weight")
        self.sink_values = tensors.get("sink")

    def prepare(self, device):
        if self.value_theta is not None:  # the nearest float32 to theta^(-2m / value_dim)
            exponent = torch.arange(0, self.value_dim, 2, dtype=torch.float64) / self.value_dim
            self.value_freq = (1.0 / (self.value_theta ** exponent)).to(torch.float32).to(device)

    def cache_need(self):
        # a chunk's keys all lie within the last `window` positions: pages behind them are given back
        return CacheNeed((CacheTensor("key", self.num_kv_heads, self.key_dim),
                          CacheTensor("value", self.num_kv_heads, self.value_dim)), self.window)

    def tokens_per_attention_tile(self):
        return attn_ops.sink_tokens_per_tile(self.num_heads // self.num_kv_heads, self.key_dim, self.value_dim)

    def forward(self, ctx, x, cache, state):
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        qkv = ops.linear(x, self.w_qkv, out_dtype=torch.float32)
        rot = self.position_encoding.rotation()
        if rot is not None and rot.layout != "halves":
            raise ValueError(f"sink_attention turns pairs (i, i + rotary_dim/2) only, not the {rot.layout!r} layout")
        if rot is not None and rot.magnitude != 1.0:
            raise ValueError("sink_attention applies pure rotations only (the encoding has a magnitude)")
        inv_freq, rotary_dim = (rot.inv_freq, rot.rotary_dim) if rot is not None else (None, 0)
        v_other = None
        if self.value_mix is not None:
            role, key = self.value_mix
            if role == "source":
                ctx.scratch[("value_mix", key)] = qkv[:, (H + G) * dk:]
            else:
                v_other = ctx.scratch.get(("value_mix", key))
                if v_other is None:
                    raise ValueError(f"sink_attention: no layer published the values {key!r} before this one")
        q = attn_ops.qkv_rotate_store(qkv, ctx.positions, ctx.seq_of_token, cache, inv_freq, rotary_dim, H, G, dk, dv,
                                      ctx.dtype, v_other=v_other, blend=self.blend, q_norm=self.q_norm,
                                      k_norm=self.k_norm, norm_eps=self.norm_eps, v_norm=self.value_norm,
                                      v_inv_freq=self.value_freq)
        out = torch.empty((q.shape[0], H * dv), dtype=q.dtype, device=q.device)
        attn_ops.sink_paged_attention(ctx, q, cache, out, H, G, dk, dv, self.window,
                                      self.scale * self.position_encoding.score_scale(), bool(self.sink),
                                      chunked=self.mask == "chunk", sink_values=self.sink_values,
                                      turn_freq=self.value_freq)
        return ops.linear(out, self.w_o, out_dtype=torch.float32)


@register_part("mixer", "differential_attention")
class DifferentialAttention(Mixer):
    """Grouped-query attention with two softmax maps per head over the same values:

        q = W_q h: per head two parts (map 1, map 2) of ``key_dim`` values; k = W_k h likewise per
        key/value head; v = W_v h.  No biases.  With ``head_norm`` every part of q and k is divided
        by its root mean square (``norm_eps`` inside the root) and multiplied by ``q.norm.weight`` /
        ``k.norm.weight`` ([key_dim], one for all heads and maps); then turned by the position
        encoding, if it turns anything.  ``q_temp`` = (coef, every): q at position p is multiplied by
        1 + coef * ln(floor((p + 1) / every) + 1).
        a_m = softmax over the visible keys of (q_m . k_m) * scale, times v        (m = 1, 2)
        o = a_1 - lambda a_2,  lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff  (one number for the layer)
        o <- o / sqrt(mean(o^2) + norm_eps) * (1 - diff) per head; with ``head_gate`` times
        sigmoid(W_g h)_head, one number per head; output W_o on the concatenated heads.

    The two parts of a key head are cached side by side as one key of width 2 * key_dim, and the
    queries of the two maps are rows that are zero outside their own part (``qkv_rotate_store`` with
    two maps): one attention with 2 H query heads over G key/value heads gives both maps, and each
    key and value row is read once for both.  Keys visible to position p: j <= p, with ``window`` W > 0
    those with p - W < j.  Scores, softmax, norms, the temperature and the combination are 32-bit."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, diff: float, norm_eps: float, position_encoding, window: int = 0,
                 head_norm: bool = True, q_temp: tuple | None = None, head_gate: bool = True):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if not float(scale) > 0.0:
            raise ValueError(f"the attention scale must be positive, got {scale}")
        if q_temp is not None and (len(q_temp) != 2 or int(q_temp[1]) < 1):
            raise ValueError(f"q_temp must be None or (coef, every >= 1), got {q_temp!r}")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale, self.diff, self.norm_eps, self.window = float(scale), float(diff), float(norm_eps), int(window)
        self.head_norm, self.head_gate = bool(head_norm), bool(head_gate)
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp is not None else None
        self.position_encoding = position_encoding
        self.w_in = self.w_o = self.q_norm = self.k_norm = None
        self.lam = 0.0

    def tensor_specs(self):
        h, H, G, dk, dv = self.hidden_size, self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        specs = {"q.weight": TensorSpec((H * 2 * dk, h)), "k.weight": TensorSpec((G * 2 * dk, h)),
                 "v.weight": TensorSpec((G * dv, h)), "o.weight": TensorSpec((h, H * dv))}
        for n in ("lq1", "lk1", "lq2", "lk2"):
            specs[n] = TensorSpec((dk,), dtype="float32")
        if self.head_norm:
            specs["q.norm.weight"] = TensorSpec((dk,), dtype="float32", init="one_plus_normal")
            specs["k.norm.weight"] = TensorSpec((dk,), dtype="float32", init="one_plus_normal")
        if self.head_gate:
            specs["g.weight"] = TensorSpec((H, h))
        return specs

    def load(self, tensors):
        rows = [tensors["q.weight"], tensors["k.weight"], tensors["v.weight"]]
        if self.head_gate:  # the gates' rows ride in the input product
            rows.append(tensors["g.weight"])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors["o.weight"]
        self.q_norm, self.k_norm = tensors.get("q.norm.weight"), tensors.get("k.norm.weight")
        dot = lambda a, b: float((tensors[a].double() * tensors[b].double()).sum())
        self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + self.diff

    def cache_need(self):
        return CacheNeed((CacheTensor("key", self.num_kv_heads, 2 * self.key_dim),
                          CacheTensor("value", self.num_kv_heads, self.value_dim)), self.window)

    def tokens_per_attention_tile(self):
        return attn_ops.sink_tokens_per_tile(2 * self.num_heads // self.num_kv_heads, 2 * self.key_dim, self.value_dim)

    def forward(self, ctx, x, cache, state):
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        z = ops.linear(x, self.w_in, out_dtype=torch.float32)  # [q parts | k parts | v | gates]
        n_qkv = (H + G) * 2 * dk + G * dv
        rot = self.position_encoding.rotation()
        if rot is not None and (rot.layout != "halves" or rot.magnitude != 1.0):
            raise ValueError("differential_attention turns pairs (i, i + rotary_dim/2) by pure rotations only")
        inv_freq, rotary_dim = (rot.inv_freq, rot.rotary_dim) if rot is not None else (None, 0)
        q = attn_ops.qkv_rotate_store(z[:, :n_qkv], ctx.positions, ctx.seq_of_token, cache, inv_freq, rotary_dim, H, G,
                                      dk, dv, ctx.dtype, q_norm=self.q_norm, k_norm=self.k_norm, norm_eps=self.norm_eps,
                                      maps=2, q_temp=self.q_temp)
        # the maps stay 32-bit: their difference is divided by its own root mean square, which would
        # magnify a rounding of the two
        maps = torch.empty((q.shape[0], 2 * H * dv), dtype=torch.float32, device=q.device)
        attn_ops.sink_paged_attention(ctx, q, cache, maps, 2 * H, G, 2 * dk, dv, self.window,
                                      self.scale * self.position_encoding.score_scale(), False)
        heads = norm32_ops.diff_heads(maps, H, self.lam, 1.0 - self.diff, self.norm_eps, ctx.dtype,
                                      gate=z[:, n_qkv:] if self.head_gate else None)
        return ops.linear(heads, self.w_o, out_dtype=torch.float32)
