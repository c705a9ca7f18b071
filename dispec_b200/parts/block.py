"""Arrangements of a layer.  The pre-norm residual block:

    x += pending;  h = norm1(x);  a = mixer(h);  x += a;  h = norm2(x);  pending = ffn(h)

(puneethgv/DiSpec dispec/engine/model_runner.py:214-219).  The sum into the residual stream
is fused into the norm that follows it and computed in 32-bit; the block hands the last
feed-forward output on as ``pending`` so that the next block's first norm (or the final norm)
adds it."""
from __future__ import annotations

import torch

from dispec_b200.ops.gemm import NormedRows
from dispec_b200 import ops
from dispec_b200.ops import norm32 as norm32_ops
from dispec_b200.parts.base import Block, Part, TensorSpec, WideStream
from dispec_b200.registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, mixer_norm, mixer, ffn_norm, feed_forward):
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ffn_norm = ffn_norm
        self.feed_forward = feed_forward

    def _takes_residual(self) -> bool:
        return (getattr(self.mixer, "adds_residual", False)
                and getattr(self.feed_forward, "adds_residual", False))

    def _defers_norms(self) -> bool:
        return (self._takes_residual() and hasattr(self.mixer_norm, "deferred")
                and hasattr(self.ffn_norm, "after_product")
                and getattr(self.mixer, "takes_deferred_norm", False)
                and getattr(self.feed_forward, "takes_deferred_norm", False))

    def first_norm_after_product(self):
        """(weight, eps) of this block's first norm if the block takes that norm as ``pending``
        (a ``NormedRows`` of its ``x``) from whoever wrote ``x``; else None."""
        if self._defers_norms() and hasattr(self.mixer_norm, "after_product"):
            return self.mixer_norm.after_product()
        return None

    def forward(self, ctx, x, pending, cache, state, then_norm=None):
        """``then_norm``: (weight, eps) of the norm that reads this block's result first (the next
        block's, offered by its ``first_norm_after_product``); a block that can hands back that
        norm, still to be applied, as ``pending``."""
        if self._defers_norms() and (pending is None or isinstance(pending, NormedRows)):
            # each norm is handed to the product after it, which takes it apart where it can: the
            # product before stores the rows times the gain beside its result, the product after
            # scales its own result rows (see ops.gemm.NormedRows); else the norm kernel runs there
            h = pending if pending is not None else self.mixer_norm.deferred(x)
            x, h = self.mixer.forward(ctx, h, cache, state, residual=x,
                                      then_norm=self.ffn_norm.after_product())
            if then_norm is None:
                return self.feed_forward.forward(ctx, h, residual=x), None
            return self.feed_forward.forward(ctx, h, residual=x, then_norm=then_norm)
        if pending is None and self._takes_residual():
            # the sums into the residual stream happen in the epilogue of the last product of the
            # mixer and of the feed-forward (32-bit sum, rounded once)
            h = self.mixer_norm.forward(ctx, x)
            x = self.mixer.forward(ctx, h, cache, state, residual=x)
            h = self.ffn_norm.forward(ctx, x)
            x = self.feed_forward.forward(ctx, h, residual=x)
            return x, None
        if pending is None:
            h = self.mixer_norm.forward(ctx, x)
        else:
            h = self.mixer_norm.forward_add(ctx, x, pending)
        a = self.mixer.forward(ctx, h, cache, state)
        h = self.ffn_norm.forward_add(ctx, x, a)
        return x, self.feed_forward.forward(ctx, h)


@register_part("block", "post_norm")
class PostNormBlock(Block):
    """Norm after the sum:

        x <- norm1(alpha * x + mixer(x));   x <- norm2(alpha * x + ffn(x))

    The sublayers read x itself (the normalised stream).  The stream is kept in 32-bit floats
    (``WideStream``): sum and norm are formed in 32-bit from the 32-bit stream and the sublayer's
    32-bit result, and a copy rounded to the model type is written beside it for the products.
    ``feed_forward`` (with ``ffn_norm``) may be None: the layer then has the first sublayer only.
    The norms must offer ``scaled_sum`` (``rms_norm_f32``)."""

    def __init__(self, mixer_norm, mixer, alpha: float, ffn_norm=None, feed_forward=None):
        if (ffn_norm is None) != (feed_forward is None):
            raise ValueError("post_norm: a feed-forward and its norm come together or not at all")
        for norm in (mixer_norm, ffn_norm):
            if norm is not None and not hasattr(norm, "scaled_sum"):
                raise ValueError(f"post_norm: the norm {type(norm).__name__} cannot take a scaled sum")
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ffn_norm = ffn_norm
        self.feed_forward = feed_forward
        self.alpha = float(alpha)

    def forward(self, ctx, x, pending, cache, state):
        if pending is not None:
            raise ValueError("post_norm: nothing can be pending in front of this block")
        h = x.rounded if isinstance(x, WideStream) else x
        x = self.mixer_norm.scaled_sum(ctx, x, self.mixer.forward(ctx, h, cache, state), self.alpha)
        if self.feed_forward is not None:
            x = self.ffn_norm.scaled_sum(ctx, x, self.feed_forward.forward(ctx, x.rounded), self.alpha)
        return x, None


@register_part("block", "gated_pre_norm")
class GatedPreNormBlock(Block):
    """Pre-norm sublayers whose results are scaled per channel and gated before the sum, on a
    residual stream kept in 32-bit floats (``WideStream``):

        h = norm1(x);  x <- x + scale1 * sigmoid(G1 h + b1) * mixer(h)
        h = norm2(x);  x <- x + scale2 * sigmoid(G2 h + b2) * ffn(h)          (if there is one)
        x <- x + rms_norm(token_input(x)) * gain                              (if there is one)

    ``token_input``: a part whose ``forward(ctx, x)`` gives a per-token addend from the stream
    (rounded to the model type) and the step's token ids, and whose ``norm_weight`` / ``eps`` say
    how the addend is RMS-normed before the sum.  The norms are given as parts (any norm with a
    float32 ``weight`` and ``eps`` whose ``forward`` reads a ``WideStream``); every sum and the
    norm that follows it run as one kernel.  The block hands the next block's first norm of its
    result on as ``pending`` when that block is of this kind too."""

    def __init__(self, hidden_size: int, mixer_norm, mixer, ffn_norm=None, feed_forward=None, token_input=None):
        if (ffn_norm is None) != (feed_forward is None):
            raise ValueError("gated_pre_norm: a feed-forward and its norm come together or not at all")
        self.hidden_size = hidden_size
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.ffn_norm, self.feed_forward = ffn_norm, feed_forward
        self.token_input = token_input

    def tensor_specs(self):
        h = self.hidden_size
        specs = {}
        for n in ("1", "2") if self.feed_forward is not None else ("1",):
            specs["scale" + n] = TensorSpec((h,), dtype="float32", init="one_plus_normal")
            specs["gate" + n + ".weight"] = TensorSpec((h, h))
            specs["gate" + n + ".bias"] = TensorSpec((h,), init="zeros")
        return specs

    def load(self, tensors):
        self.t = dict(tensors)

    def first_norm_after_product(self):
        return self.mixer_norm.weight, self.mixer_norm.eps

    def _gate(self, h, n):
        return ops.linear(h, self.t[f"gate{n}.weight"], self.t[f"gate{n}.bias"], out_dtype=torch.float32)

    def forward(self, ctx, x, pending, cache, state, then_norm=None):
        if not isinstance(x, WideStream) or x.full.dtype != torch.float32:
            raise ValueError("gated_pre_norm: the residual stream must be a 32-bit WideStream")
        full = x.full
        h = pending if pending is not None else self.mixer_norm.forward(ctx, x)
        addend = dict(y=self.mixer.forward(ctx, h, cache, state), gate=self._gate(h, 1), scale=self.t["scale1"])
        if self.feed_forward is not None:
            h = norm32_ops.stream_update(full, addend["y"], gate=addend["gate"], scale=addend["scale"],
                                         norm_weight=self.ffn_norm.weight, norm_eps=self.ffn_norm.eps,
                                         out_dtype=ctx.dtype)
            addend = dict(y=self.feed_forward.forward(ctx, h), gate=self._gate(h, 2), scale=self.t["scale2"])
        nw, ne = then_norm if then_norm is not None else (None, 0.0)
        if self.token_input is None:
            nxt = norm32_ops.stream_update(full, addend["y"], gate=addend["gate"], scale=addend["scale"], norm_weight=nw,
                                           norm_eps=ne, out_dtype=ctx.dtype if nw is not None else None)
            return x, nxt
        rounded = norm32_ops.stream_update(full, addend["y"], gate=addend["gate"], scale=addend["scale"],
                                           out_dtype=ctx.dtype)
        y = self.token_input.forward(ctx, rounded)
        nxt = norm32_ops.stream_update(full, y, rms_weight=self.token_input.norm_weight, rms_eps=self.token_input.eps,
                                       norm_weight=nw, norm_eps=ne, out_dtype=ctx.dtype if nw is not None else None)
        return x, nxt


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before and a norm after every sublayer, the normed result scaled per channel, on a
    residual stream kept in 32-bit floats (``WideStream``):

        x <- x + scale1 * out_norm1(mixer(norm1(x)))
        x <- x + scale2 * out_norm2(ffn(norm2(x)))            (if there is a feed-forward)

    The four norms are RMS norms given as parts with a float32 ``weight`` per coordinate and an
    ``eps`` (``rms_norm_f32``, ``rms_norm_scalar_f32``).  The sublayers return 32-bit rows.  Each
    sum runs as one kernel with the norm of the addend before it and the norm that reads the new
    stream after it (the out-norm's gain and the channel scale are one vector there); the block
    hands the next block's first norm of its result on as ``pending`` when that block asks for it."""

    def __init__(self, hidden_size: int, mixer_norm, mixer, mixer_out_norm, ffn_norm=None, feed_forward=None,
                 ffn_out_norm=None):
        if len({ffn_norm is None, feed_forward is None, ffn_out_norm is None}) != 1:
            raise ValueError("sandwich_norm: a feed-forward and its two norms come together or not at all")
        self.hidden_size = hidden_size
        self.mixer_norm, self.mixer, self.mixer_out_norm = mixer_norm, mixer, mixer_out_norm
        self.ffn_norm, self.feed_forward, self.ffn_out_norm = ffn_norm, feed_forward, ffn_out_norm
        self.gain1 = self.gain2 = None

    def tensor_specs(self):
        specs = {"scale1": TensorSpec((self.hidden_size,), dtype="float32", init="one_plus_normal")}
        if self.feed_forward is not None:
            specs["scale2"] = TensorSpec((self.hidden_size,), dtype="float32", init="one_plus_normal")
        return specs

    def load(self, tensors):
        self.t = dict(tensors)

    def prepare(self, device):
        # gain of the norm after the sublayer times the channel scale: what multiplies addend / rms(addend)
        self.gain1 = (self.mixer_out_norm.weight * self.t["scale1"]).contiguous()
        if self.feed_forward is not None:
            self.gain2 = (self.ffn_out_norm.weight * self.t["scale2"]).contiguous()

    def first_norm_after_product(self):
        return self.mixer_norm.weight, self.mixer_norm.eps

    def forward(self, ctx, x, pending, cache, state, then_norm=None):
        if not isinstance(x, WideStream) or x.full.dtype != torch.float32:
            raise ValueError("sandwich_norm: the residual stream must be a 32-bit WideStream")
        full = x.full
        h = pending if pending is not None else self.mixer_norm.forward(ctx, x)
        y, gain, eps = self.mixer.forward(ctx, h, cache, state), self.gain1, self.mixer_out_norm.eps
        if self.feed_forward is not None:
            h = norm32_ops.stream_update(full, y, rms_weight=gain, rms_eps=eps, norm_weight=self.ffn_norm.weight,
                                         norm_eps=self.ffn_norm.eps, norm_kind="rms", out_dtype=ctx.dtype)
            y, gain, eps = self.feed_forward.forward(ctx, h), self.gain2, self.ffn_out_norm.eps
        nw, ne = then_norm if then_norm is not None else (None, 0.0)
        nxt = norm32_ops.stream_update(full, y, rms_weight=gain, rms_eps=eps, norm_weight=nw, norm_eps=ne,
                                       norm_kind="rms", out_dtype=ctx.dtype if nw is not None else None)
        return x, nxt


@register_part("block", "output_norm")
class OutputNormBlock(Block):
    """A norm on every sublayer's result only, on a residual stream kept in 32-bit floats
    (``WideStream``):

        x <- x + out_norm1(mixer(x))
        x <- x + out_norm2(ffn(x))            (if there is a feed-forward)

    The sublayers read the stream itself (rounded to the model type for their products; on the
    32-bit path the stream's own rows).  The norms are RMS norms given as parts with a float32
    ``weight`` per coordinate and an ``eps`` (``rms_norm_f32``); the sublayers return 32-bit rows.
    Each sum runs as one kernel: RMS of the addend, gain, sum, and the rounded copy of the new
    stream that the next sublayer reads.  The block hands that copy of its result on as ``pending``
    when the block that follows asks for it (``first_norm_after_product`` answers with no norm)."""

    def __init__(self, hidden_size: int, mixer, mixer_out_norm, feed_forward=None, ffn_out_norm=None):
        if (feed_forward is None) != (ffn_out_norm is None):
            raise ValueError("output_norm: a feed-forward and its norm come together or not at all")
        self.hidden_size = hidden_size
        self.mixer, self.mixer_out_norm = mixer, mixer_out_norm
        self.feed_forward, self.ffn_out_norm = feed_forward, ffn_out_norm

    def first_norm_after_product(self):
        return None, 0.0  # no norm in front of the mixer: the rows themselves, in the products' type

    def forward(self, ctx, x, pending, cache, state, then_norm=None):
        if not isinstance(x, WideStream) or x.full.dtype != torch.float32:
            raise ValueError("output_norm: the residual stream must be a 32-bit WideStream")
        full = x.full
        copies = ctx.dtype != torch.float32  # whether the products read a rounded copy of the stream
        if not copies:
            h = full
        elif pending is not None:
            h = pending
        else:
            h = norm32_ops.stream_update(full, None, out_dtype=ctx.dtype)
        y, norm = self.mixer.forward(ctx, h, cache, state), self.mixer_out_norm
        if self.feed_forward is not None:
            h = norm32_ops.stream_update(full, y, rms_weight=norm.weight, rms_eps=norm.eps,
                                         out_dtype=ctx.dtype if copies else None)
            y, norm = self.feed_forward.forward(ctx, h if copies else full), self.ffn_out_norm
        nxt = norm32_ops.stream_update(full, y, rms_weight=norm.weight, rms_eps=norm.eps,
                                       out_dtype=ctx.dtype if (copies and then_norm is not None) else None)
        return x, nxt


@register_part("stream_input", "pass_entry")
class PassEntry(Part):
    """What enters a 32-bit residual stream where a pass over a run of repeated layers begins:

        x <- x + x0 + step[t]      (t: the number of the pass; x0, the embedding output, only in
                                    passes after the first and only with ``reinject``)

    ``step`` is a tensor [times, hidden_size].  One kernel does the sum and, when the layer that
    follows asks for it, that layer's first norm of the new stream (an RMS norm)."""

    def __init__(self, hidden_size: int, times: int, reinject: bool = True):
        if times < 1:
            raise ValueError(f"pass_entry: times={times} must be at least 1")
        self.hidden_size, self.times, self.reinject = hidden_size, int(times), bool(reinject)

    @property
    def needs_embedding(self) -> bool:
        return self.reinject and self.times > 1

    def tensor_specs(self):
        return {"step": TensorSpec((self.times, self.hidden_size), dtype="float32")}

    def load(self, tensors):
        self.step = tensors["step"]

    def forward(self, ctx, x, x0, t: int, then_norm=None):
        if not isinstance(x, WideStream) or x.full.dtype != torch.float32:
            raise ValueError("pass_entry: the residual stream must be a 32-bit WideStream")
        if not 0 <= t < self.times:
            raise ValueError(f"pass_entry: pass {t} of {self.times}")
        nw, ne = then_norm if then_norm is not None else (None, 0.0)
        y = x0 if (self.reinject and t > 0) else None
        return norm32_ops.stream_update(x.full, y, bias=self.step[t], norm_weight=nw, norm_eps=ne, norm_kind="rms",
                                        out_dtype=ctx.dtype if nw is not None else None)
