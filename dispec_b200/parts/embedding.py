"""Token embedding (row gather, no scaling: puneethgv/DiSpec dispec/engine/model_runner.py:63,199;
``scaled_embedding``: times a constant, as the first value of a 32-bit stream) and the output
head (logits = h W^T, no bias, 32-bit logits; :66,228-231; optionally squashed by
cap * tanh(logits / cap))."""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.ops import norm32 as norm32_ops
from dispec_b200.parts.base import Part, TensorSpec, WideStream
from dispec_b200.registry import register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx):
        return ops.embed(self.weight, ctx.token_ids)


@register_part("embedding", "scaled_embedding")
class ScaledEmbedding(Part):
    """x = table[token] * scale in 32-bit floats: the start of a residual stream that is kept in
    32-bit (``WideStream`` without a rounded copy; whoever needs one makes it)."""

    def __init__(self, vocab_size: int, hidden_size: int, scale: float):
        self.vocab_size, self.hidden_size, self.scale = vocab_size, hidden_size, float(scale)
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx):
        return WideStream(norm32_ops.embed_scaled(self.weight, ctx.token_ids, self.scale), None)


@register_part("head", "linear_head")
class LinearHead(Part):
    """A tied head names the embedding's checkpoint tensor; the loader then hands both parts
    the same device tensor."""

    def __init__(self, vocab_size: int, hidden_size: int, softcap: float | None = None, scale: float = 1.0):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        if softcap is not None and not softcap > 0:
            raise ValueError(f"the cap on the logits must be positive, got {softcap}")
        self.softcap = softcap  # logits <- cap * tanh(logits / cap)
        self.scale = float(scale)  # logits <- logits * scale (before the cap)
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx, h):
        logits = ops.linear(h, self.weight, out_dtype=torch.float32)
        if self.scale != 1.0:
            norm32_ops.scale_(logits, self.scale)
        if self.softcap is not None:
            norm32_ops.softcap_(logits, self.softcap)
        return logits
