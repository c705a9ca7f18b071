"""Rotary position encoding, "default" type: inv_freq[i] = theta^(-2i/rotary_dim), angle =
position * inv_freq[i] in 32-bit, pairs (i, i + rotary_dim/2) rotated (half-split layout, the
default) or pairs (2i, 2i+1) (``layout="interleaved"``); the mixer that consumes the rotation
says which layouts its kernels turn.
puneethgv/DiSpec dispec/engine/model_runner.py:35-44,121-124; the table formula in 32-bit at
dispec/kv/transfer.py:50-58.  The reference rounds the cos/sin tables to the model type and
rotates in that type; here angles, cos, sin and the rotation are 32-bit and the result is
rounded once.

``slowed`` = (factor, original, fast, slow): frequencies slowed for contexts longer than the
``original`` one, by wavelength.  With n(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta)
(the pair whose wavelength makes t turns over the original context), lo = max(floor(n(fast)), 0),
hi = min(ceil(n(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
pair i turns at inv_freq[i] / factor * ramp_i + inv_freq[i] * (1 - ramp_i): fast pairs keep their
frequency, slow pairs are divided by ``factor``, those between are blended.  Cosine and sine are
then multiplied by 0.1 ln(factor) + 1 (``Rotation.magnitude``), which a mixer's kernels apply to
queries and keys alike."""
from __future__ import annotations

import math

import torch

from dispec_b200.parts.base import PositionEncoding, Rotation
from dispec_b200.registry import register_part


@register_part("position_encoding", "rotary")
class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None, layout: str = "halves",
                 exact_table: bool = False, slowed: tuple | None = None):
        if layout not in ("halves", "interleaved"):
            raise ValueError(f"rotary layout {layout!r} is not one of 'halves', 'interleaved'")
        self.layout = layout
        # True: the frequencies are formed in 64-bit and rounded once to float32 (the nearest float32
        # to theta^(-2i/rotary_dim)); False: in float32 throughout, as the reference's table is
        self.exact_table = bool(exact_table)
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and within head_dim={head_dim}")
        self.inv_freq = None
        self.magnitude = 1.0
        self.slowed = None
        if slowed is not None:
            factor, original, fast, slow = (float(v) for v in slowed)
            if not (factor > 0.0 and original > 0 and fast > 0 and slow > 0 and self.theta > 0.0 and self.theta != 1.0):
                raise ValueError(f"slowed rotation: factor={factor} original={original} fast={fast} slow={slow} "
                                 f"theta={self.theta} do not describe one")
            self.slowed = (factor, original, fast, slow)
            self.magnitude = 0.1 * math.log(factor) + 1.0

    def prepare(self, device):
        wide = torch.float64 if (self.exact_table or self.slowed) else torch.float32
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=wide) / self.rotary_dim
        freq = 1.0 / (self.theta ** exponent)
        if self.slowed is not None:
            factor, original, fast, slow = self.slowed
            turns = lambda t: self.rotary_dim * math.log(original / (2 * math.pi * t)) / (2 * math.log(self.theta))
            lo = max(math.floor(turns(fast)), 0)
            hi = min(math.ceil(turns(slow)), self.rotary_dim - 1)
            ramp = ((torch.arange(self.rotary_dim // 2, dtype=wide) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            freq = freq / factor * ramp + freq * (1.0 - ramp)
        self.inv_freq = freq.to(torch.float32).to(device)

    def rotation(self):
        if self.inv_freq is None:
            raise RuntimeError("the rotary encoding was not prepared (load the model first)")
        return Rotation(self.inv_freq, self.rotary_dim, self.layout, self.magnitude)


@register_part("position_encoding", "none")
class NoPositionEncoding(PositionEncoding):
    """Keys and queries go to the scores as they are (``rotation()`` is None)."""
