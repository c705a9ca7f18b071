"""RMSNorm.  y = w * round(x * rsqrt(mean(x^2) + eps)): 32-bit statistics, the normalised
value rounded to the storage type before the gain is applied (the order the reference's
borrowed module was measured to use; applied at puneethgv/DiSpec
dispec/engine/model_runner.py:215,218,220)."""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.ops import gemm as gemm_ops
from dispec_b200.ops import norm32 as norm32_ops
from dispec_b200.parts.base import Norm, TensorSpec, WideStream
from dispec_b200.registry import register_part


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size = hidden_size
        self.eps = eps
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.hidden_size,), init="one_plus_normal")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx, x, rows=None):
        return ops.rms_norm(x, self.weight, self.eps, rows=rows)

    def deferred(self, x):
        """This norm of ``x`` as an input that its consumer applies (a product takes it apart
        where it can, see ``ops.gemm.NormedRows``; otherwise the norm kernel runs there)."""
        return gemm_ops.NormedRows(x, self.weight, self.eps)

    def after_product(self):
        """(weight, eps) for a product that writes the rows this norm reads (``linear(then_norm=)``)."""
        return self.weight, self.eps

    def forward_add(self, ctx, residual, delta, rows=None):
        """Norm of residual + delta (32-bit sum).  Without ``rows`` the sum replaces ``residual``."""
        return ops.rms_norm(residual, self.weight, self.eps, delta=delta, rows=rows,
                            write_back=rows is None)


@register_part("norm", "rms_norm_f32")
class RMSNorm32(Norm):
    """y = w * x / sqrt(mean(x^2) + eps), everything in 32-bit: the gain is kept as float32 in
    every mode and nothing is rounded before the result.  Reads a 32-bit stream (``WideStream``)
    or a plain tensor of either type.  ``forward`` returns the result in ``ctx.dtype`` (what a
    product reads); ``scaled_sum`` is the norm of alpha * x + delta, returned as a new
    ``WideStream`` (the arrangement with the norm after the sum)."""

    def __init__(self, hidden_size: int, eps: float, unit_offset: bool = False):
        self.hidden_size = hidden_size
        self.eps = eps
        # True: the gain is stored around zero, y = (1 + w) * x / sqrt(mean(x^2) + eps); 1 + w is formed once, in 32-bit
        self.unit_offset = bool(unit_offset)
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.hidden_size,), dtype="float32",
                                     init="normal" if self.unit_offset else "one_plus_normal")}

    def load(self, tensors):
        self.weight = (tensors["weight"] + 1.0).contiguous() if self.unit_offset else tensors["weight"]

    @staticmethod
    def _full(x):
        return x.full if isinstance(x, WideStream) else x

    def forward(self, ctx, x, rows=None):
        return norm32_ops.sum_norm(self._full(x), self.weight, self.eps, rows=rows, out_dtype=ctx.dtype,
                                   want32=False)[1]

    def scaled_sum(self, ctx, x, delta, alpha: float) -> WideStream:
        """Norm of alpha * x + delta (32-bit sum).  The 32-bit result replaces ``x.full`` when x
        is a stream of this model's own making."""
        src = self._full(x)
        into = src if isinstance(x, WideStream) and src.dtype == torch.float32 else None
        full, rounded = norm32_ops.sum_norm(src, self.weight, self.eps, delta=delta, alpha=alpha,
                                            out32=into, out_dtype=ctx.dtype)
        return WideStream(full, rounded)


@register_part("norm", "rms_norm_scalar_f32")
class ScalarRMSNorm32(RMSNorm32):
    """y = g * x / sqrt(mean(x^2) + eps) with one number g for all coordinates (a tensor without
    dimensions), everything in 32-bit.  The kernels take a gain per coordinate: ``weight`` is g
    repeated ``hidden_size`` times."""

    def tensor_specs(self):
        return {"weight": TensorSpec((), dtype="float32", init="one_plus_normal")}

    def load(self, tensors):
        self.weight = tensors["weight"].reshape(1).expand(self.hidden_size).contiguous()


@register_part("norm", "layer_norm_f32")
class LayerNorm32(Norm):
    """y = (x - mean) / sqrt(var + eps) * w with a gain and no bias (var: the mean of the squared
    deviations), everything in 32-bit; the gain is float32 in every mode.  Reads a 32-bit stream
    (``WideStream``) or a plain tensor; the result comes in ``ctx.dtype`` (what a product reads)."""

    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size = hidden_size
        self.eps = float(eps)
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.hidden_size,), dtype="float32", init="one_plus_normal")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx, x, rows=None):
        full = x.full if isinstance(x, WideStream) else x
        return norm32_ops.layer_norm(full, self.weight, self.eps, ctx.dtype, rows=rows)
