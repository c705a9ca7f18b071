"""Row-wise kernels around a residual stream kept in 32-bit floats: the RMS norm of a scaled sum,
the per-head RMS norm with gain and gate that closes a linear-attention mixer, and xIELU.
Every operand is float32 or bfloat16 on its own; the arithmetic is 32-bit."""
from __future__ import annotations

import torch

from dispec_b200.ops import library as L


def _rows2d(t: torch.Tensor, what: str) -> None:
    if not (t.is_cuda and t.dim() == 2 and t.stride(1) == 1):
        raise L.KernelError(f"{what}: a CUDA matrix with unit column stride is needed (there is no CPU path)")


def sum_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, delta: torch.Tensor | None = None,
             alpha: float = 1.0, rows: torch.Tensor | None = None, out32: torch.Tensor | None = None,
             out_dtype: torch.dtype | None = None, want32: bool = True):
    """y = weight * s / sqrt(mean(s^2) + eps) with s = alpha * x + delta, per row, in 32-bit.

    Returns (y as float32 or None, y rounded to ``out_dtype`` or None).  ``out32`` may be ``x``
    itself.  ``rows`` (int32) gathers input rows; the outputs are dense."""
    _rows2d(x, "sum_norm")
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape == (x.shape[1],)
    if delta is not None:
        _rows2d(delta, "sum_norm")
        assert delta.shape == x.shape
    n = x.shape[0] if rows is None else rows.shape[0]
    width = x.shape[1]
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    y32 = out32
    if y32 is None and want32:
        y32 = torch.empty((n, width), dtype=torch.float32, device=x.device)
    y16 = None
    if out_dtype is not None and not (out_dtype == torch.float32 and y32 is not None):
        y16 = torch.empty((n, width), dtype=out_dtype, device=x.device)
    L.check(L.core().dsp_sum_norm(
        L.ptr(x), L.dtype_code(x.dtype), L.i64(x.stride(0)), L.ptr(delta),
        L.dtype_code(delta.dtype) if delta is not None else 0, L.i64(delta.stride(0) if delta is not None else 0),
        L.ptr(weight), L.f32(alpha), L.f32(eps), L.ptr(rows), L.ptr(y32), L.i64(y32.stride(0) if y32 is not None else 0),
        L.ptr(y16), L.dtype_code(y16.dtype) if y16 is not None else 0, L.i64(y16.stride(0) if y16 is not None else 0),
        n, width, L.stream_handle()))
    if out_dtype == torch.float32 and y16 is None:
        y16 = y32
    return y32, y16


def head_norm_gate(o: torch.Tensor, num_heads: int, eps: float, out_dtype: torch.dtype,
                   gain: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                   gate_kind: str = "silu") -> torch.Tensor:
    """o float32 [T, H * dv]: every head's dv values divided by their root mean square (eps inside
    the root), times ``gain`` [dv] (optional) and act(gate[t, h * dv + j]) (optional; ``gate_kind``
    "silu" or "sigmoid").  With ``num_heads`` 1 the whole row is normed together."""
    _rows2d(o, "head_norm_gate")
    assert o.dtype == torch.float32 and o.shape[1] % num_heads == 0
    T, dv = o.shape[0], o.shape[1] // num_heads
    if gain is not None:
        assert gain.dtype == torch.float32 and gain.shape == (dv,) and gain.is_contiguous()
    if gate is not None:
        _rows2d(gate, "head_norm_gate")
        assert gate.shape == o.shape
    y = torch.empty((T, o.shape[1]), dtype=out_dtype, device=o.device)
    L.check(L.core().dsp_head_norm_gate(
        L.ptr(o), L.i64(o.stride(0)), L.ptr(gain), L.ptr(gate), L.dtype_code(gate.dtype) if gate is not None else 0,
        L.i64(gate.stride(0) if gate is not None else 0), L.ptr(y), L.dtype_code(out_dtype), L.i64(y.stride(0)),
        T, num_heads, dv, L.f32(eps), {"silu": 0, "sigmoid": 1}[gate_kind], L.stream_handle()))
    return y


def xielu(z: torch.Tensor, params: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """xIELU of every element: softplus(p) z^2 + z/2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2
    otherwise; ``params`` = (p, q) as a float32 device tensor."""
    _rows2d(z, "xielu")
    assert params.dtype == torch.float32 and params.numel() == 2 and params.is_cuda
    y = torch.empty(z.shape, dtype=out_dtype, device=z.device)
    L.check(L.core().dsp_xielu(L.ptr(z), L.dtype_code(z.dtype), L.i64(z.stride(0)), L.ptr(params), L.ptr(y),
                               L.dtype_code(out_dtype), L.i64(y.stride(0)), L.i64(z.shape[0]), z.shape[1],
                               L.stream_handle()))
    return y


def layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
               rows: torch.Tensor | None = None) -> torch.Tensor:
    """y = (x - mean) / sqrt(var + eps) * weight per row (var: the mean of the squared deviations),
    in 32-bit, written as ``out_dtype``.  ``rows`` (int32) gathers input rows."""
    _rows2d(x, "layer_norm")
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape == (x.shape[1],)
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    n = x.shape[0] if rows is None else rows.shape[0]
    y = torch.empty((n, x.shape[1]), dtype=out_dtype, device=x.device)
    L.check(L.core().dsp_layer_norm(L.ptr(x), L.dtype_code(x.dtype), L.i64(x.stride(0)), L.ptr(weight), L.f32(eps),
                                    L.ptr(rows), L.ptr(y), L.dtype_code(out_dtype), L.i64(y.stride(0)), n, x.shape[1],
                                    L.stream_handle()))
    return y


def stream_update(x32: torch.Tensor, y: torch.Tensor | None, *, gate: torch.Tensor | None = None,
                  scale: torch.Tensor | None = None, rms_weight: torch.Tensor | None = None, rms_eps: float = 0.0,
                  bias: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None, norm_eps: float = 0.0,
                  norm_kind: str = "layer", out_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """x32 += d in place (float32 rows), with d = y * scale * sigmoid(gate) when ``gate`` is given,
    d = y / sqrt(mean(y^2) + rms_eps) * rms_weight when ``rms_weight`` is, else d = y (``y`` None:
    0); ``bias`` (float32 [width]) is added to every row as well.  With ``out_dtype``: also returns
    the norm of the new rows times ``norm_weight`` (``norm_kind`` "layer": mean taken off; "rms":
    x / sqrt(mean(x^2) + norm_eps)) or, without ``norm_weight``, the new rows themselves, in that type."""
    _rows2d(x32, "stream_update")
    assert x32.dtype == torch.float32
    if y is not None:
        _rows2d(y, "stream_update")
        assert y.shape == x32.shape
    assert norm_kind in ("layer", "rms")
    width = x32.shape[1]
    for v in (scale, rms_weight, norm_weight, bias):
        assert v is None or (v.dtype == torch.float32 and v.is_contiguous() and v.shape == (width,))
    if gate is not None:
        _rows2d(gate, "stream_update")
        assert gate.shape == x32.shape
    out = torch.empty(x32.shape, dtype=out_dtype, device=x32.device) if out_dtype is not None else None
    L.check(L.core().dsp_stream_update(
        L.ptr(x32), L.i64(x32.stride(0)), L.ptr(y), L.dtype_code(y.dtype) if y is not None else 0,
        L.i64(y.stride(0) if y is not None else 0), L.ptr(gate),
        L.dtype_code(gate.dtype) if gate is not None else 0, L.i64(gate.stride(0) if gate is not None else 0),
        L.ptr(scale), L.ptr(rms_weight), L.f32(rms_eps), L.ptr(bias), L.ptr(norm_weight), L.f32(norm_eps),
        int(norm_kind == "rms"), L.ptr(out),
        L.dtype_code(out_dtype) if out is not None else 0, L.i64(out.stride(0) if out is not None else 0),
        x32.shape[0], width, L.stream_handle()))
    return out


def clamped_glu(z: torch.Tensor, limit: float, alpha: float, out_dtype: torch.dtype) -> torch.Tensor:
    """z [T, 2 n] = [gates | ups] -> [T, n]: g = min(gate, limit), u = clamp(up, -limit, limit),
    g * sigmoid(alpha * g) * (u + 1)."""
    _rows2d(z, "clamped_glu")
    assert z.shape[1] % 2 == 0
    n = z.shape[1] // 2
    y = torch.empty((z.shape[0], n), dtype=out_dtype, device=z.device)
    L.check(L.core().dsp_clamped_glu(L.ptr(z), L.dtype_code(z.dtype), L.i64(z.stride(0)), L.ptr(y),
                                     L.dtype_code(out_dtype), L.i64(y.stride(0)), L.i64(z.shape[0]), n, L.f32(limit),
                                     L.f32(alpha), L.stream_handle()))
    return y


def gelu_table_gate(z: torch.Tensor, table: torch.Tensor, offset: int, ids: torch.Tensor,
                    out_dtype: torch.dtype) -> torch.Tensor:
    """y[t, j] = gelu_tanh(z[t, j]) * table[ids[t], offset + j]."""
    _rows2d(z, "gelu_table_gate")
    _rows2d(table, "gelu_table_gate")
    assert ids.dtype == torch.int32 and ids.is_contiguous() and ids.shape[0] >= z.shape[0]
    assert 0 <= offset and offset + z.shape[1] <= table.shape[1]
    y = torch.empty(z.shape, dtype=out_dtype, device=z.device)
    L.check(L.core().dsp_gelu_table_gate(
        L.ptr(z), L.dtype_code(z.dtype), L.i64(z.stride(0)), L.ptr(table), L.dtype_code(table.dtype),
        L.i64(table.stride(0)), table.shape[0], offset, L.ptr(ids), L.ptr(y), L.dtype_code(out_dtype),
        L.i64(y.stride(0)), L.i64(z.shape[0]), z.shape[1], L.stream_handle()))
    return y


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place (float32 rows)."""
    _rows2d(x, "softcap")
    assert x.dtype == torch.float32
    L.check(L.core().dsp_softcap(L.ptr(x), L.i64(x.stride(0)), L.i64(x.shape[0]), x.shape[1], L.f32(cap),
                                 L.stream_handle()))
    return x


def embed_scaled(table: torch.Tensor, ids: torch.Tensor, scale: float) -> torch.Tensor:
    """float32 rows table[ids[t]] * scale (a token id outside the table gives zeros and sets the
    device error word)."""
    _rows2d(table, "embed_scaled")
    assert table.is_contiguous() and ids.dtype == torch.int32 and ids.is_contiguous()
    out = torch.empty((ids.shape[0], table.shape[1]), dtype=torch.float32, device=table.device)
    L.check(L.core().dsp_embed_scaled(L.ptr(table), L.dtype_code(table.dtype), table.shape[0], L.ptr(ids),
                                      L.f32(scale), L.ptr(out), L.i64(out.stride(0)), L.i64(ids.shape[0]),
                                      table.shape[1], L.stream_handle()))
    return out


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x <- x * factor in place (float32 rows)."""
    _rows2d(x, "scale_")
    assert x.dtype == torch.float32
    L.check(L.core().dsp_scale_rows(L.ptr(x), L.i64(x.stride(0)), L.i64(x.shape[0]), x.shape[1], L.f32(factor),
                                    L.stream_handle()))
    return x


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """y[t, j] = x[t, j] * sigmoid(gate[t, j // per]) with per = x's columns / gate's columns: a gate
    per element (equal widths) or one number for each run of neighbouring columns (a head)."""
    _rows2d(x, "sigmoid_gate")
    _rows2d(gate, "sigmoid_gate")
    assert gate.shape[0] == x.shape[0] and gate.shape[1] > 0 and x.shape[1] % gate.shape[1] == 0
    y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    L.check(L.core().dsp_sigmoid_gate(L.ptr(x), L.dtype_code(x.dtype), L.i64(x.stride(0)), L.ptr(gate),
                                      L.dtype_code(gate.dtype), L.i64(gate.stride(0)), x.shape[1] // gate.shape[1],
                                      L.ptr(y), L.dtype_code(out_dtype), L.i64(y.stride(0)), L.i64(x.shape[0]),
                                      x.shape[1], L.stream_handle()))
    return y


def diff_heads(a: torch.Tensor, num_heads: int, lam: float, post: float, eps: float, out_dtype: torch.dtype,
               gate: torch.Tensor | None = None) -> torch.Tensor:
    """a [T, 2 H dv]: per token the results of two attention maps per head, side by side.  Returns
    [T, H dv]: o = a1 - lam * a2, every head divided by its root mean square (eps inside the root),
    times ``post`` and sigmoid(gate[t, h]) (``gate`` [T, H], optional).  32-bit arithmetic."""
    _rows2d(a, "diff_heads")
    assert a.shape[1] % (2 * num_heads) == 0
    T, dv = a.shape[0], a.shape[1] // (2 * num_heads)
    if gate is not None:
        _rows2d(gate, "diff_heads")
        assert gate.shape == (T, num_heads)
    y = torch.empty((T, num_heads * dv), dtype=out_dtype, device=a.device)
    L.check(L.core().dsp_diff_heads(L.ptr(a), L.dtype_code(a.dtype), L.i64(a.stride(0)), L.f32(lam), L.f32(post),
                                    L.f32(eps), L.ptr(gate), L.dtype_code(gate.dtype) if gate is not None else 0,
                                    L.i64(gate.stride(0) if gate is not None else 0), L.ptr(y), L.dtype_code(out_dtype),
                                    L.i64(y.stride(0)), T, num_heads, dv, L.stream_handle()))
    return y
