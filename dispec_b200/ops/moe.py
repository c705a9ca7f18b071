"""Mixture of experts on the device: router with groups, rows sorted by expert, the experts'
products, the weighted sum.  See ``csrc/moe.cu``."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from dispec_b200.ops import library as L


def _lib():
    return L.mixer_library("moe")


def route(h: torch.Tensor, w_router: torch.Tensor, groups: int, keep: int, top: int, score: str = "softmax",
          group_score: str = "max", normalize: bool = False, weight_scale: float = 1.0, extra_rows: int = 0):
    """h [T, W] (either type), w_router float32 [E, W] -> (ids int32 [T, top], weights float32
    [T, top]): softmax over all experts in 32-bit (``score`` "sigmoid": the sigmoid of every
    expert's logit instead, chosen by the logits, so that scores which round to the same number
    do not tie); the ``top`` largest scores among the experts
    of the ``keep`` groups (of ``groups`` equal runs of neighbours) with the largest best score;
    the weights are those scores.  ``group_score`` "top2_sum": a group's score is the sum of its
    two largest scores.  ``normalize``: the weights are the chosen scores divided by their sum
    (+ 1e-20), times ``weight_scale``.  ``extra_rows`` = X > 0: the last X rows of ``w_router``
    are not experts; the sigmoids of their logits come back as a third result, float32 [T, X]."""
    if not (h.is_cuda and w_router.is_cuda):
        raise L.KernelError("moe.route: CUDA tensors only (there is no CPU path)")
    assert h.dim() == 2 and h.stride(1) == 1 and w_router.dtype == torch.float32 and w_router.is_contiguous()
    T, W = h.shape
    E = w_router.shape[0] - extra_rows
    assert w_router.shape == (E + extra_rows, W) and E > 0
    ids = torch.empty((T, top), dtype=torch.int32, device=h.device)
    wts = torch.empty((T, top), dtype=torch.float32, device=h.device)
    extra = torch.empty((T, extra_rows), dtype=torch.float32, device=h.device) if extra_rows else None
    L.check(_lib().dsp_moe_route(L.ptr(h), L.dtype_code(h.dtype), L.i64(h.stride(0)), L.ptr(w_router), T, W, E,
                                 groups, keep, top, {"softmax": 0, "sigmoid": 1}[score],
                                 {"max": 0, "top2_sum": 1}[group_score], int(bool(normalize)), L.f32(weight_scale),
                                 extra_rows, L.ptr(extra), L.ptr(ids), L.ptr(wts), L.stream_handle()))
    return (ids, wts, extra) if extra_rows else (ids, wts)


@dataclass
class ExpertPlan:
    """The (token, choice) pairs of a step listed expert by expert, cut into tiles."""
    sorted_pair: torch.Tensor  # [pairs] int32: pair index t * top + k at each sorted place
    offsets: torch.Tensor  # [E + 1] int32
    tiles: torch.Tensor  # [3, max_tiles] int32: expert, first sorted row, rows
    n_tiles: torch.Tensor  # [1] int32
    max_tiles: int
    num_pairs: int
    top: int
    tensor_cores: int  # 0: the 32-bit kernel; 1, 2: the tensor-core kernel with tiles of 64, 128 rows


def tensor_cores_supported(dtype: torch.dtype, *inner_sizes: int) -> bool:
    """The tensor-core product takes bfloat16 operands whose inner sizes are multiples of 8."""
    return dtype == torch.bfloat16 and all(k % 8 == 0 for k in inner_sizes)


WIDE_TILES_FROM = 96  # (token, choice) pairs per expert on average from which tiles of 128 rows pay


def plan(ids: torch.Tensor, num_experts: int, tensor_cores: bool = False) -> ExpertPlan:
    T, top = ids.shape
    n = T * top
    lib = _lib()
    tensor_cores = (2 if n >= WIDE_TILES_FROM * num_experts else 1) if tensor_cores else 0
    rows = int(lib.dsp_moe_tile_rows(tensor_cores))
    max_tiles = n // rows + num_experts
    dev = ids.device
    sorted_pair = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    tiles = torch.empty((3, max_tiles), dtype=torch.int32, device=dev)
    n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    L.check(lib.dsp_moe_plan(L.ptr(ids), n, num_experts, rows, L.ptr(offsets), L.ptr(sorted_pair), L.ptr(tiles[0]),
                             L.ptr(tiles[1]), L.ptr(tiles[2]), L.ptr(n_tiles), max_tiles, L.stream_handle()))
    return ExpertPlan(sorted_pair, offsets, tiles, n_tiles, max_tiles, n, top, tensor_cores)


def expert_product(p: ExpertPlan, a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, *,
                   rows_are_tokens: bool, scatter: bool, square_relu: bool = False,
                   clamped_glu: tuple | None = None, row_scale: torch.Tensor | None = None,
                   up_shift: float = 1.0) -> torch.Tensor:
    """C = act(A W_e^T) for every pair, with its expert's matrix (w: [E, N, K]).  ``rows_are_tokens``:
    A holds one row per token (a pair reads its token's row); otherwise one row per sorted place.
    ``scatter``: the result row of a pair goes to its pair index t * top + k; otherwise to its
    sorted place.  Returns [pairs, N].

    ``clamped_glu`` = (limit, alpha): the rows of every W_e alternate between a gate matrix and an
    up matrix (row 2j: gate j, row 2j + 1: up j) and the result is the gated unit
    min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + up_shift), [pairs, N / 2]
    (limit infinite, alpha 1 and ``up_shift`` 0: silu(g) * u);
    ``row_scale`` (float32 [pairs], by pair index t * top + k; needs ``rows_are_tokens``): a factor
    on the pair's input row, applied to the 32-bit sums g and u before the clamps."""
    assert a.dim() == 2 and a.stride(1) == 1 and w.dim() == 3 and w.is_contiguous() and a.dtype == w.dtype
    E, N, K = w.shape
    assert a.shape[1] == K and not (square_relu and clamped_glu)
    act, limit, alpha = (1 if square_relu else 0), 0.0, 0.0
    if clamped_glu is not None:
        act, (limit, alpha) = 2, clamped_glu
        assert N % 2 == 0
    if row_scale is not None:
        assert clamped_glu is not None and rows_are_tokens
        assert row_scale.dtype == torch.float32 and row_scale.is_contiguous() and row_scale.numel() == p.num_pairs
    out = torch.empty((max(p.num_pairs, 1), N // 2 if act == 2 else N), dtype=out_dtype, device=a.device)
    L.check(_lib().dsp_moe_product(
        L.ptr(a), L.dtype_code(a.dtype), L.i64(a.stride(0)), L.ptr(p.sorted_pair if rows_are_tokens else None),
        p.top if rows_are_tokens else 1, L.ptr(w), L.ptr(out), L.dtype_code(out_dtype), L.i64(out.stride(0)),
        L.ptr(p.sorted_pair if scatter else None), L.ptr(p.tiles[0]), L.ptr(p.tiles[1]), L.ptr(p.tiles[2]),
        L.ptr(p.n_tiles), p.max_tiles, N, K, act, L.ptr(row_scale), L.f32(limit), L.f32(alpha), L.f32(up_shift), int(p.tensor_cores),
        L.stream_handle()))
    return out[:p.num_pairs]


def combine(pair_rows: torch.Tensor, wts: torch.Tensor | None, ids: torch.Tensor,
            base: torch.Tensor | None = None, base_scale: torch.Tensor | None = None) -> torch.Tensor:
    """y[t] = base[t] * base_scale[t] + sum over k of wts[t, k] * pair_rows[t * top + k] (float32);
    without ``wts`` every weight is 1, without ``base`` the sum starts from 0, without ``base_scale``
    (float32, one number per token) the base counts as it is."""
    T, top = ids.shape
    assert pair_rows.dtype == torch.float32 and pair_rows.stride(1) == 1 and pair_rows.shape[0] == T * top
    if base is not None:
        assert base.dtype == torch.float32 and base.stride(1) == 1 and base.shape == (T, pair_rows.shape[1])
    if base_scale is not None:
        assert base is not None and base_scale.dtype == torch.float32 and base_scale.is_contiguous()
        assert base_scale.numel() == T
    y = torch.empty((T, pair_rows.shape[1]), dtype=torch.float32, device=pair_rows.device)
    L.check(_lib().dsp_moe_combine(L.ptr(pair_rows), L.i64(pair_rows.stride(0)), L.ptr(wts), L.ptr(ids), L.ptr(base),
                                   L.i64(base.stride(0) if base is not None else 0), L.ptr(base_scale), L.ptr(y),
                                   L.i64(y.stride(0)), L.i64(T), top, pair_rows.shape[1], L.stream_handle()))
    return y
