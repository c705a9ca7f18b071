"""Attention over a cached latent (one shared key/value row per token): the store of a token's
normalised latent and rotated key part into the pages, and the attention itself in 32-bit.
See ``csrc/attn_latent.cu``."""
from __future__ import annotations

import os

import torch

from dispec_b200.ops import library as L

_LAYOUTS = {"interleaved": 0, "halves": 1}  # which dimensions form pair i: (2i, 2i+1) or (i, i + rot/2)


def latent_store(down: torch.Tensor, c_off: int, r_off: int, gain: torch.Tensor, eps: float,
                 inv_freq: torch.Tensor | None, rot: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                 page_table: torch.Tensor, c_pool: torch.Tensor, r_pool: torch.Tensor,
                 layout: str = "interleaved", magnitude: float = 1.0, query_latent: tuple | None = None):
    """``down`` [T, columns]: rows of the down projection; columns c_off.. hold the R latent values
    (RMS-normed here with ``gain``), columns r_off.. the r values of the shared key part (pair i
    of its first ``rot`` values, (2i, 2i+1) or with ``layout`` "halves" (i, i + rot/2), turned by
    position * inv_freq[i], cosine and sine times ``magnitude``).  Pools:
    [num_pages, 1, page_size, R] and [num_pages, 1, page_size, r].
    ``query_latent`` = (offset, size, gain, out_dtype): the same launch also returns the RMS norm
    (same eps) of columns offset .. offset + size of every row times ``gain``, [T, size]."""
    if not (down.is_cuda and c_pool.is_cuda):
        raise L.KernelError("latent_store: CUDA tensors only (there is no CPU path)")
    assert down.dim() == 2 and down.stride(1) == 1
    num_pages, one, page_size, R = c_pool.shape
    r = r_pool.shape[3]
    assert one == 1 and r_pool.shape[:3] == (num_pages, 1, page_size) and r_pool.dtype == c_pool.dtype
    assert c_pool.is_contiguous() and r_pool.is_contiguous()
    assert gain.dtype == torch.float32 and gain.shape == (R,) and gain.is_contiguous()
    assert positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32
    assert page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.stride(1) == 1
    if rot:
        assert inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.shape[0] >= rot // 2
    cq, q_off, Qn, q_gain = None, 0, 0, None
    if query_latent is not None:
        q_off, Qn, q_gain, cq_dtype = query_latent
        assert q_gain.dtype == torch.float32 and q_gain.shape == (Qn,) and q_gain.is_contiguous()
        assert 0 <= q_off and q_off + Qn <= down.shape[1]
        cq = torch.empty((down.shape[0], Qn), dtype=cq_dtype, device=down.device)
    lib = L.mixer_library("attn_latent")
    L.check(lib.dsp_latent_store(
        L.ptr(down), L.dtype_code(down.dtype), L.i64(down.stride(0)), c_off, r_off, L.ptr(gain), L.f32(eps),
        L.ptr(inv_freq), rot, _LAYOUTS[layout], L.f32(magnitude), L.ptr(positions), L.ptr(seq_of_token),
        L.ptr(page_table), page_table.stride(0),
        L.ptr(c_pool), L.ptr(r_pool), L.dtype_code(c_pool.dtype), down.shape[0], R, r, page_size, num_pages,
        q_off, Qn, L.ptr(q_gain), L.ptr(cq), L.dtype_code(cq.dtype) if cq is not None else 0,
        L.i64(cq.stride(0) if cq is not None else 0), L.stream_handle()))
    return cq


def latent_attention(q_absorbed: torch.Tensor, q: torch.Tensor, q_head_stride: int, qr_off: int,
                     inv_freq: torch.Tensor | None, rot: int, c_pool: torch.Tensor, r_pool: torch.Tensor,
                     page_table: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                     num_heads: int, scale: float, out_dtype: torch.dtype, layout: str = "interleaved",
                     magnitude: float = 1.0, window: int = 0) -> torch.Tensor:
    """``q_absorbed`` float32 [T, H * R]: every head's query with the key map folded in.  ``q``
    [T, columns]: the projected queries; head h's part to be rotated starts at column
    h * q_head_stride + qr_off and has r values.  Returns sum_j softmax_j c_j per head as
    [T, H * R] of ``out_dtype``; the query at position p sees every cached j <= p, with ``window``
    W > 0 those with p - W < j.  ``layout`` / ``magnitude``: as in ``latent_store``."""
    if not (q_absorbed.is_cuda and c_pool.is_cuda):
        raise L.KernelError("latent_attention: CUDA tensors only (there is no CPU path)")
    num_pages, _, page_size, R = c_pool.shape
    r = r_pool.shape[3]
    T = positions.shape[0]
    assert q_absorbed.dtype == torch.float32 and q_absorbed.shape == (T, num_heads * R) and q_absorbed.stride(1) == 1
    assert q.dim() == 2 and q.stride(1) == 1 and q.shape[0] == T
    assert c_pool.is_contiguous() and r_pool.is_contiguous() and r_pool.dtype == c_pool.dtype
    assert page_table.dtype == torch.int32 and page_table.stride(1) == 1
    assert positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32
    out = torch.empty((T, num_heads * R), dtype=out_dtype, device=q.device)
    lib = L.mixer_library("attn_latent")
    L.check(lib.dsp_attn_latent(
        L.ptr(q_absorbed), L.i64(q_absorbed.stride(0)), L.ptr(q), L.dtype_code(q.dtype), L.i64(q.stride(0)),
        q_head_stride, qr_off, L.ptr(inv_freq), rot, _LAYOUTS[layout], L.f32(magnitude), int(window), L.ptr(c_pool),
        L.ptr(r_pool), L.dtype_code(c_pool.dtype),
        L.ptr(page_table), page_table.stride(0), L.ptr(positions), L.ptr(seq_of_token), L.ptr(out),
        L.dtype_code(out_dtype), L.i64(out.stride(0)), T, num_heads, R, r, page_size, num_pages, L.f32(scale),
        L.stream_handle()))
    return out


MMA_ROWS_PER_TILE = 64  # query rows, (token, head) pairs, of one tile of the tensor-core kernel
MMA_KEYS_PER_TILE = 32
_MMA_LATENT_SIZES = (64, 128, 192, 256, 384, 512)


def mma_tokens_per_tile(num_heads: int) -> int:
    """Query tokens of one request that share a tile of the tensor-core kernel."""
    return max(1, MMA_ROWS_PER_TILE // min(num_heads, MMA_ROWS_PER_TILE))


def mma_supported(kv_rank: int, rot_dim: int, pool_dtype: torch.dtype) -> bool:
    if os.environ.get("DISPEC_B200_LATENT_MMA") == "0":  # measurements: everything on the 32-bit kernel
        return False
    row_bytes = ((2 * (kv_rank + rot_dim) + 127) // 128) * 128 + 16
    return (pool_dtype == torch.bfloat16 and kv_rank in _MMA_LATENT_SIZES and rot_dim % 16 == 0
            and 128 * row_bytes + 64 * 80 + 2048 + 4 * 64 * 36 * 4 <= 227 * 1024)


def choose_key_splits(num_tiles: int, head_chunks: int, max_ctx: int, device) -> int:
    """Key ranges per single-token tile so that the launch covers the device about once, each
    range keeping at least four key tiles."""
    from dispec_b200.ops import tuning
    ctas = max(1, num_tiles * head_chunks)
    want = max(1, tuning.sm_count(device) // ctas)
    room = max(1, -(-max_ctx // MMA_KEYS_PER_TILE) // 4)
    return int(min(want, room, tuning.MAX_SPLITS))


def latent_attention_tiles(ctx, q_absorbed: torch.Tensor, q: torch.Tensor, q_head_stride: int, qr_off: int,
                           inv_freq: torch.Tensor | None, rot: int, c_pool: torch.Tensor, r_pool: torch.Tensor,
                           page_table: torch.Tensor, num_heads: int, scale: float, layout: str = "interleaved",
                           magnitude: float = 1.0, window: int = 0) -> torch.Tensor:
    """The same attention on tensor cores (bfloat16 pools), over the step's tile list for
    ``mma_tokens_per_tile(num_heads)`` tokens a tile.  Single tokens (the first tiles) have their
    keys cut into ranges that are merged by ``dsp_attn_combine``; portions of prompts run whole."""
    from dispec_b200.ops import attention as attn_ops
    num_pages, _, page_size, R = c_pool.shape
    r = r_pool.shape[3]
    T = q_absorbed.shape[0]
    tpt = mma_tokens_per_tile(num_heads)
    tile_seq, tile_tok0, n_tiles = ctx.attention_tiles[tpt]
    assert q_absorbed.dtype == torch.float32 and q_absorbed.stride(1) == 1 and q.stride(1) == 1
    assert c_pool.dtype == torch.bfloat16 and c_pool.is_contiguous() and r_pool.is_contiguous()
    out = torch.empty((T, num_heads * R), dtype=torch.bfloat16, device=q.device)
    lib = L.mixer_library("attn_latent")
    chunks = -(-num_heads // MMA_ROWS_PER_TILE)

    def launch(offset, count, splits, part_o, part_ml):
        L.check(lib.dsp_attn_latent_mma(
            L.ptr(q_absorbed), L.i64(q_absorbed.stride(0)), L.ptr(q), L.dtype_code(q.dtype), L.i64(q.stride(0)),
            q_head_stride, qr_off, L.ptr(inv_freq), rot, _LAYOUTS[layout], L.f32(magnitude), int(window),
            L.ptr(c_pool), L.ptr(r_pool), L.ptr(page_table),
            page_table.stride(0), L.ptr(ctx.q_start), L.ptr(ctx.ctx_len), L.ptr(tile_seq), L.ptr(tile_tok0), offset,
            count, L.ptr(out), L.i64(out.stride(0)), L.ptr(part_o), L.ptr(part_ml), splits, num_heads, tpt, R, r,
            page_size, num_pages, L.f32(scale), L.stream_handle()))

    n_dec = ctx.num_decode_seqs  # single tokens come first, one tile each
    if n_dec:
        keys = min(ctx.max_ctx_len, window + MMA_KEYS_PER_TILE) if window > 0 else ctx.max_ctx_len
        splits = choose_key_splits(n_dec, chunks, keys, q.device)
        if splits > 1:
            part_o, part_ml = attn_ops._partial_buffers(q.device, n_dec * num_heads, splits, R)
            launch(0, n_dec, splits, part_o, part_ml)
            L.check(L.core().dsp_attn_combine(L.ptr(part_o), L.ptr(part_ml), L.ptr(out), L.i64(out.stride(0)),
                                              n_dec, num_heads, R, splits, L.dtype_code(out.dtype), L.stream_handle()))
        else:
            launch(0, n_dec, 1, None, None)
    if n_tiles > n_dec:
        launch(n_dec, n_tiles - n_dec, 1, None, None)
    return out


def head_products_supported(x: torch.Tensor, head_stride: int, w: torch.Tensor) -> bool:
    """Whether ``head_products`` takes these operands: bfloat16, k in whole steps of 32, every
    head's block of x on 16-byte pieces."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[2] % 32 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and head_stride % 8 == 0 and x.data_ptr() % 16 == 0
            and (w.shape[1] * w.shape[2]) % 8 == 0 and w.is_contiguous())


def head_products(x: torch.Tensor, head_stride: int, w: torch.Tensor, out: torch.Tensor, out_head_stride: int,
                  gate: torch.Tensor | None = None) -> torch.Tensor:
    """out[:, h * out_head_stride : + N] = x[:, h * head_stride : + K] @ w[h].T for every head h of
    ``w`` [H, N, K] in one launch (bfloat16 operands, 32-bit accumulation; ``out`` float32 or
    bfloat16, any column offset baked into the tensors handed in).  ``gate`` (a matrix whose columns
    are laid out like ``out``'s): every result is multiplied by the sigmoid of its gate value."""
    assert head_products_supported(x, head_stride, w) and out.stride(1) == 1 and out.is_cuda
    H, N, K = w.shape
    lib = L.mixer_library("attn_latent")
    if gate is not None:
        assert gate.is_cuda and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape[0] == x.shape[0]
        assert gate.shape[1] >= (H - 1) * out_head_stride + N
    L.check(lib.dsp_head_products(L.ptr(x), L.i64(x.stride(0)), L.i64(head_stride), L.ptr(w), L.ptr(out),
                                  L.dtype_code(out.dtype), L.i64(out.stride(0)), L.i64(out_head_stride), x.shape[0],
                                  N, K, H, L.ptr(gate), L.dtype_code(gate.dtype) if gate is not None else 0,
                                  L.i64(gate.stride(0) if gate is not None else 0), L.stream_handle()))
    return out
