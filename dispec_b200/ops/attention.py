"""Causal grouped-query attention over the paged key/value cache."""
from __future__ import annotations

import ctypes

import torch

from dispec_b200.ops import library as L
from dispec_b200.ops import tuning
from dispec_b200.ops.tuning import CLUSTER_MAX_SPLITS

ROWS_PER_TILE = 64  # query rows (token, head-in-group pairs) one tensor-core tile holds
PREFILL_ROWS_PER_TILE = 128  # rows of a tile of the tcgen05 kernel for portions of prompts
DECODE_KERNEL_MAX_GROUP = 16  # query heads per KV head the warp-parallel single-token kernel holds


def tokens_per_tile(group_size: int) -> int | None:
    """Query tokens per tile of the tensor-core kernel (None: groups too large for it)."""
    if group_size > ROWS_PER_TILE:
        return None
    return ROWS_PER_TILE // group_size


def prefill_tokens_per_tile(group_size: int) -> int:
    """Query tokens per tile of the tcgen05 kernel for portions of prompts."""
    return PREFILL_ROWS_PER_TILE // group_size


def tcgen05_supported(head_dim: int, group_size: int, page_size: int, dtype: torch.dtype) -> bool:
    """The tcgen05 kernel is built for head sizes 64 and 128 and pages of 8 to 64 tokens."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128)
            and group_size <= ROWS_PER_TILE and page_size in (8, 16, 32, 64))


def paged_attention_generic(q: torch.Tensor, q_stride: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                            page_table: torch.Tensor, positions: torch.Tensor,
                            seq_of_token: torch.Tensor, out: torch.Tensor, num_heads: int,
                            num_kv_heads: int, head_dim: int, window: int, scale: float,
                            sink: bool = False, chunked: bool = False, sink_values: torch.Tensor | None = None,
                            turn_freq: torch.Tensor | None = None) -> torch.Tensor:
    """32-bit arithmetic kernel, any value size up to 512 and any group size.

    q: element (t, h, d) at q.data_ptr + (t * q_stride + h * D + d); out: [T, H * Dv], Dv being the
    width of the value pool (it may differ from the keys' D).
    The query at absolute position p = positions[t] sees keys max(0, p-window+1)..p
    (window 0: from 0) of sequence seq_of_token[t]; with ``chunked`` the keys of its own chunk of
    ``window`` positions, floor(p / window) * window .. p.  ``sink``: the softmax has one more key
    of score 0 and no value (weights exp(s_j) / (1 + sum exp(s_j))); with ``sink_values`` (float32
    [H]) that key's score is the head's own number, unscaled.  ``turn_freq`` (float32 [Dv/2]):
    every head's result is turned back, pair (m, m + Dv/2) by -p * turn_freq[m].
    """
    assert q.is_cuda and k_pool.is_cuda, "CUDA tensors only (there is no CPU path)"
    T = positions.shape[0]
    num_pages, kvh, page_size, d = k_pool.shape
    dv = v_pool.shape[3]
    assert (kvh, d) == (num_kv_heads, head_dim) and v_pool.shape[:3] == k_pool.shape[:3]
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and k_pool.dtype == q.dtype == v_pool.dtype
    assert out.is_contiguous() and out.shape == (T, num_heads * dv) and out.dtype in (q.dtype, torch.float32)
    assert page_table.dtype == torch.int32 and page_table.stride(1) == 1
    assert positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32
    _check_sink_turn(sink, sink_values, turn_freq, num_heads, dv)
    L.check(L.core().dsp_attn_generic(
        L.ptr(q), L.i64(q_stride), L.ptr(k_pool), L.ptr(v_pool), L.ptr(page_table),
        page_table.stride(0), L.ptr(positions), L.ptr(seq_of_token), L.ptr(out),
        L.i64(out.stride(0)), T, num_heads, num_kv_heads, head_dim, dv, page_size, num_pages,
        window, int(bool(chunked) and window > 0), L.f32(scale), int(bool(sink)), L.ptr(sink_values),
        L.ptr(turn_freq), L.dtype_code(q.dtype), L.dtype_code(out.dtype), L.stream_handle()))
    return out


def _check_sink_turn(sink, sink_values, turn_freq, num_heads: int, value_dim: int) -> None:
    if sink_values is not None:
        assert sink, "sink_values without a sink"
        assert sink_values.dtype == torch.float32 and sink_values.is_contiguous() and sink_values.shape == (num_heads,)
    if turn_freq is not None:
        assert value_dim % 2 == 0 and turn_freq.dtype == torch.float32 and turn_freq.is_contiguous()
        assert turn_freq.shape[0] >= value_dim // 2


_MMA_ERRORS = {1: "launch failed", 2: "unsupported head/group/split counts",
               3: "operands must be 16-byte aligned with strides in whole 16-byte pieces",
               4: "shared memory opt-in failed"}
_partials: dict = {}
_retired: list = []
_err_addr: dict = {}


def tensor_core_supported(head_dim: int, group_size: int, dtype: torch.dtype) -> bool:
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and group_size <= ROWS_PER_TILE)


def _partial_buffers(device, rows: int, splits: int, head_dim: int):
    """Scratch for split attention: unnormalised outputs and (max, sum) per row and split."""
    key = torch.device(device).index or 0
    need = rows * splits * (head_dim + 2)
    buf = _partials.get(key)
    if buf is None or buf.numel() < need:
        # a captured step keeps the address of the scratch it was captured with: a buffer that is
        # outgrown stays alive (sizes at least double, so all of them together stay below twice the last)
        if buf is not None:
            _retired.append(buf)
        buf = torch.empty(max(need, 1 << 20, 2 * (buf.numel() if buf is not None else 0)),
                          dtype=torch.float32, device=device)
        _partials[key] = buf
    n_o = rows * splits * head_dim
    return buf[:n_o], buf[n_o:n_o + rows * splits * 2]


def reserve_partials(device, rows: int, splits: int, head_dim: int) -> None:
    """Sizes the scratch ahead of time (before a CUDA graph is captured)."""
    _partial_buffers(device, rows, splits, head_dim)


def _device_error_address(device) -> int:
    key = torch.device(device).index or 0
    if key not in _err_addr:
        fn = L.core().dsp_device_error_address
        fn.restype = ctypes.c_ulonglong
        _err_addr[key] = int(fn())
    return _err_addr[key]


def choose_splits(num_decode_tiles: int, num_kv_heads: int, max_ctx: int, device=None) -> int:
    """Key splits for single-token rows on this device (see ``tuning.choose_splits``)."""
    return tuning.choose_splits(num_decode_tiles, num_kv_heads, max_ctx, tuning.attention_target_ctas(device))


def choose_outer(num_decode_tiles: int, num_kv_heads: int, max_ctx: int, splits: int, device=None) -> int:
    """Key ranges per single-token row beyond the cluster (see ``tuning.choose_outer``)."""
    return tuning.choose_outer(num_decode_tiles, num_kv_heads, max_ctx, splits,
                               tuning.attention_target_ctas(device))


def decode_rope_fusable(ctx, num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int,
                        dtype: torch.dtype) -> bool:
    """Whether the single tokens of this step go through the kernel that rotates q and k itself
    (then the separate rotation kernel must skip them)."""
    group = num_heads // num_kv_heads
    return (ctx.num_decode_seqs > 0 and tensor_core_supported(head_dim, group, dtype)
            and group <= DECODE_KERNEL_MAX_GROUP and tokens_per_tile(group) in ctx.attention_tiles
            and 0 < rotary_dim <= head_dim and rotary_dim % 16 == 0)


def _launch_mma(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq, tile_tok0,
                tile_offset, num_tiles, out, part_o, part_ml, H, KVH, D, tpt, window, splits, scale,
                cluster_combine=False, decode_only=False, fused_rope=None, outer=1):
    num_pages, _, page_size, _ = k_pool.shape
    lib = L.attention_library(D)
    fn = getattr(lib, f"dsp_attn_mma_d{D}")
    rc = fn(L.ptr(q), L.i64(q_stride), L.ptr(k_pool), L.ptr(v_pool), L.ptr(page_table),
            page_table.stride(0), L.ptr(q_start), L.ptr(ctx_len), L.ptr(tile_seq), L.ptr(tile_tok0),
            tile_offset, num_tiles, L.ptr(out), L.i64(out.stride(0)), L.ptr(part_o), L.ptr(part_ml),
            H, KVH, tpt, page_size, num_pages, window, splits, int(cluster_combine), int(decode_only),
            outer, L.f32(scale), L.ptr(fused_rope[0]) if fused_rope else None, fused_rope[1] if fused_rope else 0,
            1 if fused_rope else 0, int(fused_rope[2]) if fused_rope else 0,
            ctypes.c_void_p(_device_error_address(q.device)), L.stream_handle())
    L.LaunchCounter.n += 1
    if rc != 0:
        raise L.KernelError(f"dsp_attn_mma_d{D}: {_MMA_ERRORS.get(rc, rc)}")


def _launch_tcgen05(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq, tile_tok0,
                    tile_offset, num_tiles, out, H, KVH, D, tpt, window, scale):
    num_pages, _, page_size, _ = k_pool.shape
    lib = L.prefill_attention_library(D)
    fn = getattr(lib, f"dsp_attn_tcgen05_d{D}")
    rc = fn(L.ptr(q), L.i64(q_stride), L.ptr(k_pool), L.ptr(v_pool), L.ptr(page_table),
            page_table.stride(0), L.ptr(q_start), L.ptr(ctx_len), L.ptr(tile_seq), L.ptr(tile_tok0),
            tile_offset, num_tiles, L.ptr(out), L.i64(out.stride(0)), H, KVH, tpt, page_size, num_pages,
            window, L.f32(scale), ctypes.c_void_p(_device_error_address(q.device)), L.stream_handle())
    L.LaunchCounter.n += 1
    if rc != 0:
        raise L.KernelError(f"dsp_attn_tcgen05_d{D}: {_TCGEN05_ERRORS.get(rc, rc)}")


_TCGEN05_ERRORS = {1: "launch failed", 2: "unsupported head/group counts or page size",
                   3: "operands must be 16-byte aligned with strides in whole 16-byte pieces",
                   4: "shared memory opt-in or tensor map creation failed"}


def paged_attention_tiles(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq,
                          tile_tok0, num_tiles, num_decode_tiles, out, H, KVH, D, window, scale,
                          splits: int, prefill_tiles=None, fused_rope=None, outer: int = 1,
                          decode_kernel: bool | None = None) -> torch.Tensor:
    """Tensor-core attention over a tile list whose first ``num_decode_tiles`` tiles are single
    tokens (run with ``splits`` key splits and merged), the rest portions of prompts.  With
    ``prefill_tiles`` = (tile_seq, tile_tok0, num_tiles) of the 128-row tiling (single tokens
    first as well) the portions of prompts run on the tcgen05 kernel.  ``fused_rope`` = (inv_freq,
    rotary_dim, write_kv): ``q`` are the fused q/k/v rows and the single tokens' rows are not
    rotated yet; their kernel rotates them and stores key and value (see ``decode_rope_fusable``).
    ``outer`` > 1 cuts each single token's keys into that many ranges, each run by a cluster of
    ``splits`` CTAs; a second kernel merges the ranges (long contexts at small batches).
    ``decode_kernel``: whether single tokens take the warp-parallel kernel (default: whenever
    the group of query heads per KV head fits it) or the tile kernel."""
    assert q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and out.is_contiguous()
    tpt = tokens_per_tile(H // KVH)
    group = H // KVH
    if decode_kernel is None:
        decode_kernel = group <= DECODE_KERNEL_MAX_GROUP
    decode_kernel = decode_kernel and group <= DECODE_KERNEL_MAX_GROUP
    if num_decode_tiles > 0:
        if splits <= CLUSTER_MAX_SPLITS and (decode_kernel or splits > 1):
            # single tokens: the cluster kernels (warp-parallel keys when the group fits 16 rows)
            if outer > 1 and not decode_kernel:
                outer = 1
            part_o = part_ml = None
            if outer > 1:
                part_o, part_ml = _partial_buffers(q.device, num_decode_tiles * H, outer, D)
            _launch_mma(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq,
                        tile_tok0, 0, num_decode_tiles, out, part_o, part_ml, H, KVH, D, tpt, window,
                        splits, scale, cluster_combine=splits > 1, decode_only=decode_kernel,
                        fused_rope=fused_rope, outer=outer)
            if outer > 1:
                L.check(L.core().dsp_attn_combine(L.ptr(part_o), L.ptr(part_ml), L.ptr(out),
                                                  L.i64(out.stride(0)), num_decode_tiles, H, D, outer,
                                                  L.dtype_code(out.dtype), L.stream_handle()))
        elif fused_rope:
            raise L.KernelError("single tokens were left unrotated for a kernel that is not in use")
        elif splits > 1:
            rows = num_decode_tiles * H  # decode tokens are the first rows of the flat batch
            part_o, part_ml = _partial_buffers(q.device, rows, splits, D)
            _launch_mma(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq,
                        tile_tok0, 0, num_decode_tiles, out, part_o, part_ml, H, KVH, D, tpt, window,
                        splits, scale)
            L.check(L.core().dsp_attn_combine(L.ptr(part_o), L.ptr(part_ml), L.ptr(out),
                                              L.i64(out.stride(0)), num_decode_tiles, H, D, splits,
                                              L.dtype_code(out.dtype), L.stream_handle()))
        else:
            _launch_mma(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq,
                        tile_tok0, 0, num_decode_tiles, out, None, None, H, KVH, D, tpt, window, 1, scale)
    if prefill_tiles is not None:
        big_seq, big_tok0, big_n = prefill_tiles
        if big_n > num_decode_tiles:
            _launch_tcgen05(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, big_seq, big_tok0,
                            num_decode_tiles, big_n - num_decode_tiles, out, H, KVH, D,
                            prefill_tokens_per_tile(H // KVH), window, scale)
    elif num_tiles > num_decode_tiles:
        _launch_mma(q, q_stride, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq, tile_tok0,
                    num_decode_tiles, num_tiles - num_decode_tiles, out, None, None, H, KVH, D, tpt,
                    window, 1, scale)
    return out


def paged_attention_tensor_core(q, q_stride, k_pool, v_pool, page_table, positions, seq_of_token, out,
                                num_heads, num_kv_heads, head_dim, window, scale, q_lens, ctx_lens,
                                splits=None, decode_kernel=None, prefill_kernel=None) -> torch.Tensor:
    """Stand-alone form (tests, tools): builds the tile list for sequences given by their
    ``q_lens`` and ``ctx_lens`` (single-token sequences must come first).  ``prefill_kernel``
    "mma" keeps portions of prompts on the mma.sync kernel where the tcgen05 kernel would take
    them; ``decode_kernel`` False keeps single tokens on the tile kernel."""
    dev_ = q.device
    group = num_heads // num_kv_heads
    tpt = tokens_per_tile(group)

    def tile_list(per_tile):
        ts, t0, n_dec = [], [], 0
        for s, n in enumerate(q_lens):
            if n == 1 and n_dec == s:
                n_dec += 1
            for a in range(0, n, per_tile):
                ts.append(s)
                t0.append(a)
        return ts, t0, n_dec

    ts, t0, n_dec = tile_list(tpt)
    starts = [0]
    for n in q_lens:
        starts.append(starts[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev_)
    if splits is None:
        splits = choose_splits(n_dec, num_kv_heads, max(ctx_lens), q.device)
    prefill_tiles = None
    if prefill_kernel != "mma" and tcgen05_supported(head_dim, group, k_pool.shape[2], q.dtype):
        bs, b0, _ = tile_list(prefill_tokens_per_tile(group))
        prefill_tiles = (i32(bs), i32(b0), len(bs))
    return paged_attention_tiles(q, q_stride, k_pool, v_pool, page_table, i32(starts), i32(ctx_lens),
                                 i32(ts), i32(t0), len(ts), n_dec, out, num_heads, num_kv_heads,
                                 head_dim, window, scale, splits, prefill_tiles, decode_kernel=decode_kernel)


def paged_attention(ctx, q: torch.Tensor, q_stride: int, cache, out: torch.Tensor, num_heads: int,
                    num_kv_heads: int, head_dim: int, window: int, scale: float, fused_rope=None) -> torch.Tensor:
    """Attention of the step described by ``ctx`` over the layer cache ``cache``: the
    tensor-core kernel for bfloat16 where it is built for the sizes, the 32-bit kernel
    otherwise (and always on the float32 path)."""
    group = num_heads // num_kv_heads
    tpt = tokens_per_tile(group)
    if tensor_core_supported(head_dim, group, q.dtype) and tpt in ctx.attention_tiles:
        tile_seq, tile_tok0, num_tiles = ctx.attention_tiles[tpt]
        splits = ctx.decode_splits if ctx.decode_splits else choose_splits(
            ctx.num_decode_seqs, num_kv_heads, ctx.max_ctx_len, q.device)
        outer = ctx.decode_outer if ctx.decode_outer else choose_outer(
            ctx.num_decode_seqs, num_kv_heads, ctx.max_ctx_len, splits, q.device)
        prefill_tiles = None
        big = prefill_tokens_per_tile(group)
        if big in ctx.attention_tiles and tcgen05_supported(head_dim, group, cache.key_pool.shape[2], q.dtype):
            prefill_tiles = ctx.attention_tiles[big]
        return paged_attention_tiles(q, q_stride, cache.key_pool, cache.value_pool, cache.page_table,
                                     ctx.q_start, ctx.ctx_len, tile_seq, tile_tok0, num_tiles,
                                     ctx.num_decode_seqs, out, num_heads, num_kv_heads, head_dim,
                                     window, scale, splits, prefill_tiles, fused_rope, outer)
    if fused_rope:
        raise L.KernelError("single tokens were left unrotated for a kernel that is not in use")
    return paged_attention_generic(q, q_stride, cache.key_pool, cache.value_pool, cache.page_table,
                                   ctx.positions, ctx.seq_of_token, out, num_heads, num_kv_heads,
                                   head_dim, window, scale)


def qkv_rotate_store(qkv: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, cache,
                     inv_freq: torch.Tensor | None, rotary_dim: int, num_heads: int, num_kv_heads: int,
                     key_dim: int, value_dim: int, out_dtype: torch.dtype, v_other: torch.Tensor | None = None,
                     blend: torch.Tensor | None = None, q_norm: torch.Tensor | None = None,
                     k_norm: torch.Tensor | None = None, norm_eps: float = 0.0, v_norm: bool = False,
                     v_inv_freq: torch.Tensor | None = None, maps: int = 1,
                     q_temp: tuple | None = None) -> torch.Tensor:
    """From rows [q (H x Dk) | k (G x Dk) | v (G x Dv)] of a fused projection: turns pairs
    (i, i + rotary_dim/2) of every query and key head by position * inv_freq[i] in 32-bit, blends
    v <- (1 - blend) v + blend * v_other when ``v_other`` [T, G * Dv] is given (``blend``: a float32
    scalar on the device), stores key and value into the pages of ``cache`` (its "key" and "value"
    pools, of widths Dk and Dv) when the cache is written by this call, and returns the turned
    queries [T, H * Dk] in ``out_dtype``.  Rows with a negative position are skipped.

    ``q_norm`` / ``k_norm`` (float32 [Dk], one weight for all heads): every query / key head is
    divided by its root mean square (``norm_eps`` inside the root) and multiplied by the weight
    before it is turned.  ``v_norm``: every value head is divided by its root mean square (no
    weight).  ``v_inv_freq`` (float32 [Dv/2]): the value of position p is stored turned, pair
    (m, m + Dv/2) by p * v_inv_freq[m], after the norm.

    ``q_temp`` = (coef, every): every query is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).
    ``maps`` = M > 1: every query and key head has M parts of ``key_dim`` values, normed and turned
    each on its own (the row holds H * M query parts, G * M key parts and G values).  A key head is
    cached as its parts side by side (the "key" pool is M * Dk wide), and the queries come back as
    [T, H * M rows of M * Dk]: part m of head h, zero outside columns m * Dk .. (m + 1) * Dk, so that
    an attention with H * M query heads over the G cached key heads gives every part's map."""
    if not qkv.is_cuda:
        raise L.KernelError("qkv_rotate_store: CUDA tensors only (there is no CPU path)")
    T = qkv.shape[0]
    H, G, dk, dv = num_heads, num_kv_heads, key_dim, value_dim
    assert maps >= 1 and qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == (H + G) * maps * dk + G * dv
    k_pool, v_pool = cache.key_pool, cache.value_pool
    num_pages, g_, page_size, dk_ = k_pool.shape
    assert (g_, dk_) == (G, maps * dk) and v_pool.shape == (num_pages, G, page_size, dv)
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and k_pool.dtype == v_pool.dtype == out_dtype
    table = cache.page_table
    assert table.dtype == torch.int32 and table.stride(1) == 1
    if rotary_dim:
        assert inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.shape[0] >= rotary_dim // 2
    if v_other is not None:
        assert blend is not None and blend.dtype == torch.float32 and blend.numel() == 1 and blend.is_cuda
        assert v_other.shape == (T, G * dv) and v_other.stride(1) == 1
    for w in (q_norm, k_norm):
        assert w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.shape == (dk,))
    if v_inv_freq is not None:
        assert dv % 2 == 0 and v_inv_freq.dtype == torch.float32 and v_inv_freq.is_contiguous()
        assert v_inv_freq.shape[0] >= dv // 2
    q_out = torch.empty((T, H * maps * maps * dk), dtype=out_dtype, device=qkv.device)
    qt_coef, qt_every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    lib = L.mixer_library("attn_sink")
    L.check(lib.dsp_qkv_rotate_store(
        L.ptr(qkv), L.dtype_code(qkv.dtype), L.i64(qkv.stride(0)), L.ptr(positions), L.ptr(seq_of_token),
        L.ptr(table), table.stride(0), L.ptr(k_pool), L.ptr(v_pool), L.dtype_code(out_dtype), L.ptr(inv_freq),
        rotary_dim, L.ptr(v_other), L.dtype_code(v_other.dtype) if v_other is not None else 0,
        L.i64(v_other.stride(0) if v_other is not None else 0), L.ptr(blend if v_other is not None else None),
        L.ptr(q_norm), L.ptr(k_norm), L.f32(norm_eps), int(bool(v_norm)), L.ptr(v_inv_freq), L.ptr(q_out), L.i64(q_out.stride(0)), T, H, G, dk, dv, maps, L.f32(qt_coef), qt_every, page_size,
        num_pages, int(cache.write),
        L.stream_handle()))
    return q_out


SINK_ROWS_PER_TILE = 64  # query rows (token, head-in-group pairs) of a tile of the tensor-core kernel


def sink_mma_supported(group_size: int, key_dim: int, value_dim: int, dtype: torch.dtype = torch.bfloat16) -> bool:
    """The tensor-core kernel is compiled per pair of widths: multiples of 16, keys up to 256 and
    values up to 128 wide (the output accumulators live in registers), groups of up to 64 heads."""
    return (dtype == torch.bfloat16 and key_dim % 16 == 0 and value_dim % 16 == 0 and 16 <= key_dim <= 256
            and 16 <= value_dim <= 128 and group_size <= SINK_ROWS_PER_TILE)


def sink_tokens_per_tile(group_size: int, key_dim: int, value_dim: int):
    """Query tokens per tile that the tensor-core kernel of ``sink_paged_attention`` wants listed
    in the batch (None: the 32-bit kernel runs, which needs no tile list)."""
    if not sink_mma_supported(group_size, key_dim, value_dim):
        return None
    return SINK_ROWS_PER_TILE // group_size


def sink_choose_splits(num_single: int, num_kv_heads: int, keys: int, device=None) -> int:
    """Key splits for the single tokens of a step: enough blocks to fill the device, at least two
    key tiles of 64 a block, at most 16."""
    if num_single <= 0:
        return 1
    tiles = max(1, -(-keys // 64) + 1)
    want = -(-tuning.attention_target_ctas(device) // max(1, num_single * num_kv_heads))
    return max(1, min(16, tiles // 2, want))


def sink_attention_tiles(q, k_pool, v_pool, page_table, q_start, ctx_len, tile_seq, tile_tok0, num_tiles, out,
                         num_heads, num_kv_heads, window, scale, sink, num_single: int = 0, splits: int = 1,
                         chunked: bool = False, sink_values: torch.Tensor | None = None,
                         turn_freq: torch.Tensor | None = None, positions: torch.Tensor | None = None) -> torch.Tensor:
    """The tensor-core kernel over a tile list (``tokens per tile`` = 64 // group).  The first
    ``num_single`` tiles are single tokens (the first rows of the batch): with ``splits`` > 1
    their keys are cut into that many shares, merged by the combine kernel.  ``chunked``,
    ``sink_values``, ``turn_freq``: as in ``paged_attention_generic``; ``positions`` (of the step's
    tokens) is needed where split results are turned back."""
    num_pages, G, page_size, dk = k_pool.shape
    dv = v_pool.shape[3]
    assert q.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and q.stride(1) == 1 and out.stride(1) == 1
    fn = getattr(L.sink_attention_library(dk, dv), f"dsp_attn_sink_mma_k{dk}_v{dv}")
    tpt = SINK_ROWS_PER_TILE // (num_heads // num_kv_heads)
    _check_sink_turn(sink, sink_values, turn_freq, num_heads, dv)
    mask_mode = int(bool(chunked) and window > 0)

    def launch(offset, count, n_splits, part_o, part_ml):
        rc = fn(L.ptr(q), L.i64(q.stride(0)), L.ptr(k_pool), L.ptr(v_pool), L.ptr(page_table), page_table.stride(0),
                L.ptr(q_start), L.ptr(ctx_len), L.ptr(tile_seq), L.ptr(tile_tok0), offset, count, L.ptr(out),
                int(out.dtype == torch.float32), L.i64(out.stride(0)), num_heads, num_kv_heads, tpt, page_size, num_pages, window, mask_mode,
                L.f32(scale), int(bool(sink)), L.ptr(sink_values), L.ptr(turn_freq), n_splits, L.ptr(part_o), L.ptr(part_ml), ctypes.c_void_p(_device_error_address(q.device)),
                L.stream_handle())
        L.LaunchCounter.n += 1
        if rc != 0:
            raise L.KernelError(f"dsp_attn_sink_mma_k{dk}_v{dv}: {_MMA_ERRORS.get(rc, rc)}")

    first = 0
    if num_single > 0 and splits > 1:
        part_o, part_ml = _partial_buffers(q.device, num_single * num_heads, splits, dv)
        launch(0, num_single, splits, part_o, part_ml)
        if turn_freq is not None:
            assert positions is not None and positions.dtype == torch.int32
            L.check(L.mixer_library("attn_sink").dsp_attn_combine_turn(
                L.ptr(part_o), L.ptr(part_ml), L.ptr(out), L.dtype_code(out.dtype), L.i64(out.stride(0)),
                L.ptr(positions), L.ptr(turn_freq), num_single, num_heads, dv, splits, L.stream_handle()))
        else:
            L.check(L.core().dsp_attn_combine(L.ptr(part_o), L.ptr(part_ml), L.ptr(out), L.i64(out.stride(0)),
                                              num_single, num_heads, dv, splits, L.dtype_code(out.dtype),
                                              L.stream_handle()))
        first = num_single
    if num_tiles > first:
        launch(first, num_tiles - first, 1, None, None)
    return out


def sink_paged_attention(ctx, q: torch.Tensor, cache, out: torch.Tensor, num_heads: int, num_kv_heads: int,
                         key_dim: int, value_dim: int, window: int, scale: float, sink: bool, chunked: bool = False,
                         sink_values: torch.Tensor | None = None, turn_freq: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of the step over pools whose keys and values have widths of their own, with an
    optional sink in the softmax: q [T, H * Dk] (already turned), out [T, H * Dv] (of q's type, or
    float32 for a consumer that combines heads before it rounds).  bfloat16 runs
    on the tensor-core kernel where it is built for the sizes and the batch lists its tiles;
    everything else (and float32 always) on the 32-bit kernel.  ``chunked``: ``window`` is the
    size of the chunks a position's keys come from; ``sink_values``: the sink's score per head;
    ``turn_freq``: results are turned back by the query's position (``paged_attention_generic``)."""
    group = num_heads // num_kv_heads
    tpt = sink_tokens_per_tile(group, key_dim, value_dim)
    if q.dtype == torch.bfloat16 and tpt is not None and tpt in ctx.attention_tiles:
        tile_seq, tile_tok0, num_tiles = ctx.attention_tiles[tpt]
        keys = min(ctx.max_ctx_len, window) if window > 0 else ctx.max_ctx_len
        splits = sink_choose_splits(ctx.num_decode_seqs, num_kv_heads, keys, q.device)
        return sink_attention_tiles(q, cache.key_pool, cache.value_pool, cache.page_table, ctx.q_start, ctx.ctx_len,
                                    tile_seq, tile_tok0, num_tiles, out, num_heads, num_kv_heads, window, scale, sink,
                                    num_single=ctx.num_decode_seqs, splits=splits, chunked=chunked,
                                    sink_values=sink_values, turn_freq=turn_freq, positions=ctx.positions)
    return paged_attention_generic(q, q.stride(0), cache.key_pool, cache.value_pool, cache.page_table,
                                   ctx.positions, ctx.seq_of_token, out, num_heads, num_kv_heads, key_dim,
                                   window, scale, sink=sink, chunked=chunked, sink_values=sink_values,
                                   turn_freq=turn_freq)
