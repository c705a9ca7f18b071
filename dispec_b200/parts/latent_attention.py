"""Attention whose keys and values are linear maps of a cached latent.

Queries go through a latent of their own: c_q = norm(W_dq h), q = W_uq c_q, laid out head by
head as [dim unrotated | rot_dim rotated].  W_dkv h gives the latent c (the first kv_rank rows,
RMS-normed) and ONE key part of rot_dim values that all heads share and that is rotated like
the queries' rotated parts.  Per head the unrotated key is W_uk c and the value W_uv c, the
score (q_plain . k_plain + q_rot . k_rot) * scale, softmax over the causal keys (with ``window``
W > 0: the keys j with p - W < j <= p), output W_o on the concatenated heads; with ``gate``
"element" the concatenated heads are first multiplied, element by element, by sigmoid(W_g h)
(the gate's rows ride in the down projections' product).  The rotation's pairs may be
interleaved or halves, and it may carry a magnitude (``Rotation``).

Only c and the rotated key part are cached (two named cache tensors of one head each), and
neither keys nor values are expanded: q_plain . (W_uk c) = (W_uk^T q_plain) . c, so the key
map is folded into the query (one small product per head) and the value map is applied to
sum_j p_j c_j (another).  The attention kernel then sees one shared key/value row per token.
"""
from __future__ import annotations

import torch

from dispec_b200 import ops
from dispec_b200.ops import latent as latent_ops
from dispec_b200.ops import norm32 as norm32_ops
from dispec_b200.parts.base import CacheNeed, CacheTensor, Mixer, TensorSpec
from dispec_b200.registry import register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 q_rank: int, scale: float, eps: float, position_encoding, window: int = 0, gate: str | None = None):
        if min(hidden_size, num_heads, dim, vdim, kv_rank, q_rank) <= 0 or rot_dim < 0:
            raise ValueError("sizes of a latent-attention mixer must be positive")
        if not float(scale) > 0.0:
            raise ValueError(f"the attention scale must be positive, got {scale}")
        self.hidden_size, self.num_heads, self.dim, self.rot_dim = hidden_size, num_heads, dim, rot_dim
        self.vdim, self.kv_rank, self.q_rank = vdim, kv_rank, q_rank
        self.scale, self.eps = float(scale), float(eps)
        self.position_encoding = position_encoding
        if window < 0 or gate not in (None, "element"):
            raise ValueError(f"latent_attention: window={window} / gate={gate!r} are not known")
        self.window, self.gate = int(window), gate

    def tensor_specs(self):
        h, H, d, r, dv, R, Q = (self.hidden_size, self.num_heads, self.dim, self.rot_dim, self.vdim,
                                self.kv_rank, self.q_rank)
        gain = dict(dtype="float32", init="one_plus_normal")
        specs = {"dq.weight": TensorSpec((Q, h)), "dq.norm": TensorSpec((Q,), **gain),
                 "uq.weight": TensorSpec((H * (d + r), Q)),
                 "dkv.weight": TensorSpec((R + r, h)), "dkv.norm": TensorSpec((R,), **gain),
                 "uk.weight": TensorSpec((H * d, R)), "uv.weight": TensorSpec((H * dv, R)),
                 "o.weight": TensorSpec((h, H * dv))}
        if self.gate:
            specs["g.weight"] = TensorSpec((H * dv, h))
        return specs

    def load(self, tensors):
        H, d, R = self.num_heads, self.dim, self.kv_rank
        # one product for both down projections (and the gate): [q latent | kv latent | shared key part | gate]
        rows = [tensors["dq.weight"], tensors["dkv.weight"]] + ([tensors["g.weight"]] if self.gate else [])
        self.w_down = torch.cat(rows, dim=0).contiguous()
        self.q_gain, self.c_gain = tensors["dq.norm"], tensors["dkv.norm"]
        self.w_uq = tensors["uq.weight"]
        # the key map of head h as the matrix of the product that folds it into the query:
        # qa_h = q_plain_h W_uk_h, i.e. x W^T with W = W_uk_h^T [R, d]
        self.w_uk_t = tensors["uk.weight"].view(H, d, R).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv.weight"].view(H, self.vdim, R).contiguous()
        self.w_o = tensors["o.weight"]

    def cache_need(self):
        return CacheNeed((CacheTensor("latent", 1, self.kv_rank), CacheTensor("rotated_key", 1, self.rot_dim)),
                         self.window)

    def tokens_per_attention_tile(self):
        return latent_ops.mma_tokens_per_tile(self.num_heads)

    def forward(self, ctx, x, cache, state):
        H, d, r, dv, R, Q = self.num_heads, self.dim, self.rot_dim, self.vdim, self.kv_rank, self.q_rank
        T = x.shape[0]
        rot = self.position_encoding.rotation()
        inv_freq, rot_n = (rot.inv_freq, rot.rotary_dim) if rot is not None else (None, 0)
        turn = dict(layout=rot.layout, magnitude=rot.magnitude) if rot is not None else {}
        scale = self.scale * self.position_encoding.score_scale()
        down = ops.linear(x, self.w_down, out_dtype=torch.float32)  # [T, Q | R | r]
        c_pool, r_pool = cache.tensors["latent"], cache.tensors["rotated_key"]
        if cache.write:  # the store's block has the row at hand: it norms the query latent as well
            cq = latent_ops.latent_store(down, Q, Q + R, self.c_gain, self.eps, inv_freq, rot_n, ctx.positions,
                                         ctx.seq_of_token, cache.page_table, c_pool, r_pool,
                                         query_latent=(0, Q, self.q_gain, x.dtype), **turn)
        else:
            cq = norm32_ops.sum_norm(down[:, :Q], self.q_gain, self.eps, out_dtype=x.dtype, want32=False)[1]
        q = ops.linear(cq, self.w_uq)  # [T, H * (d + r)]
        qa = torch.empty((T, H * R), dtype=torch.float32, device=x.device)
        if latent_ops.head_products_supported(q, d + r, self.w_uk_t):
            latent_ops.head_products(q, d + r, self.w_uk_t, qa, R)
        else:
            for a in range(H):
                ops.linear(q[:, a * (d + r):a * (d + r) + d], self.w_uk_t[a], out=qa[:, a * R:(a + 1) * R])
        if (latent_ops.mma_supported(R, r, c_pool.dtype)
                and latent_ops.mma_tokens_per_tile(H) in ctx.attention_tiles):
            mixed = latent_ops.latent_attention_tiles(ctx, qa, q, d + r, d, inv_freq, rot_n, c_pool, r_pool,
                                                      cache.page_table, H, scale, window=self.window, **turn)
        else:  # the 32-bit path, and sizes the tensor-core kernel is not built for
            mixed = latent_ops.latent_attention(qa, q, d + r, d, inv_freq, rot_n, c_pool, r_pool, cache.page_table,
                                                ctx.positions, ctx.seq_of_token, H, scale, x.dtype,
                                                window=self.window, **turn)
        heads = torch.empty((T, H * dv), dtype=x.dtype, device=x.device)
        gate = down[:, Q + R + r:] if self.gate else None
        if latent_ops.head_products_supported(mixed, R, self.w_uv):
            latent_ops.head_products(mixed, R, self.w_uv, heads, dv, gate=gate)  # the gate rides in the epilogue
        else:
            for a in range(H):
                ops.linear(mixed[:, a * R:(a + 1) * R], self.w_uv[a], out=heads[:, a * dv:(a + 1) * dv])
            if gate is not None:
                heads = norm32_ops.sigmoid_gate(heads, gate, x.dtype)
        return ops.linear(heads, self.w_o, out_dtype=torch.float32)
