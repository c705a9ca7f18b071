// Kernels of the attention mixer whose keys and values have widths of their own, whose values
// may be blended with another layer's values of the same token, and whose softmax may carry a
// sink (one more key with a score of its own and no value).
//
// dsp_qkv_rotate_store: one block per token.  From a row [q (H x Dk) | k (G x Dk) | v (G x Dv)] of
// the fused projection (float or bfloat16) it
//   * with `q_norm_w` / `k_norm_w` (float [Dk], shared by the heads): divides every query / key
//     head by its root mean square (eps inside the root) and multiplies by the weight, before the
//     rotation,
//   * turns pairs (i, i + rot/2), i < rot/2, of every query and key head by the angle
//     position * inv_freq[i] (32-bit angles, sine and cosine) and leaves the other dimensions,
//   * blends v <- (1 - lambda) v + lambda v_other when `v_other` is given (lambda read from the
//     device), in 32-bit,
//   * with `v_norm`: divides every value head by its root mean square (no weight),
//   * with `v_inv_freq` (float [Dv/2]): turns pairs (m, m + Dv/2) of every value head by
//     position * v_inv_freq[m], after the norm (the attention kernel turns its result back by the
//     query's position, so that a value enters the sum turned by the distance),
//   * with `qt_every` > 0: multiplies every query by 1 + qt_coef * ln(floor((position + 1) / qt_every) + 1),
//   * writes the query to `q_out` [T, H * Dk] and the key and the value to the pages (pools
//     [num_pages, G, page_size, Dk] and [.., Dv]) in the pools' type.
// With `maps` = M > 1 every query and key head consists of M parts of Dk values that are normed and
// turned each on its own (the row holds H * M query parts, G * M key parts, G values): a key head is
// cached as its parts side by side (width M * Dk), and query part m of head h goes out as a row of
// M * Dk values that is zero outside part m, so that its product with the cached key head is the
// product of the two parts m and the M maps of a head read the same key and value rows.
// Everything between the loads and the stores is 32-bit.  A row with a negative position (padding
// of a captured step) is skipped; a page id outside the pool is recorded in the device error word
// and nothing is stored.
//
// dsp_attn_combine_turn: merges the partial results of split attention as attn_combine.cu does and
// turns pairs (m, m + D/2) of every merged head back by -position * inv_freq[m].
//
// dsp_attn_sink_mma_*: tensor-core attention over the same pools, see attn_sink_mma.cu.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256)
qkv_rotate_store_kernel(const void* __restrict__ qkv, int in_dtype, long ld, const int* __restrict__ positions,
                        const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int pt_stride,
                        void* __restrict__ k_pool, void* __restrict__ v_pool, int pool_dtype,
                        const float* __restrict__ inv_freq, int rot, const void* __restrict__ v_other, int vo_dtype,
                        long ld_vo, const float* __restrict__ lambda, const float* __restrict__ q_norm_w,
                        const float* __restrict__ k_norm_w, float norm_eps, int v_norm,
                        const float* __restrict__ v_inv_freq, void* __restrict__ q_out, long ld_q, int H,
                        int G, int Dk, int Dv, int maps, float qt_coef, int qt_every, int page_size, int num_pages,
                        int write_kv, int* err) {
  extern __shared__ float cs[];  // [rot/2] cosines, [rot/2] sines; [Dv/2] + [Dv/2] for the values; [H + 2 G] head factors
  const int t = blockIdx.x;
  const int pos = positions[t];
  if (pos < 0) return;
  const int half = rot / 2, vhalf = v_inv_freq ? Dv / 2 : 0;
  float* vcs = cs + rot;
  float* inv = vcs + 2 * vhalf;  // 1 / rms of head: queries, then keys, then values (1 where no norm is asked for)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &cs[half + i], &cs[i]);
  for (int i = threadIdx.x; i < vhalf; i += blockDim.x) sincosf((float)pos * v_inv_freq[i], &vcs[vhalf + i], &vcs[i]);
  const size_t row = (size_t)t * ld;
  const int G_v = G;
  H *= maps;  // from here on H and G count the parts of query and key heads
  G *= maps;
  const size_t k0 = row + (size_t)H * Dk, v0 = k0 + (size_t)G * Dk;
  const float q_temp = qt_every > 0 ? 1.f + qt_coef * logf((float)((pos + 1) / qt_every) + 1.f) : 1.f;
  for (int h = warp; h < H + G + G_v; h += warps) {
    const bool is_v = h >= H + G;
    const bool wanted = is_v ? v_norm != 0 : (h < H ? q_norm_w != nullptr : k_norm_w != nullptr);
    float r = 1.f;
    if (wanted) {  // (the same for the whole warp)
      const int n = is_v ? Dv : Dk;
      const size_t at = is_v ? v0 + (size_t)(h - H - G) * Dv : row + (size_t)h * Dk;
      float ss = 0.f;
      for (int i = lane; i < n; i += 32) {
        const float v = ld_any(qkv, in_dtype, at + i);
        ss = fmaf(v, v, ss);
      }
      r = 1.f / sqrtf(warp_sum(ss) / (float)n + norm_eps);
    }
    if (lane == 0) inv[h] = r;
  }
  __syncthreads();
  // element i of the head that starts at head0, normed (factor f, weight w) and turned
  auto turned = [&](size_t head0, int i, float f, const float* w) {
    const float v = ld_any(qkv, in_dtype, head0 + i) * f * (w ? w[i] : 1.f);
    if (i >= rot) return v;
    const int j = i < half ? i + half : i - half;
    const float o = ld_any(qkv, in_dtype, head0 + j) * f * (w ? w[j] : 1.f);
    return i < half ? v * cs[i] - o * cs[half + i] : v * cs[j] + o * cs[half + j];
  };
  if (maps == 1) {
    for (int idx = threadIdx.x; idx < H * Dk; idx += blockDim.x) {
      const int h = idx / Dk;
      st_any(q_out, pool_dtype, (size_t)t * ld_q + idx, turned(row + (size_t)h * Dk, idx % Dk, inv[h], q_norm_w) * q_temp);
    }
  } else {
    // the widened rows: zeros first (16 bytes a store where the row allows), then every part in its place
    const int wide = maps * Dk;
    const size_t esz = pool_dtype == DSP_BF16 ? 2 : 4, row_bytes = (size_t)H * wide * esz;
    char* qrow = reinterpret_cast<char*>(q_out) + (size_t)t * ld_q * esz;
    if (row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(qrow) % 16 == 0) {
      for (size_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(qrow)[i] = make_uint4(0, 0, 0, 0);
    } else {
      for (int idx = threadIdx.x; idx < H * wide; idx += blockDim.x) st_any(q_out, pool_dtype, (size_t)t * ld_q + idx, 0.f);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < H * Dk; idx += blockDim.x) {
      const int h = idx / Dk, i = idx % Dk;
      st_any(q_out, pool_dtype, (size_t)t * ld_q + (size_t)h * wide + (h % maps) * Dk + i,
             turned(row + (size_t)h * Dk, i, inv[h], q_norm_w) * q_temp);
    }
  }
  if (!write_kv) return;
  const int page = page_table[(size_t)seq_of_token[t] * pt_stride + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(err, DSP_ERR_BAD_PAGE);
    return;
  }
  for (int idx = threadIdx.x; idx < G * Dk; idx += blockDim.x) {
    const int g = idx / Dk, i = idx % Dk;  // part g of the key heads: part g % maps of head g / maps
    const size_t dst = (((size_t)page * G_v + g / maps) * page_size + pos % page_size) * (maps * Dk) + (g % maps) * Dk + i;
    st_any(k_pool, pool_dtype, dst, turned(k0 + (size_t)g * Dk, i, inv[H + g], k_norm_w));
  }
  const float lam = (v_other && lambda) ? *lambda : 0.f;
  auto value = [&](int g, int i) {
    float v = ld_any(qkv, in_dtype, v0 + (size_t)g * Dv + i);
    if (v_other) v = (1.f - lam) * v + lam * ld_any(v_other, vo_dtype, (size_t)t * ld_vo + (size_t)g * Dv + i);
    return v * inv[H + G + g];
  };
  for (int idx = threadIdx.x; idx < G_v * Dv; idx += blockDim.x) {
    const int g = idx / Dv, i = idx % Dv;
    float v = value(g, i);
    if (vhalf) {
      const int j = i < vhalf ? i + vhalf : i - vhalf;
      const float o = value(g, j);
      v = i < vhalf ? v * vcs[i] - o * vcs[vhalf + i] : v * vcs[j] + o * vcs[vhalf + j];
    }
    const size_t dst = (((size_t)page * G_v + g) * page_size + pos % page_size) * Dv + i;
    st_any(v_pool, pool_dtype, dst, v);
  }
}

// Merge of split attention (see attn_combine.cu) with the result turned back: one block per
// (token, head) row; the merged row is staged in shared memory, then pair (m, m + D/2) is turned
// by -position * inv_freq[m].
constexpr int TURN_MAX_SPLITS = 32;

__global__ void __launch_bounds__(128)
attn_combine_turn_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, void* __restrict__ out,
                         int out_dtype, long out_stride, const int* __restrict__ positions,
                         const float* __restrict__ inv_freq, int H, int D, int splits) {
  extern __shared__ float merged[];  // [D]
  const size_t row = blockIdx.x;  // t * H + h
  const size_t t = row / H;
  const int h = (int)(row % H);
  const int pos = positions[t];
  if (pos < 0) return;
  const int lane = threadIdx.x & 31;
  float m = -INFINITY, l = 0.f;
  if (lane < splits) {
    const float2 ml = reinterpret_cast<const float2*>(part_ml)[row * splits + lane];
    m = ml.x;
    l = ml.y;
  }
  const float M = warp_max(m);
  const float w = m == -INFINITY ? 0.f : exp2f(m - M);
  const float L = warp_sum(w * l);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  const float* po = part_o + row * splits * D;
  for (int d0 = (int)threadIdx.x - lane; d0 < D; d0 += blockDim.x) {  // the same trips for a whole warp (shuffles)
    const int d = d0 + lane;
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ws = __shfl_sync(0xffffffffu, w, s);
      // a split that saw no key has weight 0 and an output that was never written: not read
      if (d < D && ws != 0.f) acc += ws * po[(size_t)s * D + d];
    }
    if (d < D) merged[d] = acc * inv;
  }
  __syncthreads();
  const int half = inv_freq ? D / 2 : 0;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = merged[d];
    if (half) {
      const int mth = d < half ? d : d - half;
      float sn, cn;
      sincosf((float)pos * inv_freq[mth], &sn, &cn);
      // the inverse turn: (u, v) -> (u cos + v sin, v cos - u sin)
      v = d < half ? v * cn + merged[d + half] * sn : v * cn - merged[d - half] * sn;
    }
    st_any(out, out_dtype, t * out_stride + (size_t)h * D + d, v);
  }
}
}  // namespace

extern "C" int dsp_qkv_rotate_store(const void* qkv, int in_dtype, long ld, const int* positions,
                                    const int* seq_of_token, const int* page_table, int pt_stride, void* k_pool,
                                    void* v_pool, int pool_dtype, const float* inv_freq, int rot,
                                    const void* v_other, int vo_dtype, long ld_vo, const float* lambda,
                                    const float* q_norm_w, const float* k_norm_w, float norm_eps, int v_norm,
                                    const float* v_inv_freq, void* q_out,
                                    long ld_q, int T, int H, int G, int Dk, int Dv, int maps, float qt_coef,
                                    int qt_every, int page_size, int num_pages, int write_kv, cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(qkv && positions && q_out && H > 0 && G > 0 && Dk > 0 && Dv > 0, "dsp_qkv_rotate_store: missing operand");
  DSP_REQUIRE(maps >= 1 && qt_every >= 0, "dsp_qkv_rotate_store: maps=%d, qt_every=%d", maps, qt_every);
  DSP_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= Dk && (rot == 0 || inv_freq), "dsp_qkv_rotate_store: rot=%d for keys of %d", rot, Dk);
  DSP_REQUIRE(!write_kv || (k_pool && v_pool && page_table && seq_of_token && page_size > 0),
              "dsp_qkv_rotate_store: no pools to write to");
  DSP_REQUIRE(!v_other || lambda, "dsp_qkv_rotate_store: values to blend with but no weight");
  DSP_REQUIRE(!(v_other && v_norm), "dsp_qkv_rotate_store: values are blended or normed, not both");
  DSP_REQUIRE(!v_inv_freq || Dv % 2 == 0, "dsp_qkv_rotate_store: values of an odd width %d cannot be turned", Dv);
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_qkv_rotate_store: no device error word");
  const size_t smem = (size_t)(rot + (v_inv_freq ? Dv : 0) + (H + G) * maps + G) * sizeof(float);
  DSP_REQUIRE(smem <= 48 * 1024, "dsp_qkv_rotate_store: %d heads of %d and %d are more than the kernel holds", H, Dk, Dv);
  DSP_CUDA(launch_plain(qkv_rotate_store_kernel, dim3(T), dim3(256), smem, stream, qkv, in_dtype,
                        ld, positions, seq_of_token, page_table, pt_stride, k_pool, v_pool, pool_dtype, inv_freq, rot,
                        v_other, vo_dtype, ld_vo, lambda, q_norm_w, k_norm_w, norm_eps, v_norm, v_inv_freq, q_out, ld_q,
                        H, G, Dk, Dv, maps, qt_coef, qt_every, page_size, num_pages, write_kv, err));
  DSP_CHECK_LAUNCH("dsp_qkv_rotate_store");
  return 0;
}

extern "C" int dsp_attn_combine_turn(const float* part_o, const float* part_ml, void* out, int out_dtype,
                                     long out_stride, const int* positions, const float* inv_freq, int num_tokens,
                                     int H, int D, int splits, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  DSP_REQUIRE(part_o && part_ml && out && positions, "dsp_attn_combine_turn: missing operand");
  DSP_REQUIRE(splits >= 1 && splits <= TURN_MAX_SPLITS, "dsp_attn_combine_turn: splits=%d outside 1..%d", splits, TURN_MAX_SPLITS);
  DSP_REQUIRE(!inv_freq || D % 2 == 0, "dsp_attn_combine_turn: heads of an odd width %d cannot be turned", D);
  DSP_REQUIRE((size_t)D * sizeof(float) <= 48 * 1024, "dsp_attn_combine_turn: heads of %d are too wide", D);
  DSP_CUDA(launch_plain(attn_combine_turn_kernel, dim3(num_tokens * H), dim3(D >= 128 ? 128 : 64), (size_t)D * sizeof(float),
                        stream, part_o, part_ml, out, out_dtype, out_stride, positions, inv_freq, H, D, splits));
  DSP_CHECK_LAUNCH("dsp_attn_combine_turn");
  return 0;
}
