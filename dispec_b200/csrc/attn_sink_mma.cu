// Tensor-core attention (mma.sync m16n8k16, bfloat16 operands, 32-bit scores, softmax and sums)
// over paged keys of width DSP_DK and values of width DSP_DV, with a sliding window or a chunked
// mask and an optional sink in the softmax (one more key with no value, of score 0 or, with
// `sink_values`, of the head's own unscaled score z: the running pair of the online softmax starts
// at (max, sum) = (z, 1) instead of (-inf, 0)).  With `turn_freq` every head's result is turned
// back, pair (m, m + DV/2) by -p * turn_freq[m] (values that were stored turned by their own
// positions).  Compiled per pair of widths.
//
// A block of four warps takes one tile of the step's tile list and one key/value head: up to 64
// query rows = (token, head of the group) pairs of one request, 16 rows a warp.  Keys come in
// tiles of 64 from the first key any row of the tile may see, two tiles in flight (cp.async);
// a key row is found through the request's page table, a page id outside the pool is recorded
// and its keys are hidden from every row.  The query at position p sees keys j with
// p - window < j <= p (window 0: every j <= p; mask_mode 1: the keys of p's own chunk of `window`
// positions, floor(p / window) * window <= j <= p); positions follow from the request's stored length
// (ctx_len) and the number of tokens it brings.  A request of length 0 (a padding row of a
// captured step) is skipped.
//
// Key splits (single tokens, whose one tile would otherwise walk its window alone): with
// splits > 1 the grid's z index takes a share of the tile's key tiles and leaves an unnormalised
// output with its (max, sum) in the scratch that attn_combine.cu merges; only split 0 starts from
// the sink's (z, 1), so the sink is counted once; the merged result is turned back there.
#include "common.cuh"

#ifndef DSP_DK
#error "compile with -DDSP_DK=<key width> -DDSP_DV=<value width>"
#endif

namespace {
constexpr int DK = DSP_DK, DV = DSP_DV;
constexpr int BM = 64, BN = 64, PAD = 8;  // BN key rows a tile: two of the block's 128 threads a row
constexpr int LDK = DK + PAD, LDV = DV + PAD;
static_assert(DK % 16 == 0 && DV % 16 == 0, "widths are multiples of 16");

__device__ __forceinline__ void cp16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void ldsm4_trans(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(128)
attn_sink_mma_kernel(const bf16* __restrict__ q, long ldq, const bf16* __restrict__ k_pool,
                     const bf16* __restrict__ v_pool, const int* __restrict__ page_table, int pt_stride,
                     const int* __restrict__ q_start, const int* __restrict__ ctx_len,
                     const int* __restrict__ tile_seq, const int* __restrict__ tile_tok0, void* __restrict__ out, int out_f32,
                     long ldo, int H, int G, int tpt, int page_size, int num_pages, int window, int mask_mode,
                     float scale_log2, int sink, const float* __restrict__ sink_values,
                     const float* __restrict__ turn_freq, int tile_offset, int splits,
                     float* __restrict__ part_o, float* __restrict__ part_ml, int* err) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);  // [BM][LDK]
  bf16* Ks = Qs + BM * LDK;                      // [2][BN][LDK]
  bf16* Vs = Ks + 2 * BN * LDK;                  // [2][BN][LDV]
  // the last tiles of a prompt have the most keys: they start first, so that short ones fill the tail
  const int tile = (int)(gridDim.x - 1 - blockIdx.x) + tile_offset, g = blockIdx.y, split = blockIdx.z;
  const int seq = tile_seq[tile], tok0 = tile_tok0[tile];
  const int qs = q_start[seq], qlen = q_start[seq + 1] - qs, clen = ctx_len[seq];
  if (clen <= 0 || tok0 >= qlen) return;
  const int group = H / G;
  const int nt = min(tpt, qlen - tok0), rows = nt * group;
  const int pos0 = clen - qlen + tok0, p1 = pos0 + nt - 1;
  // the first key a row at position p sees
  auto first_seen = [&](int p) {
    return window > 0 ? (mask_mode == 1 ? (p / window) * window : max(0, p - window + 1)) : 0;
  };
  const int lo = first_seen(pos0);
  const int nkt_all = (p1 - lo) / BN + 1;
  const int kt0 = (int)((long)nkt_all * split / splits), kt1 = (int)((long)nkt_all * (split + 1) / splits);
  const int nkt = kt1 - kt0;  // this block's key tiles: kt0 .. kt1 - 1 (none: it leaves an empty partial)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* table = page_table + (size_t)seq * pt_stride;

  for (int c = tid; c < BM * (DK / 8); c += 128) {
    const int r = c / (DK / 8), d = (c % (DK / 8)) * 8;
    bf16* dst = Qs + r * LDK + d;
    if (r < rows)
      cp16(dst, q + (size_t)(qs + tok0 + r / group) * ldq + (size_t)(g * group + r % group) * DK + d);
    else
      *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
  }
  // returns whether one of this thread's key rows had a page id outside the pool
  auto load = [&](int stage, int kt) {
    int bad = 0;
    const int j0 = lo + (kt0 + kt) * BN;
    bf16* ks = Ks + stage * BN * LDK;
    bf16* vs = Vs + stage * BN * LDV;
    // two threads a key row: the page is looked up once a row, the row's 16-byte pieces alternate
    const int r = tid >> 1;
    const int j = j0 + r;
    long row = -1;
    if (j <= p1) {
      const int page = table[j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, DSP_ERR_BAD_PAGE);
        bad = 1;
      } else {
        row = ((long)page * G + g) * page_size + j % page_size;
      }
    }
    const bf16* ksrc = k_pool + row * DK;
    const bf16* vsrc = v_pool + row * DV;
#pragma unroll
    for (int piece = (tid & 1); piece < DK / 8; piece += 2) {
      if (row >= 0)
        cp16(ks + r * LDK + piece * 8, ksrc + piece * 8);
      else
        *reinterpret_cast<uint4*>(ks + r * LDK + piece * 8) = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int piece = (tid & 1); piece < DV / 8; piece += 2) {
      if (row >= 0)
        cp16(vs + r * LDV + piece * 8, vsrc + piece * 8);
      else
        *reinterpret_cast<uint4*>(vs + r * LDV + piece * 8) = make_uint4(0, 0, 0, 0);
    }
    return bad;
  };
  int bad_now = nkt > 0 ? load(0, 0) : 0;
  asm volatile("cp.async.commit_group;\n");

  const int ra = warp * 16 + (lane >> 2), rb = ra + 8;  // the two rows of this thread's fragments
  const int pa = ra < rows ? pos0 + ra / group : -1, pb = rb < rows ? pos0 + rb / group : -1;
  const int la = first_seen(max(pa, 0)), lb = first_seen(max(pb, 0));
  float m[2], l[2], o[DV / 8][4];
  const bool with_sink = sink && split == 0;
  m[0] = m[1] = with_sink ? 0.f : -INFINITY;
  if (with_sink && sink_values) {  // the head's own score, in the base-2 domain of the scores
    if (ra < rows) m[0] = sink_values[g * group + ra % group] * 1.4426950408889634f;
    if (rb < rows) m[1] = sink_values[g * group + rb % group] * 1.4426950408889634f;
  }
  l[0] = l[1] = (with_sink && (lane & 3) == 0) ? 1.f : 0.f;
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int kt = 0; kt < nkt; ++kt) {
    const int st = kt & 1;
    __syncthreads();  // everyone has finished with the stage that is filled next
    const int bad_next = kt + 1 < nkt ? load(st ^ 1, kt + 1) : 0;
    asm volatile("cp.async.commit_group;\n");
    asm volatile("cp.async.wait_group 1;\n");
    const bool hide_all = __syncthreads_or(bad_now) != 0;  // a bad page hides the whole key tile from every row
    bad_now = bad_next;
    const bf16* ks = Ks + st * BN * LDK;
    const bf16* vs = Vs + st * BN * LDV;
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DK; kk += 16) {
      uint32_t a[4];
      ldsm4(a, Qs + (warp * 16 + (lane & 15)) * LDK + kk + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < BN / 8; j += 2) {
        uint32_t b[4];
        ldsm4(b, ks + (j * 8 + (lane & 7) + ((lane >> 4) << 3)) * LDK + kk + ((lane >> 3) & 1) * 8);
        mma16816(s[j], a, b[0], b[1]);
        mma16816(s[j + 1], a, b[2], b[3]);
      }
    }
    const int j0 = lo + (kt0 + kt) * BN;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < BN / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + i * 8 + (lane & 3) * 2 + (e & 1);
        const int p = e < 2 ? pa : pb;
        const bool seen = !hide_all && j <= p && j >= (e < 2 ? la : lb);
        s[i][e] = seen ? s[i][e] * scale_log2 : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[i][e]);
      }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m[h], mx[h]);
      alpha[h] = m_new == -INFINITY ? 1.f : exp2f(m[h] - m_new);
      m[h] = m_new;
      l[h] *= alpha[h];
    }
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int i = 0; i < BN / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mm = m[e >> 1];
        const float p = mm == -INFINITY ? 0.f : exp2f(s[i][e] - mm);
        s[i][e] = p;
        l[e >> 1] += p;
      }
#pragma unroll
    for (int kb = 0; kb < BN / 16; ++kb) {
      uint32_t a[4] = {pack2(s[2 * kb][0], s[2 * kb][1]), pack2(s[2 * kb][2], s[2 * kb][3]),
                       pack2(s[2 * kb + 1][0], s[2 * kb + 1][1]), pack2(s[2 * kb + 1][2], s[2 * kb + 1][3])};
#pragma unroll
      for (int i = 0; i < DV / 8; i += 2) {
        uint32_t b[4];
        ldsm4_trans(b, vs + (kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + i * 8 + (lane >> 4) * 8);
        mma16816(o[i], a, b[0], b[1]);
        mma16816(o[i + 1], a, b[2], b[3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n");
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h == 0 ? ra : rb;
    if (r >= rows) continue;
    const size_t token = (size_t)(qs + tok0 + r / group);
    const int head = g * group + r % group;
    if (splits > 1) {
      const size_t part = (token * H + head) * splits + split;
      float* dst = part_o + part * DV + (lane & 3) * 2;
#pragma unroll
      for (int i = 0; i < DV / 8; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
      if ((lane & 3) == 0) reinterpret_cast<float2*>(part_ml)[part] = make_float2(m[h], l[h]);
      continue;
    }
    const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
    if (turn_freq) {  // pair (d, d + DV/2) is held by this thread: o[i] and o[i + DV/16]
      const float p = (float)(h == 0 ? pa : pb);
#pragma unroll
      for (int i = 0; i < DV / 16; ++i)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float sn, cn;
          sincosf(p * turn_freq[i * 8 + (lane & 3) * 2 + e], &sn, &cn);
          const float u = o[i][2 * h + e], v = o[i + DV / 16][2 * h + e];
          o[i][2 * h + e] = u * cn + v * sn;  // the inverse turn
          o[i + DV / 16][2 * h + e] = v * cn - u * sn;
        }
    }
    if (out_f32) {  // 32-bit rows for a consumer that combines heads before it rounds
      float* dst = reinterpret_cast<float*>(out) + token * ldo + (size_t)head * DV + (lane & 3) * 2;
#pragma unroll
      for (int i = 0; i < DV / 8; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
      continue;
    }
    bf16* dst = reinterpret_cast<bf16*>(out) + token * ldo + (size_t)head * DV + (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < DV / 8; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8) = pack2(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
  }
}
}  // namespace

#define DSP_CAT_(a, b, c, d) a##b##c##d
#define DSP_CAT(a, b, c, d) DSP_CAT_(a, b, c, d)

// Returns 0, or: 1 launch failed, 2 unsupported sizes, 3 misaligned operands, 4 shared memory opt-in failed.
extern "C" int DSP_CAT(dsp_attn_sink_mma_k, DSP_DK, _v, DSP_DV)(
    const void* q, long ldq, const void* k_pool, const void* v_pool, const int* page_table, int pt_stride,
    const int* q_start, const int* ctx_len, const int* tile_seq, const int* tile_tok0, int tile_offset, int num_tiles,
    void* out, int out_f32, long ldo, int H, int G, int tpt, int page_size, int num_pages, int window, int mask_mode, float scale,
    int sink, const float* sink_values, const float* turn_freq, int splits, float* part_o, float* part_ml, int* err,
    cudaStream_t stream) {
  if (num_tiles == 0) return 0;
  if (G <= 0 || H % G || tpt <= 0 || tpt * (H / G) > BM || G > 65535 || page_size <= 0 || !err) return 2;
  if (mask_mode < 0 || mask_mode > 1) return 2;
  if (splits < 1 || splits > 32 || (splits > 1 && (!part_o || !part_ml))) return 2;
  if (((uintptr_t)q % 16) || ((uintptr_t)k_pool % 16) || ((uintptr_t)v_pool % 16) || ((uintptr_t)out % (out_f32 ? 8 : 4)) || ldq % 8 || ldo % 2)
    return 3;
  const size_t smem = sizeof(bf16) * ((size_t)BM * LDK + 2 * (size_t)BN * LDK + 2 * (size_t)BN * LDV);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_sink_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return 4;
    configured = true;
  }
  const cudaError_t e = launch_plain(attn_sink_mma_kernel, dim3(num_tiles, G, splits), dim3(128), smem, stream, (const bf16*)q, ldq,
                                     (const bf16*)k_pool, (const bf16*)v_pool, page_table, pt_stride, q_start, ctx_len,
                                     tile_seq, tile_tok0, out, out_f32, ldo, H, G, tpt, page_size, num_pages, window,
                                     mask_mode, scale * 1.4426950408889634f, sink, sink_values, turn_freq, tile_offset,
                                     splits, part_o, part_ml, err);
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : 1;
}
