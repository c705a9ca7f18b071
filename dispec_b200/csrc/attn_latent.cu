// Attention over a cached latent, all arithmetic in 32-bit.
//
// Every token leaves two rows in the paged cache: a latent c of R values (already normalised)
// and one rotated key part of r values that all heads share.  A head's unrotated key and its
// value are linear maps of c, so neither is ever materialised: the caller folds the key map
// into the query (qa = Wk^T q, R values per head) and applies the value map to the result, and
// this kernel computes, per query token at position p and head h,
//
//     s_j = scale * (qa_h . c_j + rot(qr_h, p) . kr_j)        for every cached j <= p
//     out_h = sum_j softmax(s)_j c_j                           (R values)
//
// which is attention with ONE key/value head of key width R + r and value width R.
//
// latent_store_kernel: RMS norm (32-bit) of the first R columns of the down projection with a
// gain, rotation of the last r columns, both written to the token's place in the pages.  With
// `cq_out` it also writes the RMS norm of the query latent (columns q_off .. q_off + Qn, gain
// `q_gain`) of every row, padding rows included: the same block has the row at hand.
// The rotation turns pair i of the first `rot` of the r dimensions by the angle
// position * inv_freq[i]; the rest pass unchanged.  `layout` 0: pair i = (2i, 2i+1) (interleaved);
// 1: pair i = (i, i + rot/2) (halves).  Cosine and sine are multiplied by `mag` (a rotation that also
// stretches: both the query's and the key's part are, so their product carries mag^2).
// `window` W > 0: the query at position p sees the keys j with p - W < j <= p (0: every j <= p);
// older keys are never looked up, their pages may have been given back.
//
// pools: latent [num_pages, 1, page_size, R], rotated key [num_pages, 1, page_size, r];
// page = page_table[seq * pt_stride + position / page_size].
#include "common.cuh"

namespace {
constexpr int THREADS = 128;  // = keys per tile
constexpr int GCHUNK = 8;     // heads per block

// Element j (< rot) of a vector that is turned: which frequency, which element is its partner, and
// whether j is the second of the pair (u, v) -> (u c - v s, v c + u s).
struct PairOf {
  int freq, other;
  bool second;
};
__device__ __forceinline__ PairOf pair_of(int j, int rot, int layout) {
  if (layout == 0) return PairOf{j >> 1, j ^ 1, (j & 1) != 0};
  const int half = rot >> 1;
  return j < half ? PairOf{j, j + half, false} : PairOf{j - half, j - half, true};
}

__global__ void __launch_bounds__(THREADS)
latent_store_kernel(const void* __restrict__ down, int d_dtype, long ldd, int c_off, int r_off,
                    const float* __restrict__ gain, float eps, const float* __restrict__ inv_freq,
                    int rot, int layout, float mag, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                    const int* __restrict__ page_table, int pt_stride, void* __restrict__ c_pool,
                    void* __restrict__ r_pool, int pool_dtype, int R, int r, int page_size,
                    int num_pages, int q_off, int Qn, const float* __restrict__ q_gain,
                    void* __restrict__ cq_out, int cq_dtype, long ld_cq, int* err) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int pos = positions[t];
  if (cq_out) {
    const size_t qrow = (size_t)t * ldd + q_off;
    float qs = 0.f;
    for (int i = threadIdx.x; i < Qn; i += THREADS) {
      const float v = ld_any(down, d_dtype, qrow + i);
      qs = fmaf(v, v, qs);
    }
    const float qinv = 1.f / sqrtf(block_sum(qs, scratch) / (float)Qn + eps);
    for (int i = threadIdx.x; i < Qn; i += THREADS)
      st_any(cq_out, cq_dtype, (size_t)t * ld_cq + i, ld_any(down, d_dtype, qrow + i) * qinv * q_gain[i]);
    __syncthreads();  // the scratch of the sum is used again below
  }
  if (pos < 0) return;
  const int page = page_table[(size_t)seq_of_token[t] * pt_stride + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(err, DSP_ERR_BAD_PAGE);
    return;
  }
  const size_t place = (size_t)page * page_size + pos % page_size;
  const size_t row = (size_t)t * ldd;
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += THREADS) {
    const float v = ld_any(down, d_dtype, row + c_off + i);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)R + eps);
  for (int i = threadIdx.x; i < R; i += THREADS)
    st_any(c_pool, pool_dtype, place * R + i, ld_any(down, d_dtype, row + c_off + i) * inv * gain[i]);
  for (int i = threadIdx.x; i < r; i += THREADS) {
    float v = ld_any(down, d_dtype, row + r_off + i);
    if (i < rot) {
      const PairOf pr = pair_of(i, rot, layout);
      float sn, cs;
      sincosf((float)pos * inv_freq[pr.freq], &sn, &cs);
      sn *= mag;
      cs *= mag;
      const float other = ld_any(down, d_dtype, row + r_off + pr.other);
      v = pr.second ? v * cs + other * sn : v * cs - other * sn;
    }
    st_any(r_pool, pool_dtype, place * r + i, v);
  }
}

// One block per (query token, chunk of GCHUNK heads); a thread scores one key of the tile for
// every head of the chunk, then owns output dimensions tid, tid + 128, ...
template <typename T, int DPT>
__global__ void __launch_bounds__(THREADS)
attn_latent_kernel(const float* __restrict__ qa, long ldqa, const void* __restrict__ q, int q_dtype,
                   long ldq, int q_head_stride, int qr_off, const float* __restrict__ inv_freq, int rot,
                   int layout, float mag, int window, const T* __restrict__ c_pool, const T* __restrict__ r_pool,
                   const int* __restrict__ page_table, int pt_stride, const int* __restrict__ positions,
                   const int* __restrict__ seq_of_token, void* __restrict__ out, int out_dtype, long ldo,
                   int H, int R, int r, int page_size, int num_pages, float scale, int* err) {
  extern __shared__ float smem[];
  const int W = R + r;
  float* qs = smem;                        // [GCHUNK][W]
  float* ps = qs + GCHUNK * W;             // [GCHUNK][THREADS]
  long* place = (long*)(ps + GCHUNK * THREADS);  // [THREADS] row of each key in the pools
  __shared__ float red[GCHUNK][THREADS / 32];
  const int t = blockIdx.x, h0 = blockIdx.y * GCHUNK;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = positions[t];
  if (pos < 0) return;
  const int* table = page_table + (size_t)seq_of_token[t] * pt_stride;
  const int gn = min(GCHUNK, H - h0);

  for (int i = tid; i < gn * W; i += THREADS) {
    const int g = i / W, d = i % W;
    float v;
    if (d < R) {
      v = qa[(size_t)t * ldqa + (size_t)(h0 + g) * R + d];
    } else {
      const int j = d - R;
      const size_t at = (size_t)t * ldq + (size_t)(h0 + g) * q_head_stride + qr_off;
      v = ld_any(q, q_dtype, at + j);
      if (j < rot) {
        const PairOf pr = pair_of(j, rot, layout);
        float sn, cs;
        sincosf((float)pos * inv_freq[pr.freq], &sn, &cs);
        sn *= mag;
        cs *= mag;
        const float other = ld_any(q, q_dtype, at + pr.other);
        v = pr.second ? v * cs + other * sn : v * cs - other * sn;
      }
    }
    qs[i] = v * scale;
  }
  float m[GCHUNK], l[GCHUNK], acc[GCHUNK][DPT];
#pragma unroll
  for (int g = 0; g < GCHUNK; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DPT; ++j) acc[g][j] = 0.f;
  }
  __syncthreads();

  for (int kt = window > 0 ? max(0, pos - window + 1) : 0; kt <= pos; kt += THREADS) {
    const int key = kt + tid;
    float s[GCHUNK];
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) s[g] = -INFINITY;
    long at = -1;
    if (key <= pos) {
      const int page = table[key / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, DSP_ERR_BAD_PAGE);
      } else {
        at = (long)page * page_size + key % page_size;
        const T* cr = c_pool + at * R;
        const T* rr = r_pool + at * r;
#pragma unroll
        for (int g = 0; g < GCHUNK; ++g) s[g] = 0.f;
        for (int d = 0; d < R; ++d) {
          const float kv = to_f32(cr[d]);
#pragma unroll
          for (int g = 0; g < GCHUNK; ++g)
            if (g < gn) s[g] = fmaf(qs[g * W + d], kv, s[g]);
        }
        for (int d = 0; d < r; ++d) {
          const float kv = to_f32(rr[d]);
#pragma unroll
          for (int g = 0; g < GCHUNK; ++g)
            if (g < gn) s[g] = fmaf(qs[g * W + R + d], kv, s[g]);
        }
      }
    }
    place[tid] = at;
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      const float wm = warp_max(s[g]);
      if (lane == 0) red[g][warp] = wm;
    }
    __syncthreads();
    float alpha[GCHUNK], p[GCHUNK];
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      float tm = red[g][0];
#pragma unroll
      for (int w = 1; w < THREADS / 32; ++w) tm = fmaxf(tm, red[g][w]);
      const float m_new = fmaxf(m[g], tm);
      alpha[g] = (m_new == -INFINITY) ? 1.f : expf(m[g] - m_new);
      p[g] = (at >= 0 && g < gn) ? expf(s[g] - m_new) : 0.f;
      m[g] = m_new;
      ps[g * THREADS + tid] = p[g];
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      const float ws = warp_sum(p[g]);
      if (lane == 0) red[g][warp] = ws;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      float ts = red[g][0];
#pragma unroll
      for (int w = 1; w < THREADS / 32; ++w) ts += red[g][w];
      l[g] = l[g] * alpha[g] + ts;
#pragma unroll
      for (int j = 0; j < DPT; ++j) acc[g][j] *= alpha[g];
    }
    const int nkeys = min(THREADS, pos - kt + 1);
    for (int j = 0; j < nkeys; ++j) {
      const long vo = place[j];
      if (vo < 0) continue;
      const T* vr = c_pool + vo * R;
#pragma unroll
      for (int dd = 0; dd < DPT; ++dd) {
        const int d = tid + dd * THREADS;
        if (d < R) {
          const float vv = to_f32(vr[d]);
#pragma unroll
          for (int g = 0; g < GCHUNK; ++g)
            if (g < gn) acc[g][dd] = fmaf(ps[g * THREADS + j], vv, acc[g][dd]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int g = 0; g < GCHUNK; ++g) {
    if (g >= gn) continue;
    const float inv = l[g] > 0.f ? 1.f / l[g] : 0.f;
#pragma unroll
    for (int dd = 0; dd < DPT; ++dd) {
      const int d = tid + dd * THREADS;
      if (d < R) st_any(out, out_dtype, (size_t)t * ldo + (size_t)(h0 + g) * R + d, acc[g][dd] * inv);
    }
  }
}

template <typename T, int DPT>
int launch_attn(const float* qa, long ldqa, const void* q, int q_dtype, long ldq, int q_head_stride,
                int qr_off, const float* inv_freq, int rot, int layout, float mag, int window, const void* c_pool,
                const void* r_pool, const int* page_table, int pt_stride, const int* positions, const int* seq_of_token,
                void* out, int out_dtype, long ldo, int T_, int H, int R, int r, int page_size,
                int num_pages, float scale, int* err, cudaStream_t stream) {
  const size_t smem = (size_t)(GCHUNK * (R + r) + GCHUNK * THREADS) * sizeof(float) + THREADS * sizeof(long);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    DSP_CUDA(cudaFuncSetAttribute(attn_latent_kernel<T, DPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  dim3 grid(T_, (H + GCHUNK - 1) / GCHUNK);
  DSP_CUDA(launch_plain(attn_latent_kernel<T, DPT>, grid, dim3(THREADS), smem, stream, qa, ldqa, q, q_dtype,
                      ldq, q_head_stride, qr_off, inv_freq, rot, layout, mag, window, (const T*)c_pool, (const T*)r_pool,
                      page_table, pt_stride, positions, seq_of_token, out, out_dtype, ldo, H, R, r,
                      page_size, num_pages, scale, err));
  DSP_CHECK_LAUNCH("dsp_attn_latent");
  return 0;
}
}  // namespace

extern "C" int dsp_latent_store(const void* down, int d_dtype, long ldd, int c_off, int r_off,
                                const float* gain, float eps, const float* inv_freq, int rot, int layout,
                                float mag, const int* positions, const int* seq_of_token, const int* page_table,
                                int pt_stride, void* c_pool, void* r_pool, int pool_dtype, int T_, int R,
                                int r, int page_size, int num_pages, int q_off, int Qn, const float* q_gain,
                                void* cq_out, int cq_dtype, long ld_cq, cudaStream_t stream) {
  if (T_ == 0) return 0;
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_latent_store: no device error word");
  DSP_REQUIRE(down && gain && c_pool && r_pool && R > 0 && r >= 0, "dsp_latent_store: missing operand");
  DSP_REQUIRE(rot >= 0 && rot <= r && rot % 2 == 0 && (rot == 0 || inv_freq), "dsp_latent_store: rot=%d of %d", rot, r);
  DSP_REQUIRE(layout == 0 || layout == 1, "dsp_latent_store: unknown layout %d", layout);
  DSP_REQUIRE(!cq_out || (q_gain && Qn > 0 && q_off >= 0), "dsp_latent_store: a query latent without gain or size");
  DSP_CUDA(launch_plain(latent_store_kernel, dim3(T_), dim3(THREADS), 0, stream, down, d_dtype, ldd, c_off,
                      r_off, gain, eps, inv_freq, rot, layout, mag, positions, seq_of_token, page_table, pt_stride,
                      c_pool, r_pool, pool_dtype, R, r, page_size, num_pages, q_off, Qn, q_gain, cq_out, cq_dtype,
                      ld_cq, err));
  DSP_CHECK_LAUNCH("dsp_latent_store");
  return 0;
}

extern "C" int dsp_attn_latent(const float* qa, long ldqa, const void* q, int q_dtype, long ldq,
                               int q_head_stride, int qr_off, const float* inv_freq, int rot, int layout,
                               float mag, int window, const void* c_pool, const void* r_pool, int pool_dtype,
                               const int* page_table, int pt_stride, const int* positions,
                               const int* seq_of_token, void* out, int out_dtype, long ldo, int T_, int H,
                               int R, int r, int page_size, int num_pages, float scale,
                               cudaStream_t stream) {
  if (T_ == 0) return 0;
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_attn_latent: no device error word");
  DSP_REQUIRE(qa && q && c_pool && r_pool && out, "dsp_attn_latent: missing operand");
  DSP_REQUIRE(H > 0 && (H + GCHUNK - 1) / GCHUNK <= 65535, "dsp_attn_latent: H=%d", H);
  DSP_REQUIRE(R > 0 && R <= THREADS * 8, "dsp_attn_latent: latent size %d outside (0, %d]", R, THREADS * 8);
  DSP_REQUIRE(rot >= 0 && rot <= r && rot % 2 == 0 && (rot == 0 || inv_freq), "dsp_attn_latent: rot=%d of %d", rot, r);
  DSP_REQUIRE((layout == 0 || layout == 1) && window >= 0, "dsp_attn_latent: layout=%d window=%d", layout, window);
#define DSP_LATENT_ARGS qa, ldqa, q, q_dtype, ldq, q_head_stride, qr_off, inv_freq, rot, layout, mag, window, c_pool, r_pool, page_table, \
                        pt_stride, positions, seq_of_token, out, out_dtype, ldo, T_, H, R, r, page_size, num_pages,  \
                        scale, err, stream
  const int dpt = (R + THREADS - 1) / THREADS;
  if (pool_dtype == DSP_F32) {
    if (dpt <= 1) return launch_attn<float, 1>(DSP_LATENT_ARGS);
    if (dpt <= 2) return launch_attn<float, 2>(DSP_LATENT_ARGS);
    if (dpt <= 4) return launch_attn<float, 4>(DSP_LATENT_ARGS);
    return launch_attn<float, 8>(DSP_LATENT_ARGS);
  }
  if (pool_dtype == DSP_BF16) {
    if (dpt <= 1) return launch_attn<bf16, 1>(DSP_LATENT_ARGS);
    if (dpt <= 2) return launch_attn<bf16, 2>(DSP_LATENT_ARGS);
    if (dpt <= 4) return launch_attn<bf16, 4>(DSP_LATENT_ARGS);
    return launch_attn<bf16, 8>(DSP_LATENT_ARGS);
  }
#undef DSP_LATENT_ARGS
  DSP_REQUIRE(false, "dsp_attn_latent: unknown pool dtype %d", pool_dtype);
}

// ------------------------------------------------------------------- tensor cores (bfloat16)
// The same attention on mma.sync for bfloat16 pools: a CTA takes a tile of up to 64 query rows,
// a row being a (token, head) pair of ONE request: TPT consecutive tokens of its portion times
// HC heads (all of them up to 64).  Every head reads the same key row, so the tile shares each
// key tile it loads among all its rows.  Keys come in tiles of 32 through the page table
// (cp.async, two buffers); a key row is [latent R | rotated part r] in shared memory and its
// first R values are the value row as well.  16 warps = 4 row groups x 4 column groups:
//   S = Q K^T   warp (rg, cg) multiplies its 16 rows with all 32 keys over a quarter of the depth R + r;
//               the quarters are added in shared memory, where each warp picks up keys cg*8..
//   softmax     row maxima and sums of the four column groups meet in shared memory; P goes there
//               as bfloat16 (the sums are taken before the rounding)
//   O += P V    warp (rg, cg) owns the R / 4 output columns cg * R/4 .. of its rows
// The key tiles of a tile can be cut into `splits` ranges (grid.z), each leaving an unnormalised
// partial and (maximum in the base-2 domain, sum) per row for dsp_attn_combine: single tokens
// with long contexts then fill the device.  Keys beyond the tile's last position are never
// loaded (zero rows); a page id outside the pool is recorded and its rows are zero.
namespace tc {
constexpr int BM = 64, BN = 32, THREADS = 512, P_ROWB = 80, S_ROW = BN + 4;

struct Args {
  const float* qa; long ldqa;
  const void* q; int q_dtype; long ldq; int q_head_stride, qr_off;
  const float* inv_freq; int rot, layout; float mag; int window;
  const bf16* c_pool; const bf16* r_pool;
  const int* page_table; int pt_stride;
  const int* q_start; const int* ctx_len;
  const int* tile_seq; const int* tile_tok0; int tile_offset;
  bf16* out; long ldo;
  float* part_o; float* part_ml; int splits;
  int H, HC, TPT, R, r, page_size, num_pages;
  float scale_log2;
  int* err;
};

__device__ __forceinline__ void cp_async16(uint32_t smem, const void* gmem, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__host__ __device__ inline int key_row_bytes(int W) { return ((W * 2 + 127) / 128) * 128 + 16; }

// NT16: blocks of 16 output columns per warp = R / 64
template <int NT16>
__global__ void __launch_bounds__(THREADS, 1) attn_latent_mma_kernel(const Args p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int W = p.R + p.r, ROWB = key_row_bytes(W), CH = W / 8, CH_LAT = p.R / 8;
  const uint32_t q_s = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t k_s = q_s + BM * ROWB;
  const uint32_t p_s = k_s + 2 * BN * ROWB;
  float* red_max = reinterpret_cast<float*>(smem + (size_t)BM * ROWB + 2 * (size_t)BN * ROWB + BM * P_ROWB);  // [BM][4]
  float* red_sum = red_max + BM * 4;                                                                          // [BM][4]
  float* s_part = red_sum + BM * 4;  // [4][BM][S_ROW]: the column groups' partial scores
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rg = warp & 3, cg = warp >> 2;
  const int tile = blockIdx.x + p.tile_offset;
  const int seq = p.tile_seq[tile], tok0 = p.tile_tok0[tile];
  const int head0 = blockIdx.y * p.HC, hc = min(p.HC, p.H - head0);
  const int qs = p.q_start[seq], qlen = p.q_start[seq + 1] - qs, clen = p.ctx_len[seq];
  const int ntok = min(p.TPT, qlen - tok0), nrows = ntok * hc;
  const int pos0 = clen - qlen + tok0;
  if (clen <= 0 || pos0 < 0 || ntok <= 0) return;  // a padding row of a captured step
  const int hi = pos0 + ntok - 1;
  const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;  // the first key any row of the tile sees
  const int first = lo / BN, total = hi / BN + 1, per = (total - first + p.splits - 1) / p.splits;
  const int kb = first + blockIdx.z * per, ke = min(total, kb + per);
  const int* table = p.page_table + (size_t)seq * p.pt_stride;
  const int g = lane >> 2, c4 = lane & 3, m8 = lane >> 3, l8 = lane & 7;
  const int row_a = rg * 16 + g, row_b = row_a + 8;

  if (kb >= ke) {  // a key range with nothing in it: says so to the merge
    for (int m = tid; m < nrows; m += THREADS) {
      const size_t row = (size_t)(qs + tok0 + m / hc) * p.H + head0 + m % hc;
      p.part_ml[(row * p.splits + blockIdx.z) * 2] = -INFINITY;
      p.part_ml[(row * p.splits + blockIdx.z) * 2 + 1] = 0.f;
    }
    return;
  }

  // a warp copies whole key rows (two of the tile's 32): one page lookup and one division a row,
  // the lanes take the row's 16-byte pieces
  auto load_keys = [&](int kt, int buf) {
#pragma unroll
    for (int rr = 0; rr < BN / (THREADS / 32); ++rr) {
      const int row = warp + rr * (THREADS / 32);
      const int key = kt * BN + row;
      long at = -1;
      if (key <= hi && key >= lo) {
        const int page = table[key / p.page_size];
        if (page < 0 || page >= p.num_pages) {
          if (lane == 0) atomicOr(p.err, DSP_ERR_BAD_PAGE);
        } else {
          at = (long)page * p.page_size + key % p.page_size;
        }
      }
      const bool valid = at >= 0;
      const bf16* c_src = p.c_pool + (valid ? at : 0) * p.R;
      const bf16* r_src = p.r_pool + (valid ? at : 0) * p.r;
      const uint32_t dst = k_s + (buf * BN + row) * ROWB;
      for (int ch = lane; ch < CH; ch += 32)
        cp_async16(dst + ch * 16, ch < CH_LAT ? c_src + ch * 8 : r_src + (ch - CH_LAT) * 8, valid);
    }
    cp_async_commit();
  };
  load_keys(kb, 0);

  // the query rows as bfloat16: [absorbed query | rotated part], zero beyond the tile's rows;
  // a warp takes whole rows, its lanes pairs of values
  for (int m = warp; m < BM; m += THREADS / 32) {
    const bool real = m < nrows;
    const int tk = real ? m / hc : 0;
    const int t = qs + tok0 + tk, hd = head0 + (real ? m % hc : 0);
    const float* qa_row = p.qa + (size_t)t * p.ldqa + (size_t)hd * p.R;
    const size_t at = (size_t)t * p.ldq + (size_t)hd * p.q_head_stride + p.qr_off;
    for (int d = lane * 2; d < W; d += 64) {
      float v0 = 0.f, v1 = 0.f;
      if (real) {
        if (d < p.R) {
          const float2 v = *reinterpret_cast<const float2*>(qa_row + d);
          v0 = v.x;
          v1 = v.y;
        } else {
          const int j = d - p.R;
          v0 = ld_any(p.q, p.q_dtype, at + j);
          v1 = ld_any(p.q, p.q_dtype, at + j + 1);
          if (j < p.rot && p.layout == 0) {
            float sn, cs;
            sincosf((float)(pos0 + tk) * p.inv_freq[j >> 1], &sn, &cs);
            sn *= p.mag;
            cs *= p.mag;
            const float u = v0, w = v1;
            v0 = u * cs - w * sn;
            v1 = w * cs + u * sn;
          } else if (j < p.rot) {  // halves: each of the two elements with its partner in the other half
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const PairOf pr = pair_of(j + e, p.rot, 1);
              float sn, cs;
              sincosf((float)(pos0 + tk) * p.inv_freq[pr.freq], &sn, &cs);
              sn *= p.mag;
              cs *= p.mag;
              const float mine = e ? v1 : v0, other = ld_any(p.q, p.q_dtype, at + pr.other);
              const float turned = pr.second ? mine * cs + other * sn : mine * cs - other * sn;
              if (e) v1 = turned; else v0 = turned;
            }
          }
        }
      }
      *reinterpret_cast<uint32_t*>(smem + (size_t)m * ROWB + d * 2) = pack_bf16(v0, v1);
    }
  }

  float o[2 * NT16][4];
#pragma unroll
  for (int i = 0; i < 2 * NT16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int pos_a = row_a < nrows ? pos0 + row_a / hc : -1, pos_b = row_b < nrows ? pos0 + row_b / hc : -1;
  const int reach = p.window > 0 ? p.window : 0x40000000;

  for (int kt = kb; kt < ke; ++kt) {
    const int buf = (kt - kb) & 1;
    if (kt + 1 < ke) {
      load_keys(kt + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t kbuf = k_s + buf * BN * ROWB;
    // scores: warp (rg, cg) takes a quarter of the depth for all 32 keys of the tile (one query
    // fragment per four mma), the four partial blocks meet in shared memory
    float sp[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) sp[i][e] = 0.f;
    const int KS = W / 16, k_per = (KS + 3) / 4, k_lo = cg * k_per, k_hi = min(KS, k_lo + k_per);
    for (int kk = k_lo; kk < k_hi; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, q_s + (rg * 16 + (m8 & 1) * 8 + l8) * ROWB + (kk * 2 + (m8 >> 1)) * 16);
#pragma unroll
      for (int nn = 0; nn < 2; ++nn) {
        uint32_t b[4];
        ldmatrix_x4(b, kbuf + (nn * 16 + (m8 >> 1) * 8 + l8) * ROWB + (kk * 2 + (m8 & 1)) * 16);
        mma_bf16(sp[2 * nn], a, b[0], b[1]);
        mma_bf16(sp[2 * nn + 1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      *reinterpret_cast<float2*>(s_part + ((cg * BM + row_a) * S_ROW + nt * 8 + 2 * c4)) = make_float2(sp[nt][0], sp[nt][1]);
      *reinterpret_cast<float2*>(s_part + ((cg * BM + row_b) * S_ROW + nt * 8 + 2 * c4)) = make_float2(sp[nt][2], sp[nt][3]);
    }
    __syncthreads();
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // the quarters in a fixed order
      const float2 va = *reinterpret_cast<const float2*>(s_part + ((c * BM + row_a) * S_ROW + cg * 8 + 2 * c4));
      const float2 vb = *reinterpret_cast<const float2*>(s_part + ((c * BM + row_b) * S_ROW + cg * 8 + 2 * c4));
      s[0] += va.x;
      s[1] += va.y;
      s[2] += vb.x;
      s[3] += vb.y;
    }
    const int key0 = kt * BN + cg * 8 + 2 * c4;
    // a row sees the keys (its position - reach, its position]
    s[0] = (key0 <= pos_a && key0 > pos_a - reach) ? s[0] * p.scale_log2 : -INFINITY;
    s[1] = (key0 + 1 <= pos_a && key0 + 1 > pos_a - reach) ? s[1] * p.scale_log2 : -INFINITY;
    s[2] = (key0 <= pos_b && key0 > pos_b - reach) ? s[2] * p.scale_log2 : -INFINITY;
    s[3] = (key0 + 1 <= pos_b && key0 + 1 > pos_b - reach) ? s[3] * p.scale_log2 : -INFINITY;
    float tmax[2] = {fmaxf(s[0], s[1]), fmaxf(s[2], s[3])};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
    }
    if (c4 == 0) {
      red_max[row_a * 4 + cg] = tmax[0];
      red_max[row_b * 4 + cg] = tmax[1];
    }
    __syncthreads();
    float alpha[2], m_safe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float4 mx = *reinterpret_cast<const float4*>(red_max + (r == 0 ? row_a : row_b) * 4);
      const float m_new = fmaxf(m_run[r], fmaxf(fmaxf(mx.x, mx.y), fmaxf(mx.z, mx.w)));
      m_safe[r] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[r] = exp2f(m_run[r] - m_safe[r]);
      m_run[r] = m_new;
    }
    const float p0 = exp2f(s[0] - m_safe[0]), p1 = exp2f(s[1] - m_safe[0]);
    const float p2 = exp2f(s[2] - m_safe[1]), p3 = exp2f(s[3] - m_safe[1]);
    float psum[2] = {p0 + p1, p2 + p3};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
    }
    if (c4 == 0) {
      red_sum[row_a * 4 + cg] = psum[0];
      red_sum[row_b * 4 + cg] = psum[1];
    }
    unsigned char* pw = smem + (size_t)BM * ROWB + 2 * (size_t)BN * ROWB;
    *reinterpret_cast<uint32_t*>(pw + row_a * P_ROWB + (cg * 8 + 2 * c4) * 2) = pack_bf16(p0, p1);
    *reinterpret_cast<uint32_t*>(pw + row_b * P_ROWB + (cg * 8 + 2 * c4) * 2) = pack_bf16(p2, p3);
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float4 sm = *reinterpret_cast<const float4*>(red_sum + (r == 0 ? row_a : row_b) * 4);
      l_run[r] = l_run[r] * alpha[r] + ((sm.x + sm.y) + (sm.z + sm.w));
    }
#pragma unroll
    for (int i = 0; i < 2 * NT16; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int j = 0; j < BN / 16; ++j) {
      uint32_t a[4];
      ldmatrix_x4(a, p_s + (rg * 16 + (m8 & 1) * 8 + l8) * P_ROWB + (j * 2 + (m8 >> 1)) * 16);
#pragma unroll
      for (int dd = 0; dd < NT16; ++dd) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, kbuf + (j * 16 + (m8 & 1) * 8 + l8) * ROWB + ((cg * NT16 + dd) * 2 + (m8 >> 1)) * 16);
        mma_bf16(o[2 * dd], a, b[0], b[1]);
        mma_bf16(o[2 * dd + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int m = r == 0 ? row_a : row_b;
    if (m >= nrows) continue;
    const int t = qs + tok0 + m / hc, hd = head0 + m % hc;
    if (p.splits == 1) {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      bf16* dst = p.out + (size_t)t * p.ldo + (size_t)hd * p.R + cg * NT16 * 16 + 2 * c4;
#pragma unroll
      for (int i = 0; i < 2 * NT16; ++i)
        *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    } else {
      const size_t row = (size_t)t * p.H + hd;
      float* dst = p.part_o + (row * p.splits + blockIdx.z) * p.R + cg * NT16 * 16 + 2 * c4;
#pragma unroll
      for (int i = 0; i < 2 * NT16; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
      if (cg == 0 && c4 == 0) {
        p.part_ml[(row * p.splits + blockIdx.z) * 2] = m_run[r];
        p.part_ml[(row * p.splits + blockIdx.z) * 2 + 1] = l_run[r];
      }
    }
  }
}

template <int NT16>
int launch(const Args& a, int num_tiles, int head_chunks, cudaStream_t stream) {
  const int ROWB = key_row_bytes(a.R + a.r);
  const size_t smem = (size_t)BM * ROWB + 2 * (size_t)BN * ROWB + BM * P_ROWB + (2 * BM * 4 + 4 * BM * S_ROW) * sizeof(float);
  if (smem > 227 * 1024) return 2;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_latent_mma_kernel<NT16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return 4;
    configured = true;
  }
  if (launch_plain(attn_latent_mma_kernel<NT16>, dim3(num_tiles, head_chunks, a.splits), dim3(THREADS), smem, stream, a) != cudaSuccess)
    return 1;
  return 0;
}
}  // namespace tc

// Tiles tile_offset .. tile_offset + num_tiles - 1 of the tile list (TPT tokens a tile).  splits > 1:
// unnormalised partials go to part_o [rows, splits, R] and part_ml [rows, splits, 2], rows being
// flat token * H + head.  Sizes: R a multiple of 64 up to 512 (not 320 or 448), r a multiple of 16,
// row strides of qa in pairs of floats, pools and out in bfloat16.
extern "C" int dsp_attn_latent_mma(const float* qa, long ldqa, const void* q, int q_dtype, long ldq,
                                   int q_head_stride, int qr_off, const float* inv_freq, int rot, int layout,
                                   float mag, int window, const void* c_pool, const void* r_pool, const int* page_table,
                                   int pt_stride, const int* q_start, const int* ctx_len,
                                   const int* tile_seq, const int* tile_tok0, int tile_offset,
                                   int num_tiles, void* out, long ldo, float* part_o, float* part_ml,
                                   int splits, int H, int TPT, int R, int r, int page_size, int num_pages,
                                   float scale, cudaStream_t stream) {
  if (num_tiles == 0) return 0;
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_attn_latent_mma: no device error word");
  DSP_REQUIRE(R % 64 == 0 && r % 16 == 0 && r >= 0 && rot % 2 == 0 && rot <= r, "dsp_attn_latent_mma: R=%d r=%d rot=%d", R, r, rot);
  DSP_REQUIRE((layout == 0 || layout == 1) && window >= 0, "dsp_attn_latent_mma: layout=%d window=%d", layout, window);
  DSP_REQUIRE(ldqa % 2 == 0 && ((uintptr_t)qa % 8) == 0 && ldo % 2 == 0 && ((uintptr_t)out % 4) == 0 &&
              ((uintptr_t)c_pool % 16) == 0 && ((uintptr_t)r_pool % 16) == 0, "dsp_attn_latent_mma: operand alignment");
  DSP_REQUIRE(splits >= 1 && (splits == 1 || (part_o && part_ml)), "dsp_attn_latent_mma: splits=%d without scratch", splits);
  const int HC = H < tc::BM ? H : tc::BM;
  DSP_REQUIRE(TPT >= 1 && TPT * HC <= tc::BM, "dsp_attn_latent_mma: %d tokens x %d heads exceed a tile", TPT, HC);
  tc::Args a;
  a.qa = qa; a.ldqa = ldqa; a.q = q; a.q_dtype = q_dtype; a.ldq = ldq; a.q_head_stride = q_head_stride; a.qr_off = qr_off;
  a.inv_freq = inv_freq; a.rot = rot; a.layout = layout; a.mag = mag; a.window = window; a.c_pool = (const bf16*)c_pool; a.r_pool = (const bf16*)r_pool;
  a.page_table = page_table; a.pt_stride = pt_stride; a.q_start = q_start; a.ctx_len = ctx_len;
  a.tile_seq = tile_seq; a.tile_tok0 = tile_tok0; a.tile_offset = tile_offset;
  a.out = (bf16*)out; a.ldo = ldo; a.part_o = part_o; a.part_ml = part_ml; a.splits = splits;
  a.H = H; a.HC = HC; a.TPT = TPT; a.R = R; a.r = r; a.page_size = page_size; a.num_pages = num_pages;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.err = err;
  const int chunks = (H + HC - 1) / HC;
  int rc;
  switch (R / 64) {
    case 1: rc = tc::launch<1>(a, num_tiles, chunks, stream); break;
    case 2: rc = tc::launch<2>(a, num_tiles, chunks, stream); break;
    case 3: rc = tc::launch<3>(a, num_tiles, chunks, stream); break;
    case 4: rc = tc::launch<4>(a, num_tiles, chunks, stream); break;
    case 6: rc = tc::launch<6>(a, num_tiles, chunks, stream); break;
    case 8: rc = tc::launch<8>(a, num_tiles, chunks, stream); break;
    default: DSP_REQUIRE(false, "dsp_attn_latent_mma: latent size %d is not built", R);
  }
  DSP_REQUIRE(rc == 0, "dsp_attn_latent_mma: launch failed (%d)", rc);
  DSP_CHECK_LAUNCH("dsp_attn_latent_mma");
  return 0;
}

// ------------------------------------------------------ the per-head products around the attention
// C_h = A_h W_h^T for every head h in one launch (bfloat16 operands, 32-bit accumulation):
// folding the key map into the queries (A_h: the head's unrotated query part, W_h = Wk_h^T) and
// applying the value map to the attention's result (A_h: sum_j p_j c_j, W_h = Wv_h).  A_h and C_h
// are column blocks of row-major matrices (row strides lda / ldc, head strides a_hs / c_hs);
// W is [H, N, K] contiguous.  64 x 64 tiles, k in steps of 32, cp.async in two buffers, mma.sync.
// With `gate` (a row-major matrix laid out like C's columns) every result is multiplied by the
// sigmoid of its gate value before it is stored: an output gate on the heads.
namespace hp {
constexpr int BM = 64, BN = 64, BK = 32, THREADS = 128, ROWB = 80;

struct Args {
  const bf16* A; long lda, a_hs;
  const bf16* W;
  void* C; int c_dtype; long ldc, c_hs;
  int M, N, K;
  const void* gate; int g_dtype; long ldg;  // optional: C[m, h, n] *= sigmoid(gate[m * ldg + h * c_hs + n])
};

__global__ void __launch_bounds__(THREADS) head_products_kernel(const Args p) {
  __shared__ __align__(128) unsigned char sm[2][2][BM * ROWB];
  const int z = blockIdx.z, m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const bf16* A = p.A + (size_t)z * p.a_hs;
  const bf16* W = p.W + (size_t)z * p.N * p.K;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wm = warp & 1, wn = warp >> 1;
  const int g = lane >> 2, c4 = lane & 3, m8 = lane >> 3, l8 = lane & 7;
  auto load = [&](int kb, int buf) {
#pragma unroll
    for (int c = tid; c < BM * 4; c += THREADS) {
      const int row = c >> 2, ch = c & 3;
      const bool va = m0 + row < p.M, vw = n0 + row < p.N;
      const bf16* sa = va ? A + (size_t)(m0 + row) * p.lda + kb * BK + ch * 8 : A;
      const bf16* sw = vw ? W + (size_t)(n0 + row) * p.K + kb * BK + ch * 8 : W;
      tc::cp_async16((uint32_t)__cvta_generic_to_shared(&sm[buf][0][row * ROWB + ch * 16]), sa, va);
      tc::cp_async16((uint32_t)__cvta_generic_to_shared(&sm[buf][1][row * ROWB + ch * 16]), sw, vw);
    }
    tc::cp_async_commit();
  };
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
  const int nk = p.K / BK;
  load(0, 0);
  for (int kb = 0; kb < nk; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < nk) {
      load(kb + 1, buf ^ 1);
      tc::cp_async_wait<1>();
    } else {
      tc::cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t as = (uint32_t)__cvta_generic_to_shared(&sm[buf][0][0]);
    const uint32_t ws = (uint32_t)__cvta_generic_to_shared(&sm[buf][1][0]);
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
      uint32_t a[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        tc::ldmatrix_x4(a[i], as + (wm * 32 + i * 16 + (m8 & 1) * 8 + l8) * ROWB + (kk * 2 + (m8 >> 1)) * 16);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t b[4];
        tc::ldmatrix_x4(b, ws + (wn * 32 + j * 16 + (m8 >> 1) * 8 + l8) * ROWB + (kk * 2 + (m8 & 1)) * 16);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          tc::mma_bf16(acc[i][2 * j], a[i], b[0], b[1]);
          tc::mma_bf16(acc[i][2 * j + 1], a[i], b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = m0 + wm * 32 + i * 16 + g + (e >> 1) * 8;
        const int col = n0 + wn * 32 + j * 8 + 2 * c4 + (e & 1);
        if (row < p.M && col < p.N) {
          float v = acc[i][j][e];
          if (p.gate) v /= 1.f + expf(-ld_any(p.gate, p.g_dtype, (size_t)row * p.ldg + (size_t)z * p.c_hs + col));
          st_any(p.C, p.c_dtype, (size_t)row * p.ldc + (size_t)z * p.c_hs + col, v);
        }
      }
}
}  // namespace hp

extern "C" int dsp_head_products(const void* A, long lda, long a_hs, const void* W, void* C, int c_dtype,
                                 long ldc, long c_hs, int M, int N, int K, int H, const void* gate, int g_dtype,
                                 long ldg, cudaStream_t stream) {
  if (M == 0 || N == 0 || H == 0) return 0;
  DSP_REQUIRE(A && W && C && K > 0 && K % hp::BK == 0, "dsp_head_products: K=%d must be a positive multiple of %d", K, hp::BK);
  DSP_REQUIRE(lda % 8 == 0 && a_hs % 8 == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0 && ((long)N * K) % 8 == 0,
              "dsp_head_products: operands must lie on 16-byte pieces");
  DSP_REQUIRE(H <= 65535 && (M + hp::BM - 1) / hp::BM <= 65535, "dsp_head_products: grid too large");
  hp::Args a;
  a.A = (const bf16*)A; a.lda = lda; a.a_hs = a_hs; a.W = (const bf16*)W;
  a.C = C; a.c_dtype = c_dtype; a.ldc = ldc; a.c_hs = c_hs; a.M = M; a.N = N; a.K = K;
  a.gate = gate; a.g_dtype = g_dtype; a.ldg = ldg;
  DSP_CUDA(launch_plain(hp::head_products_kernel, dim3((N + hp::BN - 1) / hp::BN, (M + hp::BM - 1) / hp::BM, H),
                        dim3(hp::THREADS), 0, stream, a));
  DSP_CHECK_LAUNCH("dsp_head_products");
  return 0;
}
