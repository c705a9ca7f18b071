// Causal grouped-query attention over the paged key/value cache, all arithmetic in 32-bit.
//
// One block per (query token, KV head); the G = H / KVH query heads of the group share every
// key and value load.  The query at absolute position p sees keys b with
//     max(0, p - window + 1) <= b <= p        (window == 0: every key from 0)
// which is the lower-right aligned causal mask for a portion of a prompt on top of cached
// tokens, and a single decoded token alike.  Online softmax (running max m, running sum l)
// over tiles of 128 keys.  Keys have D dimensions and values Dv (the pools have their own widths).
// With `mask_mode` 1 the number `window` is a chunk size instead: position p sees the keys of its own
// chunk, floor(p / size) * size <= b <= p (chunks counted from position 0 of the sequence).
// With `sink` the softmax has one more, imaginary key and no value for it: the weights are
// exp(s_j) / (exp(z) + sum exp(s_j)), z = sink_values[head] (unscaled), or 0 without `sink_values`;
// the running pair starts at (m, l) = (z, 1) instead of (-inf, 0).
// With `turn_freq` (float [Dv/2]) the result of every head is turned back: pair (m, m + Dv/2) by
// -p * turn_freq[m] (the values were stored turned by their own positions).  Any head_dim that is a multiple of 4 (float) / 8 (bfloat16) up to
// 512, any G.  This kernel is the attention of the 32-bit path and the fallback of the
// bfloat16 path for head sizes the tensor-core kernel is not built for.
//
// q:   element (t, head, d) at q[t * q_stride + head * D + d]
// out: element (t, head, d) at out[t * out_stride + head * Dv + d]
// pools: [num_pages, KVH, page_size, D] (keys) and [..., Dv] (values); page = page_table[seq * pt_stride + b / page_size]
#include "common.cuh"

namespace {
constexpr int THREADS = 128;   // = keys per tile
constexpr int GCHUNK = 8;      // query heads handled per pass
constexpr int DPT = 4;         // output dims per thread: head_dim <= THREADS * DPT

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_generic_kernel(const T* __restrict__ q, long q_stride, const T* __restrict__ k_pool,
                    const T* __restrict__ v_pool, const int* __restrict__ page_table,
                    int pt_stride, const int* __restrict__ positions,
                    const int* __restrict__ seq_of_token, void* __restrict__ out, int out_dtype, long out_stride,
                    int H, int KVH, int D, int Dv, int page_size, int num_pages, int window, int mask_mode,
                    float scale, int sink, const float* __restrict__ sink_values,
                    const float* __restrict__ turn_freq, int* err) {
  extern __shared__ float smem[];
  float* qs = smem;                       // [GCHUNK][D]
  float* ps = qs + GCHUNK * D;            // [GCHUNK][THREADS]
  long* slot = (long*)(ps + GCHUNK * THREADS);  // [THREADS] row of each key in the pools (-1: none)
  float* os = (float*)(slot + THREADS);   // [GCHUNK][Dv] results before they are turned back (with turn_freq)
  __shared__ float red[GCHUNK][THREADS / 32];

  const int t = blockIdx.x, kvh = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = positions[t];
  if (pos < 0) return;
  const int seq = seq_of_token[t];
  const int G = H / KVH;
  const int lo = window > 0 ? (mask_mode == 1 ? (pos / window) * window : max(0, pos - window + 1)) : 0;
  const int hi = pos;
  const int* table = page_table + (size_t)seq * pt_stride;

  for (int g0 = 0; g0 < G; g0 += GCHUNK) {
    const int gn = min(GCHUNK, G - g0);
    __syncthreads();
    for (int i = tid; i < gn * D; i += THREADS) {
      const int g = i / D, d = i % D;
      qs[g * D + d] = to_f32(q[(size_t)t * q_stride + (size_t)(kvh * G + g0 + g) * D + d]) * scale;
    }
    float m[GCHUNK], l[GCHUNK], acc[GCHUNK][DPT];
#pragma unroll
    for (int g = 0; g < GCHUNK; ++g) {
      m[g] = sink ? ((sink_values && g < gn) ? sink_values[kvh * G + g0 + g] : 0.f) : -INFINITY;
      l[g] = sink ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < DPT; ++j) acc[g][j] = 0.f;
    }
    __syncthreads();

    for (int kt = lo; kt <= hi; kt += THREADS) {
      const int key = kt + tid;
      const bool valid = key <= hi;
      float s[GCHUNK];
#pragma unroll
      for (int g = 0; g < GCHUNK; ++g) s[g] = -INFINITY;
      long off = -1;
      if (valid) {
        const int page = table[key / page_size];
        if (page < 0 || page >= num_pages) {
          atomicOr(err, DSP_ERR_BAD_PAGE);
        } else {
          off = ((long)page * KVH + kvh) * page_size + (key % page_size);
          const T* kr = k_pool + off * D;
#pragma unroll
          for (int g = 0; g < GCHUNK; ++g) s[g] = 0.f;
          for (int d = 0; d < D; ++d) {
            const float kv = to_f32(kr[d]);
#pragma unroll
            for (int g = 0; g < GCHUNK; ++g)
              if (g < gn) s[g] = fmaf(qs[g * D + d], kv, s[g]);
          }
        }
      }
      slot[tid] = off;
      // tile maxima, one per head
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
        // m_new stays -inf only for heads beyond gn or when every page id was bad
        alpha[g] = (m_new == -INFINITY) ? 1.f : expf(m[g] - m_new);
        p[g] = (off >= 0 && g < gn) ? expf(s[g] - m_new) : 0.f;
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
      // weighted sum of values: thread owns dims tid, tid+128, ...
      const int nkeys = min(THREADS, hi - kt + 1);
      for (int j = 0; j < nkeys; ++j) {
        const long vo = slot[j];
        if (vo < 0) continue;
        const T* vr = v_pool + vo * Dv;
#pragma unroll
        for (int dd = 0; dd < DPT; ++dd) {
          const int d = tid + dd * THREADS;
          if (d < Dv) {
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
        if (d >= Dv) continue;
        if (turn_freq)
          os[g * Dv + d] = acc[g][dd] * inv;
        else
          st_any(out, out_dtype, (size_t)t * out_stride + (size_t)(kvh * G + g0 + g) * Dv + d, acc[g][dd] * inv);
      }
    }
    if (turn_freq) {
      __syncthreads();
      const int half = Dv / 2;
      for (int i = tid; i < gn * Dv; i += THREADS) {
        const int g = i / Dv, d = i % Dv;
        const int mth = d < half ? d : d - half;
        float sn, cn;
        sincosf((float)pos * turn_freq[mth], &sn, &cn);
        // the inverse turn: (u, v) -> (u cos + v sin, v cos - u sin)
        const float v = d < half ? os[i] * cn + os[i + half] * sn : os[i] * cn - os[i - half] * sn;
        st_any(out, out_dtype, (size_t)t * out_stride + (size_t)(kvh * G + g0 + g) * Dv + d, v);
      }
    }
  }
}
}  // namespace

extern "C" int dsp_attn_generic(const void* q, long q_stride, const void* k_pool,
                                const void* v_pool, const int* page_table, int pt_stride,
                                const int* positions, const int* seq_of_token, void* out,
                                long out_stride, int T, int H, int KVH, int D, int Dv, int page_size,
                                int num_pages, int window, int mask_mode, float scale, int sink,
                                const float* sink_values, const float* turn_freq, int dtype, int out_dtype,
                                cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(KVH > 0 && H % KVH == 0, "dsp_attn_generic: H=%d is not a multiple of KVH=%d", H, KVH);
  DSP_REQUIRE(D > 0 && Dv > 0 && Dv <= THREADS * DPT && D <= 4096,
              "dsp_attn_generic: key size %d or value size %d outside the kernel's range (values up to %d)", D, Dv,
              THREADS * DPT);
  DSP_REQUIRE(KVH <= 65535, "dsp_attn_generic: too many KV heads");
  DSP_REQUIRE(mask_mode == 0 || mask_mode == 1, "dsp_attn_generic: unknown mask mode %d", mask_mode);
  DSP_REQUIRE(!turn_freq || Dv % 2 == 0, "dsp_attn_generic: values of an odd width %d cannot be turned", Dv);
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_attn_generic: no device error word");
  const size_t smem = (size_t)(GCHUNK * D + GCHUNK * THREADS + (turn_freq ? GCHUNK * Dv : 0)) * sizeof(float) +
                      THREADS * sizeof(long);
  dim3 grid(T, KVH);
  if (dtype == DSP_F32) {
    static size_t configured = 0;
    if (smem > configured) {
      DSP_CUDA(cudaFuncSetAttribute(attn_generic_kernel<float>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured = smem;
    }
    attn_generic_kernel<float><<<grid, THREADS, smem, stream>>>(
        (const float*)q, q_stride, (const float*)k_pool, (const float*)v_pool, page_table, pt_stride,
        positions, seq_of_token, out, out_dtype, out_stride, H, KVH, D, Dv, page_size, num_pages, window,
        mask_mode, scale, sink, sink_values, turn_freq, err);
  } else if (dtype == DSP_BF16) {
    static size_t configured = 0;
    if (smem > configured) {
      DSP_CUDA(cudaFuncSetAttribute(attn_generic_kernel<bf16>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured = smem;
    }
    attn_generic_kernel<bf16><<<grid, THREADS, smem, stream>>>(
        (const bf16*)q, q_stride, (const bf16*)k_pool, (const bf16*)v_pool, page_table, pt_stride,
        positions, seq_of_token, out, out_dtype, out_stride, H, KVH, D, Dv, page_size, num_pages, window,
        mask_mode, scale, sink, sink_values, turn_freq, err);
  } else {
    DSP_REQUIRE(false, "dsp_attn_generic: unknown dtype %d", dtype);
  }
  DSP_CHECK_LAUNCH("dsp_attn_generic");
  return 0;
}
