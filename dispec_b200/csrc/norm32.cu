// Row-wise kernels around a residual stream that is kept in 32-bit floats: the RMS norm of a
// scaled sum (the arrangement with the norm after the sum), the per-head RMS norm with an
// optional gain and gate that closes a linear-attention mixer, and the xIELU activation.
// All arithmetic is 32-bit; each operand has its own storage type (float or bfloat16).
#include "common.cuh"

namespace {

// y = w * s / sqrt(mean(s^2) + eps),   s = alpha * x + delta   (delta optional)
// `rows` (optional) gathers input rows.  y goes to y32 (float) and/or y16 (any type); y32 may
// be x itself.  One block per row, the row held in shared memory between the two passes.
__global__ void __launch_bounds__(256)
sum_norm_kernel(const void* __restrict__ x, int x_dtype, long ldx, const void* __restrict__ delta,
                int d_dtype, long ldd, const float* __restrict__ w, float alpha, float eps,
                const int* __restrict__ rows, float* y32, long ld32, void* __restrict__ y16,
                int y_dtype, long ld16, int width) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const size_t in_row = rows ? (size_t)rows[r] : (size_t)r;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float s = alpha * ld_any(x, x_dtype, in_row * ldx + i);
    if (delta) s += ld_any(delta, d_dtype, in_row * ldd + i);
    row[i] = s;
    ss = fmaf(s, s, ss);
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(total / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float y = row[i] * inv * w[i];
    if (y32) y32[(size_t)r * ld32 + i] = y;
    if (y16) st_any(y16, y_dtype, (size_t)r * ld16 + i, y);
  }
}

// Per (token, head): y = o / sqrt(mean(o^2) + eps) * gain[j] * act(gate[t, head, j])
// (gain and gate optional; act is silu, or the logistic sigmoid when gate_kind is 1).
// o is float [T, H * dv]; one warp per (token, head).
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, long ldo, const float* __restrict__ gain,
                      const void* __restrict__ gate, int g_dtype, long ldg, void* __restrict__ y,
                      int y_dtype, long ldy, int T, int H, int dv, float eps, int gate_kind) {
  const int lane = threadIdx.x & 31;
  const long pair = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= (long)T * H) return;
  const int t = (int)(pair / H), h = (int)(pair % H);
  const float* row = o + (size_t)t * ldo + (size_t)h * dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss = fmaf(row[j], row[j], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)dv + eps);
  for (int j = lane; j < dv; j += 32) {
    float v = row[j] * inv;
    if (gain) v *= gain[j];
    if (gate) {
      const float g = ld_any(gate, g_dtype, (size_t)t * ldg + (size_t)h * dv + j);
      v *= (gate_kind == 1 ? 1.f : g) / (1.f + expf(-g));
    }
    st_any(y, y_dtype, (size_t)t * ldy + (size_t)h * dv + j, v);
  }
}

// The same for wide heads (a "head" may be the whole row): one block per (token, head).
__global__ void __launch_bounds__(256)
head_norm_gate_wide_kernel(const float* __restrict__ o, long ldo, const float* __restrict__ gain,
                           const void* __restrict__ gate, int g_dtype, long ldg, void* __restrict__ y,
                           int y_dtype, long ldy, int H, int dv, float eps, int gate_kind) {
  __shared__ float scratch[32];
  const int t = blockIdx.x / H, h = blockIdx.x % H;
  const float* row = o + (size_t)t * ldo + (size_t)h * dv;
  float ss = 0.f;
  for (int j = threadIdx.x; j < dv; j += blockDim.x) ss = fmaf(row[j], row[j], ss);
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)dv + eps);
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    float v = row[j] * inv;
    if (gain) v *= gain[j];
    if (gate) {
      const float g = ld_any(gate, g_dtype, (size_t)t * ldg + (size_t)h * dv + j);
      v *= (gate_kind == 1 ? 1.f : g) / (1.f + expf(-g));
    }
    st_any(y, y_dtype, (size_t)t * ldy + (size_t)h * dv + j, v);
  }
}

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// xIELU with the two raw parameters (p, q) read from the device:
//   z > 0:  softplus(p) z^2 + z / 2
//   z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
__global__ void __launch_bounds__(256)
xielu_kernel(const void* __restrict__ z, int z_dtype, long ldz, const float* __restrict__ pq,
             void* __restrict__ y, int y_dtype, long ldy, long rows, int cols) {
  const float ap = softplus_f(pq[0]), an = 0.5f + softplus_f(pq[1]);
  auto act = [&](float v) { return v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v); };
  // four elements a thread where rows are whole groups of four on 16-byte (8-byte) pieces
  const bool vec = z_dtype == DSP_F32 && y_dtype == DSP_BF16 && cols % 4 == 0 && ldz % 4 == 0 && ldy % 4 == 0 &&
                   ((uintptr_t)z % 16) == 0 && ((uintptr_t)y % 8) == 0;
  if (vec) {
    const int c4 = cols / 4;
    const long n = rows * c4;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
      const long r = i / c4;
      const int c = (int)(i % c4) * 4;
      const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(z) + (size_t)r * ldz + c);
      __nv_bfloat162 lo = __floats2bfloat162_rn(act(v.x), act(v.y)), hi = __floats2bfloat162_rn(act(v.z), act(v.w));
      uint2 out;
      out.x = *reinterpret_cast<uint32_t*>(&lo);
      out.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(y) + (size_t)r * ldy + c) = out;
    }
    return;
  }
  const long n = rows * cols;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long r = i / cols;
    const int c = (int)(i % cols);
    st_any(y, y_dtype, (size_t)r * ldy + c, act(ld_any(z, z_dtype, (size_t)r * ldz + c)));
  }
}

// Layer norm with a gain and no bias: y = (x - mean) / sqrt(var + eps) * w, var the mean of the
// squared deviations (two passes over the row held in shared memory).  `rows` gathers input rows.
__global__ void __launch_bounds__(256)
layer_norm_kernel(const void* __restrict__ x, int x_dtype, long ldx, const float* __restrict__ w, float eps,
                  const int* __restrict__ rows, void* __restrict__ y, int y_dtype, long ldy, int width) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const size_t in_row = rows ? (size_t)rows[r] : (size_t)r;
  float s = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = ld_any(x, x_dtype, in_row * ldx + i);
    row[i] = v;
    s += v;
  }
  const float mean = block_sum(s, scratch) / (float)width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float d = row[i] - mean;
    ss = fmaf(d, d, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    st_any(y, y_dtype, (size_t)r * ldy + i, (row[i] - mean) * inv * w[i]);
}

// One update of a 32-bit residual stream and, optionally, what the next reader wants of it:
//
//     x <- x + d,   d = y * scale[i] * sigmoid(gate)        (gate given: a gated, scaled sublayer)
//                   d = y / sqrt(mean(y^2) + eps) * rms_w   (rms_w given: an RMS-normed addend)
//                   d = y                                   (neither; y may be missing: d = 0)
//     and d += bias[i] when a row `bias` is given (the same for every row),
//     out = layer_norm(x) * norm_w  (norm_w given; with `norm_rms` the RMS norm
//           x / sqrt(mean(x^2) + eps) * norm_w instead)  or  x   (out given without norm_w)
//
// One block per row; the new row stays in shared memory between the passes.
__global__ void __launch_bounds__(256)
stream_update_kernel(float* __restrict__ x32, long ldx, const void* __restrict__ y, int y_dtype, long ldy,
                     const void* __restrict__ gate, int g_dtype, long ldg, const float* __restrict__ scale,
                     const float* __restrict__ rms_w, float rms_eps, const float* __restrict__ bias,
                     const float* __restrict__ norm_w, float norm_eps, int norm_rms, void* __restrict__ out,
                     int out_dtype, long ldo, int width) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const size_t r = blockIdx.x;
  float inv_rms = 1.f;
  if (rms_w) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      const float v = ld_any(y, y_dtype, r * ldy + i);
      ss = fmaf(v, v, ss);
    }
    inv_rms = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + rms_eps);
  }
  float s = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float d = y ? ld_any(y, y_dtype, r * ldy + i) : 0.f;
    if (gate) {
      const float g = ld_any(gate, g_dtype, r * ldg + i);
      d *= (scale ? scale[i] : 1.f) * (1.f / (1.f + expf(-g)));
    } else if (rms_w) {
      d *= inv_rms * rms_w[i];
    }
    if (bias) d += bias[i];
    const float v = x32[r * ldx + i] + d;
    x32[r * ldx + i] = v;
    row[i] = v;
    s += v;
  }
  if (!out) return;
  if (!norm_w) {
    __syncthreads();
    for (int i = threadIdx.x; i < width; i += blockDim.x) st_any(out, out_dtype, r * ldo + i, row[i]);
    return;
  }
  const float mean = norm_rms ? 0.f : block_sum(s, scratch) / (float)width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float d = row[i] - mean;
    ss = fmaf(d, d, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)width + norm_eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    st_any(out, out_dtype, r * ldo + i, (row[i] - mean) * inv * norm_w[i]);
}

// Gated linear unit with clamps: row = [gates | ups]; g = min(gate, limit), u = clamp(up, -limit, limit);
// y = g * sigmoid(alpha * g) * (u + 1).
__global__ void __launch_bounds__(256)
clamped_glu_kernel(const void* __restrict__ z, int z_dtype, long ldz, void* __restrict__ y, int y_dtype, long ldy,
                   long rows, int cols, float limit, float alpha) {
  const long n = rows * cols;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long r = i / cols;
    const int c = (int)(i % cols);
    const float g = fminf(ld_any(z, z_dtype, (size_t)r * ldz + c), limit);
    const float u = fminf(fmaxf(ld_any(z, z_dtype, (size_t)r * ldz + cols + c), -limit), limit);
    st_any(y, y_dtype, (size_t)r * ldy + c, g * (1.f / (1.f + expf(-alpha * g))) * (u + 1.f));
  }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// y[t, j] = gelu_tanh(z[t, j]) * table[ids[t], offset + j]: a gate on a per-token table row.
__global__ void __launch_bounds__(256)
gelu_table_gate_kernel(const void* __restrict__ z, int z_dtype, long ldz, const void* __restrict__ table,
                       int t_dtype, long ldt, int table_rows, int offset, const int* __restrict__ ids,
                       void* __restrict__ y, int y_dtype, long ldy, long rows, int cols, int* err) {
  const long n = rows * cols;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long r = i / cols;
    const int c = (int)(i % cols);
    const int id = ids[r];
    float e = 0.f;
    if (id < 0 || id >= table_rows)
      atomicOr(err, DSP_ERR_BAD_TOKEN);
    else
      e = ld_any(table, t_dtype, (size_t)id * ldt + offset + c);
    st_any(y, y_dtype, (size_t)r * ldy + c, gelu_tanh_f(ld_any(z, z_dtype, (size_t)r * ldz + c)) * e);
  }
}

// x <- cap * tanh(x / cap), in place on 32-bit rows.
__global__ void __launch_bounds__(256) softcap_kernel(float* x, long ldx, long rows, int cols, float cap) {
  const long n = rows * cols;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float* p = x + (size_t)(i / cols) * ldx + (i % cols);
    *p = cap * tanhf(*p / cap);
  }
}

// x <- x * s (float rows): a constant factor on the logits.
__global__ void __launch_bounds__(256) scale_rows_kernel(float* x, long ldx, long rows, int cols, float s) {
  const long n = rows * cols;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    x[(size_t)(i / cols) * ldx + (i % cols)] *= s;
}

// y[t, j] = x[t, j] * sigmoid(gate[t, j / per]): an output gate with one number for every `per`
// neighbouring columns (per 1: a gate per element; per = a head's width: a gate per head).
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(const void* __restrict__ x, int x_dtype, long ldx, const void* __restrict__ gate, int g_dtype,
                    long ldg, int per, void* __restrict__ y, int y_dtype, long ldy, long rows, int cols) {
  const long n = rows * cols;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long r = i / cols;
    const int c = (int)(i % cols);
    const float g = ld_any(gate, g_dtype, (size_t)r * ldg + c / per);
    st_any(y, y_dtype, (size_t)r * ldy + c, ld_any(x, x_dtype, (size_t)r * ldx + c) / (1.f + expf(-g)));
  }
}

// Differential heads.  a holds, per token, the results of `2 H` attention maps of width dv, the two
// maps of head h next to each other (h * 2, h * 2 + 1).  Per (token, head):
//   o = a1 - lambda * a2;  y = o / sqrt(mean(o^2) + eps) * post * sigmoid(gate[t, h])   (gate optional)
// One warp per (token, head).
__global__ void __launch_bounds__(128)
diff_heads_kernel(const void* __restrict__ a, int a_dtype, long lda, float lambda, float post, float eps,
                  const void* __restrict__ gate, int g_dtype, long ldg, void* __restrict__ y, int y_dtype, long ldy,
                  int T, int H, int dv) {
  const int lane = threadIdx.x & 31;
  const long pair = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= (long)T * H) return;
  const int t = (int)(pair / H), h = (int)(pair % H);
  const size_t a1 = (size_t)t * lda + (size_t)(2 * h) * dv, a2 = a1 + dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) {
    const float o = fmaf(-lambda, ld_any(a, a_dtype, a2 + j), ld_any(a, a_dtype, a1 + j));
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  float f = post / sqrtf(ss / (float)dv + eps);
  if (gate) f /= 1.f + expf(-ld_any(gate, g_dtype, (size_t)t * ldg + h));
  for (int j = lane; j < dv; j += 32) {
    const float o = fmaf(-lambda, ld_any(a, a_dtype, a2 + j), ld_any(a, a_dtype, a1 + j));
    st_any(y, y_dtype, (size_t)t * ldy + (size_t)h * dv + j, o * f);
  }
}

// out32[t] = table[ids[t]] * scale: the embedding as the first value of a 32-bit stream.
__global__ void __launch_bounds__(256)
embed_scaled_kernel(const void* __restrict__ table, int t_dtype, int table_rows, const int* __restrict__ ids,
                    float scale, float* __restrict__ out, long ldo, long rows, int cols, int* err) {
  const long n = rows * cols;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long r = i / cols;
    const int c = (int)(i % cols);
    const int id = ids[r];
    float v = 0.f;
    if (id < 0 || id >= table_rows)
      atomicOr(err, DSP_ERR_BAD_TOKEN);
    else
      v = ld_any(table, t_dtype, (size_t)id * cols + c) * scale;
    out[(size_t)r * ldo + c] = v;
  }
}

inline unsigned flat_grid(long n) {
  const int sms = dsp_num_sms();
  const long want = (n + 255) / 256, cap = (long)(sms > 0 ? sms : 148) * 16;
  return (unsigned)(want < cap ? want : cap);
}

inline int row_smem(const void* kernel, size_t smem, size_t* configured) {
  if (smem > *configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 1;
    *configured = smem;
  }
  return 0;
}
}  // namespace

extern "C" int dsp_sum_norm(const void* x, int x_dtype, long ldx, const void* delta, int d_dtype,
                            long ldd, const float* w, float alpha, float eps, const int* rows,
                            float* y32, long ld32, void* y16, int y_dtype, long ld16, int n_rows,
                            int width, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  DSP_REQUIRE(x && w && width > 0 && (y32 || y16), "dsp_sum_norm: missing operand");
  const size_t smem = (size_t)width * sizeof(float);
  DSP_REQUIRE(smem <= 200 * 1024, "dsp_sum_norm: a row of %d values does not fit shared memory", width);
  static size_t configured = 48 * 1024;
  if (smem > configured) {
    DSP_CUDA(cudaFuncSetAttribute(sum_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  DSP_CUDA(launch_plain(sum_norm_kernel, dim3(n_rows), dim3(256), smem, stream, x, x_dtype, ldx, delta,
                      d_dtype, ldd, w, alpha, eps, rows, y32, ld32, y16, y_dtype, ld16, width));
  DSP_CHECK_LAUNCH("dsp_sum_norm");
  return 0;
}

extern "C" int dsp_head_norm_gate(const float* o, long ldo, const float* gain, const void* gate,
                                  int g_dtype, long ldg, void* y, int y_dtype, long ldy, int T, int H,
                                  int dv, float eps, int gate_kind, cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(o && y && H > 0 && dv > 0, "dsp_head_norm_gate: missing operand");
  DSP_REQUIRE(gate_kind == 0 || gate_kind == 1, "dsp_head_norm_gate: unknown gate kind %d", gate_kind);
  const long pairs = (long)T * H;
  if (dv >= 512) {
    DSP_CUDA(launch_plain(head_norm_gate_wide_kernel, dim3((unsigned)pairs), dim3(256), 0, stream, o, ldo, gain, gate,
                          g_dtype, ldg, y, y_dtype, ldy, H, dv, eps, gate_kind));
    DSP_CHECK_LAUNCH("dsp_head_norm_gate");
    return 0;
  }
  DSP_CUDA(launch_plain(head_norm_gate_kernel, dim3((unsigned)((pairs + 3) / 4)), dim3(128), 0, stream, o,
                      ldo, gain, gate, g_dtype, ldg, y, y_dtype, ldy, T, H, dv, eps, gate_kind));
  DSP_CHECK_LAUNCH("dsp_head_norm_gate");
  return 0;
}

extern "C" int dsp_xielu(const void* z, int z_dtype, long ldz, const float* pq, void* y, int y_dtype,
                         long ldy, long rows, int cols, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  DSP_REQUIRE(z && pq && y, "dsp_xielu: missing operand");
  const long n = rows * cols;
  const int sms = dsp_num_sms();
  const long want = (n + 255) / 256, cap = (long)(sms > 0 ? sms : 148) * 16;
  DSP_CUDA(launch_plain(xielu_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), 0, stream, z,
                      z_dtype, ldz, pq, y, y_dtype, ldy, rows, cols));
  DSP_CHECK_LAUNCH("dsp_xielu");
  return 0;
}

extern "C" int dsp_layer_norm(const void* x, int x_dtype, long ldx, const float* w, float eps, const int* rows,
                              void* y, int y_dtype, long ldy, int n_rows, int width, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  DSP_REQUIRE(x && w && y && width > 0, "dsp_layer_norm: missing operand");
  const size_t smem = (size_t)width * sizeof(float);
  DSP_REQUIRE(smem <= 200 * 1024, "dsp_layer_norm: a row of %d values does not fit shared memory", width);
  static size_t configured = 48 * 1024;
  DSP_REQUIRE(row_smem((const void*)layer_norm_kernel, smem, &configured) == 0, "dsp_layer_norm: shared memory opt-in failed");
  DSP_CUDA(launch_plain(layer_norm_kernel, dim3(n_rows), dim3(256), smem, stream, x, x_dtype, ldx, w, eps, rows, y,
                        y_dtype, ldy, width));
  DSP_CHECK_LAUNCH("dsp_layer_norm");
  return 0;
}

extern "C" int dsp_stream_update(float* x32, long ldx, const void* y, int y_dtype, long ldy, const void* gate,
                                 int g_dtype, long ldg, const float* scale, const float* rms_w, float rms_eps,
                                 const float* bias, const float* norm_w, float norm_eps, int norm_rms, void* out,
                                 int out_dtype, long ldo, int n_rows, int width, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  DSP_REQUIRE(x32 && width > 0, "dsp_stream_update: missing operand");
  DSP_REQUIRE(y || (!gate && !rms_w), "dsp_stream_update: a gate or a norm but no addend");
  DSP_REQUIRE(!(gate && rms_w), "dsp_stream_update: an addend is gated or RMS-normed, not both");
  const size_t smem = (size_t)width * sizeof(float);
  DSP_REQUIRE(smem <= 200 * 1024, "dsp_stream_update: a row of %d values does not fit shared memory", width);
  static size_t configured = 48 * 1024;
  DSP_REQUIRE(row_smem((const void*)stream_update_kernel, smem, &configured) == 0, "dsp_stream_update: shared memory opt-in failed");
  DSP_CUDA(launch_plain(stream_update_kernel, dim3(n_rows), dim3(256), smem, stream, x32, ldx, y, y_dtype, ldy, gate,
                        g_dtype, ldg, scale, rms_w, rms_eps, bias, norm_w, norm_eps, norm_rms, out, out_dtype, ldo, width));
  DSP_CHECK_LAUNCH("dsp_stream_update");
  return 0;
}

extern "C" int dsp_clamped_glu(const void* z, int z_dtype, long ldz, void* y, int y_dtype, long ldy, long rows,
                               int cols, float limit, float alpha, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  DSP_REQUIRE(z && y, "dsp_clamped_glu: missing operand");
  DSP_CUDA(launch_plain(clamped_glu_kernel, dim3(flat_grid(rows * cols)), dim3(256), 0, stream, z, z_dtype, ldz, y,
                        y_dtype, ldy, rows, cols, limit, alpha));
  DSP_CHECK_LAUNCH("dsp_clamped_glu");
  return 0;
}

extern "C" int dsp_gelu_table_gate(const void* z, int z_dtype, long ldz, const void* table, int t_dtype, long ldt,
                                   int table_rows, int offset, const int* ids, void* y, int y_dtype, long ldy,
                                   long rows, int cols, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  DSP_REQUIRE(z && table && ids && y, "dsp_gelu_table_gate: missing operand");
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_gelu_table_gate: no device error word");
  DSP_CUDA(launch_plain(gelu_table_gate_kernel, dim3(flat_grid(rows * cols)), dim3(256), 0, stream, z, z_dtype, ldz,
                        table, t_dtype, ldt, table_rows, offset, ids, y, y_dtype, ldy, rows, cols, err));
  DSP_CHECK_LAUNCH("dsp_gelu_table_gate");
  return 0;
}

extern "C" int dsp_softcap(float* x, long ldx, long rows, int cols, float cap, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  DSP_REQUIRE(x && cap > 0.f, "dsp_softcap: missing operand or cap <= 0");
  DSP_CUDA(launch_plain(softcap_kernel, dim3(flat_grid(rows * cols)), dim3(256), 0, stream, x, ldx, rows, cols, cap));
  DSP_CHECK_LAUNCH("dsp_softcap");
  return 0;
}

extern "C" int dsp_scale_rows(float* x, long ldx, long rows, int cols, float s, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  DSP_REQUIRE(x, "dsp_scale_rows: missing operand");
  DSP_CUDA(launch_plain(scale_rows_kernel, dim3(flat_grid(rows * cols)), dim3(256), 0, stream, x, ldx, rows, cols, s));
  DSP_CHECK_LAUNCH("dsp_scale_rows");
  return 0;
}

extern "C" int dsp_sigmoid_gate(const void* x, int x_dtype, long ldx, const void* gate, int g_dtype, long ldg, int per,
                                void* y, int y_dtype, long ldy, long rows, int cols, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  DSP_REQUIRE(x && gate && y && per > 0, "dsp_sigmoid_gate: missing operand");
  DSP_CUDA(launch_plain(sigmoid_gate_kernel, dim3(flat_grid(rows * cols)), dim3(256), 0, stream, x, x_dtype, ldx, gate,
                        g_dtype, ldg, per, y, y_dtype, ldy, rows, cols));
  DSP_CHECK_LAUNCH("dsp_sigmoid_gate");
  return 0;
}

extern "C" int dsp_diff_heads(const void* a, int a_dtype, long lda, float lambda, float post, float eps, const void* gate,
                              int g_dtype, long ldg, void* y, int y_dtype, long ldy, int T, int H, int dv,
                              cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(a && y && H > 0 && dv > 0, "dsp_diff_heads: missing operand");
  const long pairs = (long)T * H;
  DSP_CUDA(launch_plain(diff_heads_kernel, dim3((unsigned)((pairs + 3) / 4)), dim3(128), 0, stream, a, a_dtype, lda, lambda,
                        post, eps, gate, g_dtype, ldg, y, y_dtype, ldy, T, H, dv));
  DSP_CHECK_LAUNCH("dsp_diff_heads");
  return 0;
}

extern "C" int dsp_embed_scaled(const void* table, int t_dtype, int table_rows, const int* ids, float scale,
                                float* out, long ldo, long rows, int cols, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  DSP_REQUIRE(table && ids && out, "dsp_embed_scaled: missing operand");
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr, "dsp_embed_scaled: no device error word");
  DSP_CUDA(launch_plain(embed_scaled_kernel, dim3(flat_grid(rows * cols)), dim3(256), 0, stream, table, t_dtype,
                        table_rows, ids, scale, out, ldo, rows, cols, err));
  DSP_CHECK_LAUNCH("dsp_embed_scaled");
  return 0;
}
