// Mixture of experts: a router with groups of experts, and the experts' products over rows that
// are sorted by expert on the device (no host round trip: every launch has a fixed upper bound of
// tiles and blocks beyond the real number leave at once, so a step can be captured in a graph).
//
//   dsp_moe_route    scores = softmax(W_router h) over all experts in 32-bit (W_router float, h of
//                    either type), or with `score_kind` 1 the sigmoid of every logit; experts form `groups` equal runs of neighbours, a group's score
//                    is its largest score, only experts of the `keep` best groups can be chosen;
//                    the `top` largest of those are the token's experts, their scores its weights
//                    (not renormalised).  Equal scores: the lower index wins.  One block per token.
//                    `group_kind` 1: a group's score is the sum of its two largest scores instead.
//                    `normalize`: the weights are the chosen scores divided by their sum (+ 1e-20),
//                    times `weight_scale`.  `extra` > 0: W_router has that many more rows after the
//                    experts'; the sigmoids of their logits go to `extra_out` [T, extra] (gates that
//                    are formed from the same row in the same 32-bit arithmetic).
//   dsp_moe_plan     counts the (token, choice) pairs per expert, lists the pairs expert by expert
//                    and cuts every expert's run into tiles of TILE_ROWS rows.  One block.
//   dsp_moe_product  C[c_row(i)] = act(A[a_row(i)] B_e^T) for the sorted pairs i of every expert e
//                    (B: [experts, N, K]); a_row / c_row are optional index lists (gather, scatter).
//                    act 0: none, 1: the square of relu, 2: a clamped gated unit over neighbouring
//                    columns: column 2j is the gate and 2j + 1 the up value of output j (B holds the
//                    two matrices' rows in turn), both times row_scale[pair] when that is given (a
//                    factor on the pair's input row, applied to the 32-bit sums, which is the same
//                    product), g = min(gate, limit), u = clamp(up, -limit, limit),
//                    C[., j] = g * sigmoid(alpha * g) * (u + up_shift); C is N / 2 wide (limit +inf,
//                    alpha 1 and up_shift 0: silu(gate) * up).
//                    Every output is one chain of fused
//                    multiply-adds in ascending k, so a pair's result depends on nothing but its own
//                    row and its expert.  With `tensor_cores` (bfloat16 operands): mma.sync tiles of
//                    64 pairs (1) or 128 pairs (2); the plan must have been made for tiles of that many rows.
//   dsp_moe_combine  y[t] = base[t] * base_scale[t] + sum_k weight[t, k] * P[t * top + k], in ascending k
//                    (without `base`: from 0; without `base_scale`: 1; without `weight`: every weight 1).
#include <climits>

#include "common.cuh"

namespace {
constexpr int TILE_ROWS = 32, TILE_COLS = 64, TILE_K = 32;
// the tensor-core product comes in two shapes: 64 rows x 4 stages (few rows an expert: decoding)
// and 128 rows x 3 stages (many rows an expert: prompts)
constexpr int MMA_ROWS = 64, MMA_ROWS_WIDE = 128, MMA_COLS = 128, MMA_K = 64, MMA_PAD = 8;
constexpr int MMA_LD = MMA_K + MMA_PAD;
constexpr size_t mma_smem_bytes(int rows, int stages) { return sizeof(bf16) * stages * (rows + MMA_COLS) * MMA_LD; }

__device__ __forceinline__ float clamped_glu(float gate, float up, float limit, float alpha, float up_shift) {
  const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);
  return g * (1.f / (1.f + expf(-alpha * g))) * (u + up_shift);
}

constexpr int GROUPS_PER_LANE = 8;  // the router ranks up to 32 * 8 groups

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.i >= 0 && (a.i < 0 || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
  return a;
}
__device__ __forceinline__ Best warp_best(Best b) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
    b = better(b, other);
  }
  return b;
}

// (two blocks of 1,024 threads an SM: 32 registers a thread, so that prompts' blocks of 16 warps fit four an SM)
__global__ void __launch_bounds__(1024, 2)
moe_route_kernel(const void* __restrict__ h, int h_dtype, long ldh, const float* __restrict__ w, int T, int W, int E,
                 int groups, int keep, int top, int score_kind, int group_kind, int normalize, float weight_scale,
                 int extra, float* __restrict__ extra_out, int* __restrict__ ids, float* __restrict__ wts) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const long t = blockIdx.x;
  float* sc = sm;              // [E + extra] scores (logits of the extra rows)
  float* ok = sc + E + extra;  // [E] 1: may still be chosen
  float* gb = ok + E;          // [groups] best score of each group
  float* hs = gb + groups;     // [W] the token's row
  for (int i = threadIdx.x; i < W; i += blockDim.x) hs[i] = ld_any(h, h_dtype, (size_t)t * ldh + i);
  __syncthreads();
  // every expert's logit is the same sum whatever the block's shape: lane i takes columns i, i + 32, ...
  // in four interleaved chains (so that four loads are in flight), added in a fixed order
  for (int e = warp; e < E + extra; e += warps) {
    const float* we = w + (size_t)e * W;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    int i = lane;
#pragma unroll 4
    for (; i + 96 < W; i += 128) {
      a0 = fmaf(we[i], hs[i], a0);
      a1 = fmaf(we[i + 32], hs[i + 32], a1);
      a2 = fmaf(we[i + 64], hs[i + 64], a2);
      a3 = fmaf(we[i + 96], hs[i + 96], a3);
    }
    for (; i < W; i += 32) a0 = fmaf(we[i], hs[i], a0);
    const float acc = warp_sum((a0 + a1) + (a2 + a3));
    if (lane == 0) sc[e] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  for (int j = lane; j < extra; j += 32) extra_out[t * extra + j] = 1.f / (1.f + expf(-sc[E + j]));
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, sc[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) sum += expf(sc[e] - mx);
  sum = warp_sum(sum);
  __syncwarp();
  // sigmoid scores are chosen by their logits: the order is the same, and two logits whose sigmoids
  // both round to 1 still differ
  for (int e = lane; e < E; e += 32) {
    if (score_kind != 1) sc[e] = expf(sc[e] - mx) / sum;
    ok[e] = 0.f;
  }
  __syncwarp();
  const int per = E / groups;
  // Group scores live in registers (lane i: groups i, i + 32, ...) as a whole number plus a small
  // part: a sigmoid above one half is kept as 1 - sigmoid(-z), so that the sum of two scores near 1 is
  // 2 minus two small deficits that float arithmetic holds exactly enough to rank groups whose plain
  // 32-bit sums would all round to 2 (a saturated router would otherwise send every token to the
  // first groups).  Group a beats group b when (a.whole - b.whole) + (a.part - b.part) > 0.
  int whole[GROUPS_PER_LANE];
  float part[GROUPS_PER_LANE];
#pragma unroll
  for (int k = 0; k < GROUPS_PER_LANE; ++k) {
    const int g = lane + 32 * k;
    whole[k] = INT_MIN;  // no group, or one that is open already
    part[k] = 0.f;
    if (g >= groups) continue;
    float b = -INFINITY, b2 = -INFINITY;  // the group's largest and second largest
    for (int j = 0; j < per; ++j) {
      const float v = sc[g * per + j];
      if (v > b) {
        b2 = b;
        b = v;
      } else {
        b2 = fmaxf(b2, v);
      }
    }
    whole[k] = 0;
    if (group_kind == 1 && score_kind == 1) {  // the sum of the two largest sigmoids (sc holds logits)
      const int n = per < 2 ? 1 : 2;
      for (int i = 0; i < n; ++i) {
        const float z = i ? b2 : b;
        const float small = 1.f / (1.f + expf(fabsf(z)));  // sigmoid(-|z|)
        whole[k] += z > 0.f;
        part[k] += z > 0.f ? -small : small;
      }
    } else if (group_kind == 1) {
      part[k] = b + (per < 2 ? 0.f : b2);
    } else {
      part[k] = b;
    }
  }
  auto beats = [](int wa, float pa, int ia, int wb, float pb, int ib) {
    if (wa == INT_MIN) return false;
    if (wb == INT_MIN) return true;
    const float d = (float)(wa - wb) + (pa - pb);
    return d > 0.f || (d == 0.f && ia < ib);
  };
  for (int r = 0; r < keep; ++r) {
    int bw = INT_MIN, bi = -1;
    float bp = 0.f;
#pragma unroll
    for (int k = 0; k < GROUPS_PER_LANE; ++k) {
      const int g = lane + 32 * k;
      if (g < groups && beats(whole[k], part[k], g, bw, bp, bi)) {
        bw = whole[k];
        bp = part[k];
        bi = g;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const int ow = __shfl_xor_sync(0xffffffffu, bw, o), oi = __shfl_xor_sync(0xffffffffu, bi, o);
      const float op = __shfl_xor_sync(0xffffffffu, bp, o);
      if (beats(ow, op, oi, bw, bp, bi)) {
        bw = ow;
        bp = op;
        bi = oi;
      }
    }
    if (bw == INT_MIN) break;
    for (int j = lane; j < per; j += 32) ok[bi * per + j] = 1.f;
#pragma unroll
    for (int k = 0; k < GROUPS_PER_LANE; ++k)
      if (lane + 32 * k == bi) whole[k] = INT_MIN;
    __syncwarp();
  }
  // every lane holds each round's winner: the weights' sum is formed in registers (ascending r), the
  // weights wait in shared memory (the token's row is no longer needed) and go out once, scaled
  float wsum = 0.f;
  for (int r = 0; r < top; ++r) {
    Best b = {-INFINITY, -1};
    for (int e = lane; e < E; e += 32) b = better(b, Best{sc[e], ok[e] > 0.f ? e : -1});
    b = warp_best(b);
    const float wr = b.i < 0 ? 0.f : score_kind == 1 ? 1.f / (1.f + expf(-b.v)) : b.v;
    wsum += wr;
    if (lane == 0) {
      ids[t * top + r] = b.i;
      hs[r] = wr;
      if (b.i >= 0) ok[b.i] = 0.f;
    }
    __syncwarp();
  }
  const float f = normalize ? weight_scale / (wsum + 1e-20f) : 1.f;
  for (int r = lane; r < top; r += 32) wts[t * top + r] = hs[r] * f;
}

__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int n_pairs, int E, int tile_rows_max, int* __restrict__ offsets,
                int* __restrict__ sorted_pair, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                int* __restrict__ tile_rows, int* __restrict__ n_tiles, int max_tiles) {
  extern __shared__ int ism[];
  int* cnt = ism;      // [E]
  int* cur = ism + E;  // [E]
  int* off = cur + E;  // [E + 1]
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = cur[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      for (int r = 0; r < cnt[e] && nt < max_tiles; r += tile_rows_max, ++nt) {
        tile_expert[nt] = e;
        tile_row0[nt] = o + r;
        tile_rows[nt] = min(tile_rows_max, cnt[e] - r);
      }
      o += cnt[e];
    }
    off[E] = o;
    *n_tiles = nt;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) sorted_pair[off[e] + atomicAdd(&cur[e], 1)] = i;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_product_kernel(const T* __restrict__ A, long lda, const int* __restrict__ a_rows, int a_div,
                   const T* __restrict__ B, void* __restrict__ C, int c_dtype, long ldc,
                   const int* __restrict__ c_rows, const int* __restrict__ tile_expert,
                   const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                   const int* __restrict__ n_tiles, int N, int K, int act, const float* __restrict__ row_scale,
                   float limit, float alpha, float up_shift) {
  const int tile = blockIdx.x;
  if (tile >= *n_tiles) return;
  __shared__ float As[TILE_K][TILE_ROWS + 1];
  __shared__ float Bs[TILE_K][TILE_COLS + 1];
  __shared__ long arow[TILE_ROWS], crow[TILE_ROWS];
  __shared__ float rscale[TILE_ROWS];
  const int e = tile_expert[tile], r0 = tile_row0[tile], nr = tile_rows[tile];
  const int n0 = blockIdx.y * TILE_COLS;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (tid < TILE_ROWS) {
    const int i = r0 + tid;
    arow[tid] = tid < nr ? (a_rows ? (long)(a_rows[i] / a_div) : (long)i) : -1;
    crow[tid] = tid < nr ? (c_rows ? (long)c_rows[i] : (long)i) : -1;
    rscale[tid] = (tid < nr && row_scale) ? row_scale[a_rows ? a_rows[i] : i] : 1.f;
  }
  __syncthreads();
  const T* Be = B + (size_t)e * N * K;
  float acc[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += TILE_K) {
    for (int idx = tid; idx < TILE_ROWS * TILE_K; idx += 256) {
      const int r = idx / TILE_K, k = idx % TILE_K;
      As[k][r] = (arow[r] >= 0 && k0 + k < K) ? to_f32(A[(size_t)arow[r] * lda + k0 + k]) : 0.f;
    }
    for (int idx = tid; idx < TILE_COLS * TILE_K; idx += 256) {
      const int n = idx / TILE_K, k = idx % TILE_K;
      Bs[k][n] = (n0 + n < N && k0 + k < K) ? to_f32(Be[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TILE_K; ++k) {
      const float a0 = As[k][ty * 2], a1 = As[k][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = Bs[k][tx * 4 + j];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const long cr = crow[ty * 2 + i];
    if (cr < 0) continue;
    if (act == 2) {
      const float f = rscale[ty * 2 + i];
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = n0 + tx * 4 + j;
        if (n + 1 >= N) continue;
        st_any(C, c_dtype, (size_t)cr * ldc + n / 2, clamped_glu(acc[i][j] * f, acc[i][j + 1] * f, limit, alpha, up_shift));
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (act == 1) {
        v = fmaxf(v, 0.f);
        v *= v;
      }
      st_any(C, c_dtype, (size_t)cr * ldc + n, v);
    }
  }
}


// The same product on tensor cores (bfloat16 operands, 32-bit accumulators): a tile of up to ROWS
// pairs x 128 outputs per block of ROWS / 16 warps (ROWS / 32 x 2, each 32 x 64 in m16n8k16 pieces),
// k in blocks of 64 through a ring of STAGES cp.async stages (two blocks an SM); A rows are
// gathered by their indices.
// K and the row strides are multiples of 8 elements and the operands 16-byte aligned.
__device__ __forceinline__ void cp16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int ROWS, int STAGES>
__global__ void __launch_bounds__(ROWS * 2, 2)
moe_product_mma_kernel(const bf16* __restrict__ A, long lda, const int* __restrict__ a_rows, int a_div,
                       const bf16* __restrict__ B, void* __restrict__ C, int c_dtype, long ldc,
                       const int* __restrict__ c_rows, const int* __restrict__ tile_expert,
                       const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                       const int* __restrict__ n_tiles, int N, int K, int act, const float* __restrict__ row_scale,
                       float limit, float alpha, float up_shift) {
  const int tile = blockIdx.x;
  if (tile >= *n_tiles) return;
  extern __shared__ __align__(16) unsigned char mma_smem[];
  bf16 (*As)[ROWS][MMA_LD] = reinterpret_cast<bf16 (*)[ROWS][MMA_LD]>(mma_smem);
  bf16 (*Bs)[MMA_COLS][MMA_LD] =
      reinterpret_cast<bf16 (*)[MMA_COLS][MMA_LD]>(mma_smem + sizeof(bf16) * STAGES * ROWS * MMA_LD);
  __shared__ long arow[ROWS], crow[ROWS];
  __shared__ float rscale[ROWS];
  const int e = tile_expert[tile], r0 = tile_row0[tile], nr = tile_rows[tile];
  const int n0 = blockIdx.y * MMA_COLS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1;  // the warp's 32 rows and 64 columns of the tile
  if (tid < ROWS) {
    const int i = r0 + tid;
    arow[tid] = tid < nr ? (a_rows ? (long)(a_rows[i] / a_div) : (long)i) : -1;
    crow[tid] = tid < nr ? (c_rows ? (long)c_rows[i] : (long)i) : -1;
    rscale[tid] = (tid < nr && row_scale) ? row_scale[a_rows ? a_rows[i] : i] : 1.f;
  }
  __syncthreads();
  const bf16* Be = B + (size_t)e * N * K;
  auto load = [&](int stage, int k0) {
    for (int c = tid; c < ROWS * (MMA_K / 8); c += (ROWS * 2)) {
      const int r = c / (MMA_K / 8), k = (c % (MMA_K / 8)) * 8;
      bf16* dst = &As[stage][r][k];
      if (arow[r] >= 0 && k0 + k < K)
        cp16(dst, A + (size_t)arow[r] * lda + k0 + k);
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    for (int c = tid; c < MMA_COLS * (MMA_K / 8); c += (ROWS * 2)) {
      const int n = c / (MMA_K / 8), k = (c % (MMA_K / 8)) * 8;
      bf16* dst = &Bs[stage][n][k];
      if (n0 + n < N && k0 + k < K)
        cp16(dst, Be + (size_t)(n0 + n) * K + k0 + k);
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;\n");
  };
  float acc[2][8][4] = {};
  const int nk = (K + MMA_K - 1) / MMA_K;
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nk)
      load(s, s * MMA_K);
    else
      asm volatile("cp.async.commit_group;\n");
  }
  for (int kt = 0; kt < nk; ++kt) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2));
    __syncthreads();  // stage kt has landed for everyone; stage kt - 1 has been read by everyone
    if (kt + STAGES - 1 < nk)
      load((kt + STAGES - 1) % STAGES, (kt + STAGES - 1) * MMA_K);
    else
      asm volatile("cp.async.commit_group;\n");
    const int st = kt % STAGES;
#pragma unroll
    for (int kk = 0; kk < MMA_K; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) ldsm4(a[i], &As[st][wm * 32 + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        uint32_t b[4];  // two blocks of eight columns: (n, k 0-7), (n, k 8-15), (n + 8, k 0-7), (n + 8, k 8-15)
        ldsm4(b, &Bs[st][wn * 64 + j * 8 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          mma16816(acc[i][j], a[i], b[0], b[1]);
          mma16816(acc[i][j + 1], a[i], b[2], b[3]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const long cr = crow[wm * 32 + i * 16 + half * 8 + (lane >> 2)];
      if (cr < 0) continue;
      if (act == 2) {  // the thread's two neighbouring columns are a gate and its up value
        const float f = rscale[wm * 32 + i * 16 + half * 8 + (lane >> 2)];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int n = n0 + wn * 64 + j * 8 + (lane & 3) * 2;
          if (n + 1 >= N) continue;
          st_any(C, c_dtype, (size_t)cr * ldc + n / 2,
                 clamped_glu(acc[i][j][half * 2] * f, acc[i][j][half * 2 + 1] * f, limit, alpha, up_shift));
        }
        continue;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int n = n0 + wn * 64 + j * 8 + (lane & 3) * 2 + q;
          if (n >= N) continue;
          float v = acc[i][j][half * 2 + q];
          if (act == 1) {
            v = fmaxf(v, 0.f);
            v *= v;
          }
          st_any(C, c_dtype, (size_t)cr * ldc + n, v);
        }
    }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ P, long ldp, const float* __restrict__ wts, const int* __restrict__ ids,
                   const float* __restrict__ base, long ldb, const float* __restrict__ base_scale,
                   float* __restrict__ y, long ldy, long T, int top, int width) {
  const long n = T * width;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long t = i / width;
    const int c = (int)(i % width);
    float acc = base ? base[(size_t)t * ldb + c] * (base_scale ? base_scale[t] : 1.f) : 0.f;
    for (int k = 0; k < top; ++k)
      if (ids[t * top + k] >= 0) acc = fmaf(wts ? wts[t * top + k] : 1.f, P[(size_t)(t * top + k) * ldp + c], acc);
    y[(size_t)t * ldy + c] = acc;
  }
}
}  // namespace

// Rows of a tile of dsp_moe_product: the tensor-core kernel's (bfloat16) or the 32-bit kernel's.
extern "C" int dsp_moe_tile_rows(int tensor_cores) { return tensor_cores == 2 ? MMA_ROWS_WIDE : tensor_cores ? MMA_ROWS : TILE_ROWS; }

extern "C" int dsp_moe_route(const void* h, int h_dtype, long ldh, const float* w, int T, int W, int E, int groups,
                             int keep, int top, int score_kind, int group_kind, int normalize, float weight_scale,
                             int extra, float* extra_out, int* ids, float* wts, cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(score_kind == 0 || score_kind == 1, "dsp_moe_route: unknown score kind %d", score_kind);
  DSP_REQUIRE(h && w && ids && wts, "dsp_moe_route: missing operand");
  DSP_REQUIRE(top <= W, "dsp_moe_route: top=%d exceeds the row's width %d", top, W);
  DSP_REQUIRE(groups <= 32 * GROUPS_PER_LANE, "dsp_moe_route: %d groups are more than the router ranks (%d)", groups,
              32 * GROUPS_PER_LANE);
  DSP_REQUIRE((group_kind == 0 || group_kind == 1) && extra >= 0 && (extra == 0 || extra_out),
              "dsp_moe_route: group kind %d, %d extra rows", group_kind, extra);
  DSP_REQUIRE(E > 0 && groups > 0 && E % groups == 0 && keep > 0 && keep <= groups && top > 0 &&
                  top <= keep * (E / groups),
              "dsp_moe_route: experts=%d groups=%d keep=%d top=%d do not fit together", E, groups, keep, top);
  const size_t smem = (size_t)(2 * E + extra + groups + W) * sizeof(float);
  DSP_REQUIRE(smem <= 48 * 1024, "dsp_moe_route: %d experts over a width of %d are more than the router kernel holds", E, W);
  // a warp an expert where the block can hold them: the logits are chains of dependent rounds of loads,
  // and a step of a few tokens waits for the longest chain (the sums do not depend on the block's shape)
  // With many tokens the SMs are full of blocks anyway and what counts is how many fit: warps in a power of
  // two (17 rows in 17 warps leave room for three blocks an SM, in 16 warps for four).
  int warps = min(max(E + extra, 4), 32);
  if (T > 512)
    for (int w = 32; w >= 4; w >>= 1)
      if (w <= warps) {
        warps = w;
        break;
      }
  const unsigned threads = 32u * (unsigned)warps;
  DSP_CUDA(launch_plain(moe_route_kernel, dim3((unsigned)T), dim3(threads), smem, stream, h, h_dtype, ldh, w, T, W, E,
                        groups, keep, top, score_kind, group_kind, normalize, weight_scale, extra, extra_out, ids, wts));
  DSP_CHECK_LAUNCH("dsp_moe_route");
  return 0;
}

extern "C" int dsp_moe_plan(const int* ids, int n_pairs, int E, int rows_per_tile, int* offsets, int* sorted_pair,
                            int* tile_expert, int* tile_row0, int* tile_rows, int* n_tiles, int max_tiles,
                            cudaStream_t stream) {
  DSP_REQUIRE(ids && offsets && sorted_pair && tile_expert && tile_row0 && tile_rows && n_tiles, "dsp_moe_plan: missing operand");
  DSP_REQUIRE(rows_per_tile == TILE_ROWS || rows_per_tile == MMA_ROWS || rows_per_tile == MMA_ROWS_WIDE, "dsp_moe_plan: tiles of %d rows", rows_per_tile);
  DSP_REQUIRE(max_tiles >= n_pairs / rows_per_tile + E, "dsp_moe_plan: room for %d tiles, %d may be needed", max_tiles,
              n_pairs / rows_per_tile + E);
  const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
  DSP_REQUIRE(smem <= 48 * 1024, "dsp_moe_plan: %d experts are more than the planning kernel holds", E);
  DSP_CUDA(launch_plain(moe_plan_kernel, dim3(1), dim3(1024), smem, stream, ids, n_pairs, E, rows_per_tile, offsets, sorted_pair,
                        tile_expert, tile_row0, tile_rows, n_tiles, max_tiles));
  DSP_CHECK_LAUNCH("dsp_moe_plan");
  return 0;
}

extern "C" int dsp_moe_product(const void* A, int ab_dtype, long lda, const int* a_rows, int a_div, const void* B,
                               void* C, int c_dtype, long ldc, const int* c_rows, const int* tile_expert,
                               const int* tile_row0, const int* tile_rows, const int* n_tiles, int max_tiles, int N,
                               int K, int act, const float* row_scale, float limit, float alpha, float up_shift,
                               int tensor_cores, cudaStream_t stream) {
  if (max_tiles == 0 || N == 0) return 0;
  DSP_REQUIRE(A && B && C && tile_expert && tile_row0 && tile_rows && n_tiles && a_div > 0, "dsp_moe_product: missing operand");
  DSP_REQUIRE(act >= 0 && act <= 2, "dsp_moe_product: unknown activation %d", act);
  DSP_REQUIRE(act != 2 || N % 2 == 0, "dsp_moe_product: a gated unit needs an even number of columns, not %d", N);
  DSP_REQUIRE(act == 2 || !row_scale, "dsp_moe_product: row factors come with the gated unit only");
  if (tensor_cores) {
    DSP_REQUIRE(ab_dtype == DSP_BF16 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)B % 16) == 0,
                "dsp_moe_product: the tensor-core kernel takes 16-byte aligned bfloat16 operands with K and the row "
                "stride multiples of 8 (K=%d, stride %ld)", K, lda);
    dim3 mgrid(max_tiles, (N + MMA_COLS - 1) / MMA_COLS);
    DSP_REQUIRE(mgrid.y <= 65535, "dsp_moe_product: N=%d is too wide", N);
    static bool configured = false;
    if (!configured) {
      DSP_CUDA(cudaFuncSetAttribute(moe_product_mma_kernel<MMA_ROWS, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)mma_smem_bytes(MMA_ROWS, 4)));
      DSP_CUDA(cudaFuncSetAttribute(moe_product_mma_kernel<MMA_ROWS_WIDE, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)mma_smem_bytes(MMA_ROWS_WIDE, 3)));
      configured = true;
    }
    if (tensor_cores == 2)
      DSP_CUDA(launch_plain(moe_product_mma_kernel<MMA_ROWS_WIDE, 3>, mgrid, dim3(MMA_ROWS_WIDE * 2), mma_smem_bytes(MMA_ROWS_WIDE, 3),
                            stream, (const bf16*)A, lda, a_rows, a_div, (const bf16*)B, C, c_dtype, ldc, c_rows, tile_expert,
                            tile_row0, tile_rows, n_tiles, N, K, act, row_scale, limit, alpha, up_shift));
    else
      DSP_CUDA(launch_plain(moe_product_mma_kernel<MMA_ROWS, 4>, mgrid, dim3(MMA_ROWS * 2), mma_smem_bytes(MMA_ROWS, 4), stream,
                            (const bf16*)A, lda, a_rows, a_div, (const bf16*)B, C, c_dtype, ldc, c_rows, tile_expert,
                            tile_row0, tile_rows, n_tiles, N, K, act, row_scale, limit, alpha, up_shift));
    DSP_CHECK_LAUNCH("dsp_moe_product (tensor cores)");
    return 0;
  }
  dim3 grid(max_tiles, (N + TILE_COLS - 1) / TILE_COLS);
  DSP_REQUIRE(grid.y <= 65535, "dsp_moe_product: N=%d is too wide", N);
  if (ab_dtype == DSP_F32) {
    DSP_CUDA(launch_plain(moe_product_kernel<float>, grid, dim3(256), 0, stream, (const float*)A, lda, a_rows, a_div,
                          (const float*)B, C, c_dtype, ldc, c_rows, tile_expert, tile_row0, tile_rows, n_tiles, N, K, act, row_scale, limit, alpha, up_shift));
  } else {
    DSP_CUDA(launch_plain(moe_product_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)A, lda, a_rows, a_div,
                          (const bf16*)B, C, c_dtype, ldc, c_rows, tile_expert, tile_row0, tile_rows, n_tiles, N, K, act, row_scale, limit, alpha, up_shift));
  }
  DSP_CHECK_LAUNCH("dsp_moe_product");
  return 0;
}

extern "C" int dsp_moe_combine(const float* P, long ldp, const float* wts, const int* ids, const float* base, long ldb,
                               const float* base_scale, float* y, long ldy, long T, int top, int width,
                               cudaStream_t stream) {
  if (T == 0) return 0;
  DSP_REQUIRE(P && ids && y, "dsp_moe_combine: missing operand");
  const long n = T * width;
  const int sms = dsp_num_sms();
  const long want = (n + 255) / 256, cap = (long)(sms > 0 ? sms : 148) * 16;
  DSP_CUDA(launch_plain(moe_combine_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), 0, stream, P, ldp,
                        wts, ids, base, ldb, base_scale, y, ldy, T, top, width));
  DSP_CHECK_LAUNCH("dsp_moe_combine");
  return 0;
}
