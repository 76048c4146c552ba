// hy_experts.cuh — routed gated feed-forward of the layered hybrid decoders (libjf_hybrid.so).
//
//   route     per token: sigmoid scores of the router logits, group-limited choice of `top` experts, normalised weights;
//             per-expert pair counts by atomic add (the counts, not their order, decide the layout)
//   offsets   exclusive prefix of the counts, the list of (expert, first row) tiles of the grouped products
//   scatter   every (token, choice) pair gets a row in its expert's range of the sorted order
//   products  gate/up with the gated activation in the epilogue, then down, both grouped by expert: a block looks up its
//             tile, reads activation rows through the sorted order and the expert's weight matrix
//   combine   per token the weighted sum of its pairs' rows in the order of its choices, then the sublayer's output norm,
//             layer scale and the residual sum
// A token's result does not depend on the batch: its choices, its weights and the order of its sum are its own, and a
// row of a product does not depend on the other rows of its tile.  Router scores, weights and the combine are fp32.
#pragma once
#include "hy_kernels.cuh"

namespace hy {

struct RouteCfg { int experts, top, groups, keep; float scale; };

// One warp per token.  Scores live in shared memory; lane 0 makes the (tiny, serial) choice.  Ties go to the lower index.
// A group is worth the sum of its two best scores (its single score when groups hold one expert).
__global__ void __launch_bounds__(32) route_kernel(const float* __restrict__ logits, int ldl, RouteCfg c, int* __restrict__ ids,
                                                   float* __restrict__ wts, int* __restrict__ counts) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  float* s = reinterpret_cast<float*>(hy_smem);                // [experts] scores, negated once chosen
  float* gs = s + c.experts;                                   // [groups]; -1 once kept
  const int t = blockIdx.x, lane = threadIdx.x;
  for (int e = lane; e < c.experts; e += 32) s[e] = sigmoid_f(logits[(size_t)t * ldl + e]);
  __syncwarp();
  const int per = c.experts / c.groups;
  for (int g = lane; g < c.groups; g += 32) {
    float m1 = -1.0f, m2 = -1.0f;
    for (int i = 0; i < per; ++i) {
      const float v = s[g * per + i];
      if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
    }
    gs[g] = per >= 2 ? m1 + m2 : m1;
  }
  __syncwarp();
  if (lane != 0) return;
  // keep the best groups: kept groups are marked by a score below every real one (scores are sums of sigmoids, > 0)
  for (int k = 0; k < c.keep; ++k) {
    int best = 0; float bv = -1.0f;
    for (int g = 0; g < c.groups; ++g) if (gs[g] > bv) { bv = gs[g]; best = g; }
    gs[best] = -2.0f;
  }
  float sum = 0.0f;
  for (int k = 0; k < c.top; ++k) {
    int best = 0; float bv = -1.0f;
    for (int g = 0; g < c.groups; ++g) {
      if (gs[g] != -2.0f) continue;
      for (int i = 0; i < per; ++i) { const float v = s[g * per + i]; if (v > bv) { bv = v; best = g * per + i; } }
    }
    ids[(size_t)t * c.top + k] = best;
    wts[(size_t)t * c.top + k] = bv;
    sum += bv;
    s[best] = -1.0f;
    if (counts) atomicAdd(&counts[best], 1);
  }
  const float f = c.scale / (sum + 1e-20f);
  for (int k = 0; k < c.top; ++k) wts[(size_t)t * c.top + k] *= f;
}

// The other way to score: the `top` largest router logits (bias added here, ties to the lower index), weights = softmax
// over the chosen logits alone.  One warp per token, lane 0 makes the choice.
__global__ void __launch_bounds__(32) route_top_kernel(const float* __restrict__ logits, int ldl, const float* __restrict__ bias,
                                                       int experts, int top, int* __restrict__ ids, float* __restrict__ wts,
                                                       int* __restrict__ counts) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  float* s = reinterpret_cast<float*>(hy_smem);                // [experts] logits, -inf once chosen
  const int t = blockIdx.x, lane = threadIdx.x;
  for (int e = lane; e < experts; e += 32) s[e] = logits[(size_t)t * ldl + e] + (bias ? bias[e] : 0.0f);
  __syncwarp();
  if (lane != 0) return;
  float mx = 0.0f, sum = 0.0f;
  for (int k = 0; k < top; ++k) {
    int best = 0; float bv = -INFINITY;
    for (int e = 0; e < experts; ++e) if (s[e] > bv) { bv = s[e]; best = e; }
    if (k == 0) mx = bv;                                       // the first choice is the largest: the softmax's maximum
    const float w = expf(bv - mx);
    ids[(size_t)t * top + k] = best;
    wts[(size_t)t * top + k] = w;
    sum += w;
    s[best] = -INFINITY;
    if (counts) atomicAdd(&counts[best], 1);
  }
  const float f = 1.0f / sum;
  for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] *= f;
}

// out[t, f] = act(in[t, f]) * in[t, n + f] (or the clamped pair, see gated_pair_f): the gated pair of a dense feed-forward whose gate and up rows are stacked.
template <typename AT>
__global__ void gated_act_kernel(const AT* __restrict__ in, int ldi, int n, int act, float limit, AT* __restrict__ out, int ldo) {
  const int t = blockIdx.y;
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f < n) out[(size_t)t * ldo + f] = from_f<AT>(gated_pair_f(act, to_f(in[(size_t)t * ldi + f]), to_f(in[(size_t)t * ldi + n + f]), limit));
}

// Tiles of tile_rows rows of one expert (HY_XT for the SIMT product, 128 for the tensor-core product).  meta: [0] number
// of tiles; offs [experts + 1]; fill [experts] zeroed here.
constexpr int HY_XT = 64;
__global__ void route_offsets_kernel(int* __restrict__ counts, int experts, int tile_rows, int* __restrict__ offs,
                                     int* __restrict__ fill, int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                     int* __restrict__ meta) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int at = 0, nt = 0;
  for (int e = 0; e < experts; ++e) {
    const int n = counts[e];
    offs[e] = at;
    for (int r = 0; r < n; r += tile_rows) { tile_expert[nt] = e; tile_row0[nt] = at + r; ++nt; }
    at += n;
    fill[e] = 0;
    counts[e] = 0;                                             // ready for the next routed layer
  }
  offs[experts] = at;
  meta[0] = nt;
}

// pair i = (token i / top, choice i % top) -> row of the sorted order; row_tok[row] = token, pair_row[i] = row.
__global__ void route_scatter_kernel(int pairs, int top, const int* __restrict__ ids, const int* __restrict__ offs,
                                     int* __restrict__ fill, int* __restrict__ row_tok, int* __restrict__ pair_row) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  const int e = ids[i];
  const int row = offs[e] + atomicAdd(&fill[e], 1);
  row_tok[row] = i / top;
  pair_row[i] = row;
}

// Grouped product over the sorted rows: C[row, n] = sum_k A[src(row), k] W_e[n, k], e the expert of the row's tile.
// GLU: W_e is [2 N, K] (gate rows, then up rows) and the result is act(gate) * up; without GLU the result passes through
// the activation when act >= 0 (act: 0 silu, 1 tanh-gelu, 2 erf-gelu; see act_f).  src(row) = row_map[row] when a map
// is given (activation rows of the tokens), else row.  Tiled SIMT, fp32 FMAs in k order: both builds can use it.
template <typename TA, typename TW, typename TO, bool GLU>
__global__ void __launch_bounds__(256) expert_gemm_simt_kernel(const TA* __restrict__ A, int lda, const int* __restrict__ row_map,
                                                               const TW* __restrict__ W, size_t w_stride, int N, int K,
                                                               const int* __restrict__ offs, const int* __restrict__ tile_expert,
                                                               const int* __restrict__ tile_row0, const int* __restrict__ meta,
                                                               TO* __restrict__ out, int ldo, int act) {
  constexpr int BM = HY_XT, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[GLU ? 2 : 1][BK][BN + 4];
  __shared__ int src[BM];
  for (int tile = blockIdx.y; tile < meta[0]; tile += gridDim.y) {
    const int e = tile_expert[tile], r0 = tile_row0[tile];
    const int rows = min(BM, offs[e + 1] - r0);
    const TW* We = W + (size_t)e * w_stride;
    const int n0 = blockIdx.x * BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    __syncthreads();
    const int tid = (int)threadIdx.x;
    if (tid < BM) src[tid] = tid < rows ? (row_map ? row_map[r0 + tid] : r0 + tid) : -1;
    __syncthreads();
    float acc[4][4] = {}, acc2[GLU ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
      for (int i = threadIdx.x; i < BM * BK; i += 256) {
        const int r = i / BK, kk = i % BK, k = k0 + kk;
        As[kk][r] = (src[r] >= 0 && k < K) ? to_f(A[(size_t)src[r] * lda + k]) : 0.0f;
      }
      for (int i = threadIdx.x; i < BN * BK; i += 256) {
        const int r = i / BK, kk = i % BK, n = n0 + r, k = k0 + kk;
        const bool ok = n < N && k < K;
        Ws[0][kk][r] = ok ? to_f(We[(size_t)n * K + k]) : 0.0f;
        if (GLU) Ws[GLU ? 1 : 0][kk][r] = ok ? to_f(We[(size_t)(N + n) * K + k]) : 0.0f;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        float a[4], w[4], u[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) { w[j] = Ws[0][kk][tx * 4 + j]; u[j] = GLU ? Ws[GLU ? 1 : 0][kk][tx * 4 + j] : 0.0f; }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
            if (GLU) acc2[GLU ? i : 0][j] = fmaf(a[i], u[j], acc2[GLU ? i : 0][j]);
          }
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty * 4 + i;
      if (r >= rows) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        if (n >= N) continue;
        const float c = GLU ? act_f(act, acc[i][j]) * acc2[GLU ? i : 0][j] : act >= 0 ? act_f(act, acc[i][j]) : acc[i][j];
        out[(size_t)(r0 + r) * ldo + n] = from_f<TO>(c);
      }
    }
  }
}

// Few pairs (decode steps): one block row per pair, a warp per output column, the expert's weight rows streamed 16 bytes
// per lane; the pair's activation row is staged in shared memory.  pair = (token, choice); no sorted order is needed:
// A row = row_map ? row_map[pair] : pair, expert = ids[pair], output row = pair.
template <typename TA, typename TW, typename TO, bool GLU>
__global__ void __launch_bounds__(256) expert_rows_kernel(const TA* __restrict__ A, int lda, const int* __restrict__ ids, int top,
                                                          int a_per_token, const TW* __restrict__ W, size_t w_stride, int N, int K,
                                                          TO* __restrict__ out, int ldo, int act) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  TA* As = reinterpret_cast<TA*>(hy_smem);
  constexpr int VEC = 16 / sizeof(TW);
  const int pair = blockIdx.y;
  const TA* ar = A + (size_t)(a_per_token ? pair / top : pair) * lda;
  for (int k = threadIdx.x; k < K; k += blockDim.x) As[k] = ar[k];
  __syncthreads();
  const TW* We = W + (size_t)ids[pair] * w_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool vec_ok = K % VEC == 0 && (reinterpret_cast<uintptr_t>(We) & 15) == 0;
  for (int n = blockIdx.x * 8 + warp; n < N; n += gridDim.x * 8) {
    float acc = 0.0f, acc2 = 0.0f;
    const TW* wr = We + (size_t)n * K;
    const TW* ur = We + (size_t)(N + n) * K;
    if (vec_ok) {
#pragma unroll 2
      for (int k = lane * VEC; k < K; k += 32 * VEC) {
        const VecN<TW, VEC> wv = *reinterpret_cast<const VecN<TW, VEC>*>(wr + k);
        VecN<TW, VEC> uv;
        if (GLU) uv = *reinterpret_cast<const VecN<TW, VEC>*>(ur + k);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const float a = to_f(As[k + j]);
          acc = fmaf(a, to_f(wv.v[j]), acc);
          if (GLU) acc2 = fmaf(a, to_f(uv.v[j]), acc2);
        }
      }
    } else {
      for (int k = lane; k < K; k += 32) {
        const float a = to_f(As[k]);
        acc = fmaf(a, to_f(wr[k]), acc);
        if (GLU) acc2 = fmaf(a, to_f(ur[k]), acc2);
      }
    }
    acc = warp_sum(acc);
    if (GLU) acc2 = warp_sum(acc2);
    if (lane == 0) out[(size_t)pair * ldo + n] = from_f<TO>(GLU ? act_f(act, acc) * acc2 : act >= 0 ? act_f(act, acc) : acc);
  }
}

// x[t] += ls * (tanh(alpha y) w + b),  y = sum_k wts[t, k] rows[pair_row ? pair_row[t top + k] : t top + k]  (k in order).
// post.w == NULL: x[t] += y (designs without an output norm on the feed-forward).
// next.w != NULL: the updated stream also leaves through the next layer's input norm into next_out [T, width].
template <typename AT>
__global__ void expert_combine_kernel(const float* __restrict__ rows, int ldr, const int* __restrict__ pair_row,
                                      const float* __restrict__ wts, int top, int width, TanhNorm post,
                                      const float* __restrict__ ls, float* __restrict__ x, TanhNorm next,
                                      AT* __restrict__ next_out) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float y = 0.0f;
    for (int k = 0; k < top; ++k) {
      const int i = t * top + k;
      y = fmaf(wts[i], rows[(size_t)(pair_row ? pair_row[i] : i) * ldr + c], y);
    }
    if (post.w) y = ls[c] * fmaf(tanhf(post.alpha * y), post.w[c], post.b[c]);
    const float v = x[(size_t)t * width + c] + y;
    x[(size_t)t * width + c] = v;
    if (next.w) next_out[(size_t)t * width + c] = from_f<AT>(fmaf(tanhf(next.alpha * v), next.w[c], next.b[c]));
  }
}

}  // namespace hy
