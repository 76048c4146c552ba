// hy_kernels.cuh — device kernels of the layered hybrid decoders (libjf_hybrid.so).
//
// Precision rule shared by every kernel here: the residual stream, norms, attention scores and weights, positions and
// angles, recurrent states, decays, step sizes, gates of a recurrence and unit norms are fp32; projections, short
// convolutions with their activations and the operands of the matrix products are AT (bf16 in the serving build, fp32 in
// the all-fp32 build).  A step is a packed batch of entries (portions of prompts beside single decoded tokens); no
// result depends on how a request was cut or on what else is in the batch: every reduction runs over absolute key
// positions / a fixed k order.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hy {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z * sigmoid_f(z); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }
__device__ __forceinline__ float gelu_erf_f(float z) { return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f)); }
// activation by kind: 0 silu, 1 the tanh form of gelu, 2 gelu with the error function
__device__ __forceinline__ float act_f(int kind, float z) { return kind == 1 ? gelu_tanh_f(z) : kind == 2 ? gelu_erf_f(z) : silu_f(z); }
// a gated pair by kind: act(gate) * up, or (kind 3) the clamped pair g = min(gate, limit), u = clamp(up, -limit, limit),
// g sigmoid(1.702 g) (u + 1)
__device__ __forceinline__ float gated_pair_f(int kind, float g, float u, float limit) {
  if (kind == 3) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoid_f(1.702f * g) * (u + 1.0f);
  }
  return act_f(kind, g) * u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum over the block; every thread gets the result.  red: >= 33 floats of shared memory.  Deterministic order.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float s = lane < nw ? red[lane] : 0.0f;
    s = warp_sum(s);
    if (lane == 0) red[32] = s;
  }
  __syncthreads();
  return red[32];
}

// Per-step batch description (device pointers, all int32).
struct Batch {
  const int* tok;        // [T] token ids
  const int* tok_ent;    // [T] entry of a token
  const int* tok_pos;    // [T] absolute position in its request
  const int* ent_start;  // [E + 1]
  const int* ent_pos0;   // [E]
  const int* ent_slot;   // [E]
  const int* pages;      // [E, max_pages]
  int T, E, max_pages, page_size;
};

// ---- embedding: table row times a scale, plus the sinusoid of the position ----------------------------------------------
// entry 2i = sin(p f_i), entry 2i+1 = cos(p f_i); f_i = 10000^(-2i / width) comes from a host-made fp64 table and the angle
// is formed and reduced in fp64 (at position 1000 an fp32 angle is already 6e-5 off), the result enters the fp32 stream.
// inv_freq == NULL: no positional term (designs whose positions enter through a rotation inside attention).
template <typename WT>
__global__ void embed_kernel(Batch b, const WT* __restrict__ table, const double* __restrict__ inv_freq, float scale,
                             int width, float* __restrict__ x) {
  const int t = blockIdx.x;
  const int tok = b.tok[t];
  const double p = (double)b.tok_pos[t];
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float pe = 0.0f;
    if (inv_freq) {
      const double ang = p * inv_freq[c >> 1];
      pe = (float)((c & 1) ? cos(ang) : sin(ang));
    }
    x[(size_t)t * width + c] = to_f(table[(size_t)tok * width + c]) * scale + pe;
  }
}

// ---- element-wise tanh norm: tanh(alpha x) w + b, no statistics ------------------------------------------------------------
// rows: NULL = row r of x, else x row rows[r].  Parameters are fp32.
struct TanhNorm { const float* w; const float* b; float alpha; };
template <typename OT>
__global__ void tanh_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows, TanhNorm n, int width,
                                 OT* __restrict__ out) {
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(size_t)r * width + c] = from_f<OT>(fmaf(tanhf(n.alpha * xr[c]), n.w[c], n.b[c]));
}

// ---- RMS norm; the weight is w_offset + w (1: stored as an offset from one, 0: plain) -----------------------------------------
// rows: NULL = row r of x, else x row rows[r].  out row r.
template <typename WT, typename OT>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const WT* __restrict__ w,
                               float eps, int width, float w_offset, OT* __restrict__ out) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) { const float v = xr[c]; ss += v * v; }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(size_t)r * width + c] = from_f<OT>(xr[c] * inv * (w_offset + to_f(w[c])));
}

// ---- generic matrix product C[t, n] = sum_k A[t, k] W[n, k], fp32 accumulation in k order -----------------------------------
// Destinations: resid != NULL: resid[t, n] += alpha * c (fp32, the residual stream).  Otherwise columns < split go to
// out1[t * ld1 + n], columns >= split to out2[t * ld2 + n - split], squared ReLU first when act2 (the feed-forward's
// hidden activation leaves the merged input projection already activated).  With post_w set, the residual receives
// post_ls[n] * (tanh(post_alpha c) post_w[n] + post_b[n]): a sublayer's output norm (element-wise, so it needs no second
// pass) and its layer scale, applied to the fp32 accumulator.
// With next_w set as well, the element of the updated residual also leaves through the NEXT sublayer's input norm
// (tanh(next_alpha x) next_w[n] + next_b[n]) into next_out [T, ldr] in the activation type: no separate norm launch.
// act2 == 3: every column passes through the activation act_kind (act_f) before it is stored.  out2_f32: the columns from
// `split` on leave as fp32 whatever the output type (gate pre-activations of a recurrence beside its bf16 operands).
// bias: added to the scaled accumulator of column n before anything else (projections with biases).  act_limit: the limit
// of the clamped gated pair (act2 == 2 with act_kind 3).
struct GemmOut {
  void* out1; int ld1; int split; void* out2; int ld2; int act2;
  float* resid; int ldr; float alpha;
  const float* post_w; const float* post_b; const float* post_ls; float post_alpha;
  const float* next_w; const float* next_b; float next_alpha; void* next_out; int next_f32;
  int act_kind; int out2_f32;
  const float* bias; float act_limit;
};

template <typename TO>
__device__ __forceinline__ void gemm_store(const GemmOut& o, int t, int n, float c) {
  c *= o.alpha;
  if (o.bias) c += o.bias[n];
  if (o.resid) {
    if (o.post_w) c = o.post_ls[n] * fmaf(tanhf(o.post_alpha * c), o.post_w[n], o.post_b[n]);
    const float v = o.resid[(size_t)t * o.ldr + n] + c;
    o.resid[(size_t)t * o.ldr + n] = v;
    if (o.next_w) {
      const float y = fmaf(tanhf(o.next_alpha * v), o.next_w[n], o.next_b[n]);
      if (o.next_f32) ((float*)o.next_out)[(size_t)t * o.ldr + n] = y;
      else ((bf16*)o.next_out)[(size_t)t * o.ldr + n] = __float2bfloat16_rn(y);
    }
    return;
  }
  if (o.act2 == 3) c = act_f(o.act_kind, c);
  if (n < o.split) { ((TO*)o.out1)[(size_t)t * o.ld1 + n] = from_f<TO>(c); return; }
  if (o.act2 == 1) { c = fmaxf(c, 0.0f); c = c * c; }
  if (o.out2_f32) ((float*)o.out2)[(size_t)t * o.ld2 + (n - o.split)] = c;
  else ((TO*)o.out2)[(size_t)t * o.ld2 + (n - o.split)] = from_f<TO>(c);
}

// ---- RMS norm on a sublayer's output, layer scale and the residual sum --------------------------------------------------------
// x[t] <- (add ? x[t] : 0) + ls * y[t] / sqrt(mean(y[t]^2) + eps) * w   (ls == NULL: one), and the updated row also leaves
// in the activation type (the next sublayer reads the stream itself).  y[t] is row t of ybuf, or, when `rows` is given,
// the mixture of a routed feed-forward: sum_k wts[t, k] rows[pair_row ? pair_row[t top + k] : t top + k] in the order of
// the token's choices, plus shared_rows[t] (an expert every token uses) when given.  ybuf may be x itself (add = 0).
template <typename AT>
__global__ void post_norm_add_kernel(const float* ybuf, int ldy, const float* __restrict__ rows, int ldr,
                                     const int* __restrict__ pair_row, const float* __restrict__ wts, int top,
                                     const float* __restrict__ shared_rows, const float* __restrict__ w,
                                     const float* __restrict__ ls, float eps, int width, int add, float* x,
                                     AT* __restrict__ next_out) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  float* ys = reinterpret_cast<float*>(hy_smem);               // [width]
  __shared__ float red[33];
  const int t = blockIdx.x;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float y;
    if (rows) {
      y = 0.0f;
      for (int k = 0; k < top; ++k) {
        const int i = t * top + k;
        y = fmaf(wts[i], rows[(size_t)(pair_row ? pair_row[i] : i) * ldr + c], y);
      }
      if (shared_rows) y += shared_rows[(size_t)t * ldr + c];
    } else {
      y = ybuf[(size_t)t * ldy + c];
    }
    ys[c] = y;
    ss = fmaf(y, y, ss);
  }
  ss = block_sum(ss, red);
  const float inv = w ? 1.0f / sqrtf(ss / (float)width + eps) : 1.0f;      // w == NULL: no norm, the row passes as it is
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float n = ys[c] * inv * (w ? w[c] : 1.0f) * (ls ? ls[c] : 1.0f);
    const float v = add ? x[(size_t)t * width + c] + n : n;
    x[(size_t)t * width + c] = v;
    if (next_out) next_out[(size_t)t * width + c] = from_f<AT>(v);
  }
}

// Tiled SIMT kernel: any shape, any leading dimensions; the all-fp32 build's matrix product (true fp32 FMAs).
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, int ldw,
                                                        int T, int N, int K, GemmOut o) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int t0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;     // tx: 4 columns, ty: 4 rows
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int i = threadIdx.x; i < BM * BK; i += 256) {
      const int r = i / BK, kk = i % BK;
      const int t = t0 + r, k = k0 + kk;
      As[kk][r] = (t < T && k < K) ? to_f(A[(size_t)t * lda + k]) : 0.0f;
    }
    for (int i = threadIdx.x; i < BN * BK; i += 256) {
      const int r = i / BK, kk = i % BK;
      const int n = n0 + r, k = k0 + kk;
      Ws[kk][r] = (n < N && k < K) ? to_f(W[(size_t)n * ldw + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) gemm_store<TO>(o, t, n, acc[i][j]);
    }
  }
}

// Few-row kernel (decode steps): the weight matrix is streamed once, 16 bytes per lane per load, four loads in flight per
// lane; one warp owns one output column for up to ROWS rows; the rows' operand sits in shared memory in its own type and
// is read back 16 bytes at a time (conflict-free).  K order: lane-strided partial sums, then an xor tree.
template <typename T, int N>
struct VecN { T v[N]; };

template <typename TA, typename TW, typename TO, int ROWS>
__global__ void __launch_bounds__(256) gemm_rows_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, int ldw,
                                                        int T, int N, int K, int ksplit, GemmOut o) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  __shared__ float parts[8][ROWS];
  TA* As = reinterpret_cast<TA*>(hy_smem);                     // [ROWS][Kp], Kp = K rounded up to the vector width
  constexpr int VEC = 16 / sizeof(TW);
  const int Kp = (K + VEC - 1) / VEC * VEC;
  const int t0 = blockIdx.y * ROWS;
  constexpr int VA = 16 / sizeof(TA);
  if (K % VA == 0 && lda % VA == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 && Kp == K) {
    const int kv = K / VA;                                     // 16 bytes per thread per load
    for (int i = threadIdx.x; i < ROWS * kv; i += blockDim.x) {
      const int r = i / kv, k = (i % kv) * VA;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (t0 + r < T) v = *reinterpret_cast<const uint4*>(A + (size_t)(t0 + r) * lda + k);
      *reinterpret_cast<uint4*>(As + r * Kp + k) = v;
    }
  } else {
    for (int i = threadIdx.x; i < ROWS * Kp; i += blockDim.x) {
      const int r = i / Kp, k = i % Kp;
      As[i] = (t0 + r < T && k < K) ? A[(size_t)(t0 + r) * lda + k] : from_f<TA>(0.0f);
    }
  }
  __syncthreads();
  // ksplit warps share a column (long k, few columns: more loads in flight); their sums are added in part order
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cpb = 8 / ksplit, part = warp % ksplit, cib = warp / ksplit;
  const int Kc = ((K + ksplit - 1) / ksplit + 32 * VEC - 1) / (32 * VEC) * (32 * VEC);
  const int lo = part * Kc, hi = min(K, lo + Kc);
  for (int base = blockIdx.x * cpb; base < N; base += gridDim.x * cpb) {
    const int n = base + cib;
    float acc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.0f;
    if (n < N) {
      const TW* wr = W + (size_t)n * ldw;
      const bool vec_ok = ((reinterpret_cast<uintptr_t>(wr) & 15) == 0);
      int kdone = lo;
      if (vec_ok) {
        const int kv = min(hi, K / VEC * VEC);
#pragma unroll 4
        for (int k = lo + lane * VEC; k < kv; k += 32 * VEC) {
          const VecN<TW, VEC> wv = *reinterpret_cast<const VecN<TW, VEC>*>(wr + k);
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
            const VecN<TA, VEC> av = *reinterpret_cast<const VecN<TA, VEC>*>(As + r * Kp + k);
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[r] = fmaf(to_f(av.v[j]), to_f(wv.v[j]), acc[r]);
          }
        }
        kdone = max(lo, kv);
      }
      for (int k = kdone + lane; k < hi; k += 32) {
        const float w = to_f(wr[k]);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = fmaf(to_f(As[r * Kp + k]), w, acc[r]);
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) acc[r] = warp_sum(acc[r]);
    }
    if (ksplit > 1) {
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) parts[warp][r] = acc[r];
      }
      __syncthreads();
      if (lane == 0 && part == 0) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          float v = 0.0f;
          for (int p = 0; p < ksplit; ++p) v += parts[warp + p][r];
          acc[r] = v;
        }
      }
    }
    if (lane == 0 && part == 0 && n < N) {
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
        if (t0 + r < T) gemm_store<TO>(o, t0 + r, n, acc[r]);
    }
    if (ksplit > 1) __syncthreads();
  }
}

// ---- short causal convolution over time with a carried tail ------------------------------------------------------------------
// u [T, ldu] (columns col0 .. col0 + C), w [C, taps] (last tap = current token), state [slot][taps - 1][C] fp32 holds the
// last taps - 1 inputs of the request in time order.  Inputs before the request's start are zero.
template <typename AT, typename WT>
__global__ void conv_kernel(Batch b, const AT* __restrict__ u, int ldu, int col0, int C, int taps, const WT* __restrict__ w,
                            const WT* __restrict__ bias, int act_silu, const float* __restrict__ state, AT* __restrict__ out,
                            int ldo) {
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int e = b.tok_ent[t];
  const int start = b.ent_start[e], pos0 = b.ent_pos0[e];
  const int j = t - start;                                   // index inside the entry
  const float* st = state + (size_t)b.ent_slot[e] * (taps - 1) * C;
  float acc = bias ? to_f(bias[c]) : 0.0f;
  for (int i = 0; i < taps; ++i) {
    const int src = j - (taps - 1) + i;
    float v;
    if (src >= 0) v = to_f(u[(size_t)(start + src) * ldu + col0 + c]);
    else if (pos0 + src >= 0) v = st[(size_t)(taps - 1 + src) * C + c];
    else v = 0.0f;
    acc = fmaf(to_f(w[(size_t)c * taps + i]), v, acc);
  }
  if (act_silu) acc = silu_f(acc);
  out[(size_t)t * ldo + c] = from_f<AT>(acc);
}

// New tail = the last taps - 1 of (old tail ++ this entry's inputs).  Runs after conv_kernel of the same step.
constexpr int HY_MAX_TAPS = 16;
template <typename AT>
__global__ void conv_tail_kernel(Batch b, const AT* __restrict__ u, int ldu, int col0, int C, int taps, float* __restrict__ state) {
  const int e = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int start = b.ent_start[e], cnt = b.ent_start[e + 1] - start, pos0 = b.ent_pos0[e];
  float* st = state + (size_t)b.ent_slot[e] * (taps - 1) * C;
  float nv[HY_MAX_TAPS];
  for (int s = 0; s < taps - 1; ++s) {
    const int i = cnt + s;                                   // index in old tail ++ inputs
    float v;
    if (i >= taps - 1) v = to_f(u[(size_t)(start + i - (taps - 1)) * ldu + col0 + c]);
    else v = (pos0 - (taps - 1) + i >= 0) ? st[(size_t)i * C + c] : 0.0f;
    nv[s] = v;
  }
  for (int s = 0; s < taps - 1; ++s) st[(size_t)s * C + c] = nv[s];
}

// ---- key cache: [page][kv head][slot in page][dim] ---------------------------------------------------------------------------
template <typename AT>
__global__ void cache_append_kernel(Batch b, const AT* __restrict__ k, int ldk, int col0, int G, int dim, AT* __restrict__ cache) {
  const int t = blockIdx.x;
  const int e = b.tok_ent[t], pos = b.tok_pos[t];
  const int page = b.pages[(size_t)e * b.max_pages + pos / b.page_size], in_page = pos % b.page_size;
  for (int i = threadIdx.x; i < G * dim; i += blockDim.x) {
    const int g = i / dim, d = i % dim;
    cache[(((size_t)page * G + g) * b.page_size + in_page) * dim + d] = k[(size_t)t * ldk + col0 + i];
  }
}

// ---- causal softmax attention with a sink; values are the keys -----------------------------------------------------------------
// One warp per (token, query head).  Keys are walked in groups of 32 aligned to absolute positions; the running maximum
// starts at the sink logit and the denominator at exp(sink - sink) = 1: the sink has no key and no value.  The query is
// multiplied by its position's temperature in fp32.  The value of a key is its first vdim dimensions (vdim == dim: the
// values are the keys; vdim < dim: a latent followed by a part that only enters the score).  Output: heads concatenated
// [H, vdim], times sigmoid(gate) when there is a gate, times out_scale.
constexpr int HY_ATT_MAXD = 20;     // dims per lane: dim <= 640
template <typename AT, typename WT, typename OT>
__global__ void __launch_bounds__(128) attn_sink_kernel(Batch b, const AT* __restrict__ q, int ldq, const AT* __restrict__ cache,
                                                        const WT* __restrict__ sink, const AT* __restrict__ gate, int ldg,
                                                        int H, int G, int dim, int vdim, float scale, float qt_coef,
                                                        int qt_every, float out_scale, OT* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = reinterpret_cast<float*>(hy_smem) + warp * dim;
  const int unit = blockIdx.x * 4 + warp;
  if (unit >= b.T * H) return;
  const int t = unit / H, h = unit % H;
  const int e = b.tok_ent[t], pos = b.tok_pos[t];
  const int g = h / (H / G);
  const float temp = 1.0f + qt_coef * logf(floorf((float)(pos + 1) / (float)qt_every) + 1.0f);
  for (int d = lane; d < dim; d += 32) qs[d] = to_f(q[(size_t)t * ldq + h * dim + d]) * temp;
  __syncwarp();
  const int* pg = b.pages + (size_t)e * b.max_pages;
  float m = to_f(sink[h]), l = 1.0f;
  float acc[HY_ATT_MAXD];
#pragma unroll
  for (int i = 0; i < HY_ATT_MAXD; ++i) acc[i] = 0.0f;
  for (int j0 = 0; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    const AT* kr = nullptr;
    if (j <= pos) {
      kr = cache + (((size_t)pg[j / b.page_size] * G + g) * b.page_size + j % b.page_size) * dim;
      float dot = 0.0f;
      for (int d = 0; d < dim; ++d) dot = fmaf(qs[d], to_f(kr[d]), dot);
      s = dot * scale;
    }
    const float mn = fmaxf(m, warp_max(s));
    const float corr = expf(m - mn);
    const float p = (j <= pos) ? expf(s - mn) : 0.0f;
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int i = 0; i < HY_ATT_MAXD; ++i) acc[i] *= corr;
    const int cnt = min(32, pos + 1 - j0);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int ja = j0 + jj;
      const AT* kj = cache + (((size_t)pg[ja / b.page_size] * G + g) * b.page_size + ja % b.page_size) * dim;
#pragma unroll
      for (int i = 0; i < HY_ATT_MAXD; ++i) {
        const int d = lane + 32 * i;
        if (d < vdim) acc[i] = fmaf(pj, to_f(kj[d]), acc[i]);
      }
    }
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < HY_ATT_MAXD; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) {
      const float gt = gate ? sigmoid_f(to_f(gate[(size_t)t * ldg + h * vdim + d])) : 1.0f;
      out[(size_t)t * ldo + h * vdim + d] = from_f<OT>(acc[i] * inv * gt * out_scale);
    }
  }
}

// ---- selective scan -------------------------------------------------------------------------------------------------------------
// S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n ; y_c = sum_n S[c, n] C_n + D_c x_c ; out = y silu(z) out_scale.
// L lanes (a power of two) share a channel, each holding NPER states.  dt_raw is the step-size projection before bias
// and softplus.  low [T, ldl] holds [dt-rank part | B | C].  state [slot][inner][nstate] fp32.
// Inputs of HY_SCAN_TB tokens are staged in shared memory by the whole block (one exposed load latency per batch of
// tokens instead of one per token); the recurrence itself then runs out of shared memory and registers.
constexpr int HY_SCAN_TB = 16;
template <typename AT, typename WT, int NPER>
__global__ void __launch_bounds__(128) scan_kernel(Batch b, const AT* __restrict__ x, int ldx, const AT* __restrict__ z, int ldz,
                                                   const float* __restrict__ dt_raw, int lddt, const WT* __restrict__ dt_bias,
                                                   const float* __restrict__ low, int ldl, int col_b, int col_c,
                                                   const float* __restrict__ A, const WT* __restrict__ D, int inner, int nstate,
                                                   int L, float out_scale, float* __restrict__ state, AT* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  const int e = blockIdx.y;
  const int per_block = blockDim.x / L;
  float* sB = reinterpret_cast<float*>(hy_smem);              // [TB][nstate]
  float* sC = sB + HY_SCAN_TB * nstate;                       // [TB][nstate]
  float* sdt = sC + HY_SCAN_TB * nstate;                      // [TB][per_block]
  float* sx = sdt + HY_SCAN_TB * per_block;
  float* sz = sx + HY_SCAN_TB * per_block;
  const int c0 = blockIdx.x * per_block;
  const int cl = threadIdx.x / L;
  const int c = c0 + cl;
  const int sub = threadIdx.x % L;
  const bool live = c < inner;
  const int cc = live ? c : inner - 1;
  const int start = b.ent_start[e], cnt = b.ent_start[e + 1] - start, pos0 = b.ent_pos0[e];
  float* st = state + ((size_t)b.ent_slot[e] * inner + cc) * nstate;
  float S[NPER], a[NPER];
#pragma unroll
  for (int i = 0; i < NPER; ++i) {
    const int n = sub + i * L;
    S[i] = (n < nstate && pos0 > 0) ? st[n] : 0.0f;
    a[i] = n < nstate ? A[(size_t)cc * nstate + n] : 0.0f;
  }
  const float dd = to_f(D[cc]);
  for (int j0 = 0; j0 < cnt; j0 += HY_SCAN_TB) {
    const int nb = min(HY_SCAN_TB, cnt - j0);
    __syncthreads();
    for (int i = threadIdx.x; i < nb * nstate; i += blockDim.x) {
      const int tt = i / nstate, n = i % nstate;
      const size_t row = (size_t)(start + j0 + tt) * ldl;
      sB[tt * nstate + n] = low[row + col_b + n];
      sC[tt * nstate + n] = low[row + col_c + n];
    }
    for (int i = threadIdx.x; i < nb * per_block; i += blockDim.x) {
      const int tt = i / per_block, k = i % per_block;
      const int ch = min(c0 + k, inner - 1);
      const size_t t = (size_t)(start + j0 + tt);
      sdt[i] = softplus_f(dt_raw[t * lddt + ch] + to_f(dt_bias[ch]));
      sx[i] = to_f(x[t * ldx + ch]);
      sz[i] = to_f(z[t * ldz + ch]);
    }
    __syncthreads();
    for (int tt = 0; tt < nb; ++tt) {
      const float dt = sdt[tt * per_block + cl], xv = sx[tt * per_block + cl];
      const float dx = dt * xv;
      float y = 0.0f;
#pragma unroll
      for (int i = 0; i < NPER; ++i) {
        const int n = sub + i * L;
        if (n < nstate) {
          S[i] = fmaf(expf(dt * a[i]), S[i], dx * sB[tt * nstate + n]);
          y = fmaf(S[i], sC[tt * nstate + n], y);
        }
      }
      for (int o = L >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (live && sub == 0) {
        y = fmaf(dd, xv, y);
        out[(size_t)(start + j0 + tt) * ldo + c] = from_f<AT>(y * silu_f(sz[tt * per_block + cl]) * out_scale);
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
      const int n = sub + i * L;
      if (n < nstate) st[n] = S[i];
    }
  }
}

// ---- gated delta rule with one decay per head and key channel ---------------------------------------------------------------------
// Per head, S [dim, vdim] in shared memory, one block per (head, entry), thread j owns column j of S:
//   S <- g * S (rows) ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q   (the read-out sees the current token's write)
// q, k are made unit vectors per head (q also times dim^-1/2); g = exp(-exp(A_log_h) softplus(a + dt_bias));
// out = o / rms(o) * norm_w * sigmoid(gate).  state [slot][H][dim][vdim] fp32.
template <typename AT, typename WT>
__global__ void delta_kernel(Batch b, const AT* __restrict__ qkv, int ldq, int col_q, int col_k, int col_v,
                             const AT* __restrict__ beta_in, int ldb, int col_beta, const float* __restrict__ a_in, int lda,
                             const float* __restrict__ gate_in, int ldg, const WT* __restrict__ A_log,
                             const WT* __restrict__ dt_bias, const WT* __restrict__ norm_w, int H, int G, int dim, int vdim,
                             float eps, float* __restrict__ state, AT* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  float* S = reinterpret_cast<float*>(hy_smem);                // [dim][vdim]
  float* ks = S + (size_t)dim * vdim;
  float* qs = ks + dim;
  float* gs = qs + dim;
  float* red = gs + dim;                                       // 33
  const int h = blockIdx.x, e = blockIdx.y, tid = threadIdx.x;
  const int g = h / (H / G);
  const int start = b.ent_start[e], cnt = b.ent_start[e + 1] - start, pos0 = b.ent_pos0[e];
  float* st = state + ((size_t)b.ent_slot[e] * H + h) * dim * vdim;
  for (int i = tid; i < dim * vdim; i += blockDim.x) S[i] = pos0 > 0 ? st[i] : 0.0f;
  const float rate = expf(to_f(A_log[h]));
  const float qscale = rsqrtf((float)dim);
  __syncthreads();
  for (int j = 0; j < cnt; ++j) {
    const int t = start + j;
    float qv = 0.0f, kv = 0.0f;
    if (tid < dim) {
      qv = to_f(qkv[(size_t)t * ldq + col_q + g * dim + tid]);
      kv = to_f(qkv[(size_t)t * ldq + col_k + g * dim + tid]);
      gs[tid] = expf(-rate * softplus_f(a_in[(size_t)t * lda + h * dim + tid] + to_f(dt_bias[h * dim + tid])));
    }
    const float q2 = block_sum(qv * qv, red);
    const float k2 = block_sum(kv * kv, red);
    if (tid < dim) {
      qs[tid] = qv / sqrtf(q2 + 1e-6f) * qscale;
      ks[tid] = kv / sqrtf(k2 + 1e-6f);
    }
    __syncthreads();
    float o = 0.0f;
    if (tid < vdim) {
      float sk = 0.0f;
      for (int i = 0; i < dim; ++i) {
        const float s = S[i * vdim + tid] * gs[i];
        S[i * vdim + tid] = s;
        sk = fmaf(s, ks[i], sk);
      }
      const float bt = sigmoid_f(to_f(beta_in[(size_t)t * ldb + col_beta + h]));
      const float u = bt * (to_f(qkv[(size_t)t * ldq + col_v + h * vdim + tid]) - sk);
      for (int i = 0; i < dim; ++i) {
        const float s = fmaf(ks[i], u, S[i * vdim + tid]);
        S[i * vdim + tid] = s;
        o = fmaf(s, qs[i], o);
      }
    }
    const float o2 = block_sum(tid < vdim ? o * o : 0.0f, red);
    if (tid < vdim) {
      const float r = o / sqrtf(o2 / (float)vdim + eps);
      const float gt = sigmoid_f(gate_in[(size_t)t * ldg + h * vdim + tid]);
      out[(size_t)t * ldo + h * vdim + tid] = from_f<AT>(r * to_f(norm_w[tid]) * gt);
    }
  }
  __syncthreads();
  for (int i = tid; i < dim * vdim; i += blockDim.x) st[i] = S[i];
}

// Sum of two values over the block in one pass (same order rules as block_sum).  red: >= 66 floats.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = warp_sum(a); b = warp_sum(b);
  __syncthreads();
  if (lane == 0) { red[w] = a; red[33 + w] = b; }
  __syncthreads();
  if (w == 0) {
    float sa = lane < nw ? red[lane] : 0.0f, sb = lane < nw ? red[33 + lane] : 0.0f;
    sa = warp_sum(sa); sb = warp_sum(sb);
    if (lane == 0) { red[32] = sa; red[65] = sb; }
  }
  __syncthreads();
  return make_float2(red[32], red[65]);
}

// The same recurrence with thread j keeping column j of S in registers (key size <= DR): no shared-memory traffic for
// the state, four partial sums per dot product so the per-token chain is short.  Same results up to summation order.
// Inputs of HY_DELTA_TB tokens are staged by the whole block; unit vectors and decays of those tokens are made by one
// warp per token (shuffles only), the per-token recurrence then runs without any block barrier, and the output norms of
// the batch are again made by one warp per token: four barriers per batch of tokens instead of seven per token.
constexpr int HY_DELTA_TB = 16;

// PARTS neighbouring lanes share a column of S, each keeping DR / PARTS of its rows in registers (PARTS > 1 ends each dot
// product in log2(PARTS) shuffles).  Measured at key size 128, 128 value columns: PARTS = 1 (one warp per scheduler, 128
// rows in registers) 2.1 us per token, PARTS = 4 (four warps per scheduler) 3.6 us: the chain through shuffles and the
// read-out store costs more than the shorter loops save, so the dispatcher uses PARTS = 1.
template <typename AT, typename WT, int DR, int PARTS>
__global__ void __launch_bounds__(DR / PARTS > 32 ? 256 : 512)
delta_reg_kernel(Batch b, const AT* __restrict__ qkv, int ldq, int col_q, int col_k, int col_v,
                 const AT* __restrict__ beta_in, int ldb, int col_beta, const float* __restrict__ a_in, int lda,
                 const float* __restrict__ gate_in, int ldg, const WT* __restrict__ A_log, const WT* __restrict__ dt_bias,
                 const WT* __restrict__ norm_w, int H, int G, int dim, int vdim, float eps, float* __restrict__ state,
                 AT* __restrict__ out, int ldo) {
  constexpr int RP = DR / PARTS;
  extern __shared__ __align__(16) unsigned char hy_smem[];
  const int nt = blockDim.x, nwarps = nt >> 5, nc = nt / PARTS;
  float* sq = reinterpret_cast<float*>(hy_smem);               // [TB][DR] unit queries (times dim^-1/2)
  float* skk = sq + HY_DELTA_TB * DR;                           // [TB][DR] unit keys
  float* sa = skk + HY_DELTA_TB * DR;                           // [TB][DR] decays
  float* sv = sa + HY_DELTA_TB * DR;                            // [TB][nc] values
  float* sg = sv + HY_DELTA_TB * nc;                            // [TB][nc] output gates (pre-sigmoid)
  float* so = sg + HY_DELTA_TB * nc;                            // [TB][nc] raw read-outs
  float* sbeta = so + HY_DELTA_TB * nc;                         // [TB]
  const int h = blockIdx.x, e = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int jc = tid / PARTS, r0 = (tid % PARTS) * RP;
  const int g = h / (H / G);
  const int start = b.ent_start[e], cnt = b.ent_start[e + 1] - start, pos0 = b.ent_pos0[e];
  float* st = state + ((size_t)b.ent_slot[e] * H + h) * dim * vdim;
  const bool col = jc < vdim;
  float S[RP];
#pragma unroll
  for (int i = 0; i < RP; ++i) S[i] = (col && r0 + i < dim && pos0 > 0) ? st[(size_t)(r0 + i) * vdim + jc] : 0.0f;
  const float rate = expf(to_f(A_log[h]));
  const float qscale = rsqrtf((float)dim);
  for (int j0 = 0; j0 < cnt; j0 += HY_DELTA_TB) {
    const int nb = min(HY_DELTA_TB, cnt - j0);
    __syncthreads();                                           // the previous batch is finished with the staging area
    for (int i = tid; i < nb * DR; i += nt) {
      const int tt = i / DR, k = i % DR;
      const size_t t = (size_t)(start + j0 + tt);
      const bool ok = k < dim;
      sq[i] = ok ? to_f(qkv[t * ldq + col_q + g * dim + k]) : 0.0f;
      skk[i] = ok ? to_f(qkv[t * ldq + col_k + g * dim + k]) : 0.0f;
      sa[i] = ok ? expf(-rate * softplus_f(a_in[t * lda + h * dim + k] + to_f(dt_bias[h * dim + k]))) : 1.0f;
    }
    for (int i = tid; i < nb * nc; i += nt) {
      const int tt = i / nc, k = i % nc;
      const size_t t = (size_t)(start + j0 + tt);
      sv[i] = k < vdim ? to_f(qkv[t * ldq + col_v + h * vdim + k]) : 0.0f;
      sg[i] = k < vdim ? gate_in[t * ldg + h * vdim + k] : 0.0f;
    }
    if (tid < nb) sbeta[tid] = sigmoid_f(to_f(beta_in[(size_t)(start + j0 + tid) * ldb + col_beta + h]));
    __syncthreads();
    for (int tt = warp; tt < nb; tt += nwarps) {               // unit vectors: one warp per token
      float q2 = 0.0f, k2 = 0.0f;
      for (int k = lane; k < DR; k += 32) { q2 = fmaf(sq[tt * DR + k], sq[tt * DR + k], q2); k2 = fmaf(skk[tt * DR + k], skk[tt * DR + k], k2); }
      q2 = warp_sum(q2); k2 = warp_sum(k2);
      const float qi = qscale / sqrtf(q2 + 1e-6f), ki = 1.0f / sqrtf(k2 + 1e-6f);
      for (int k = lane; k < DR; k += 32) { sq[tt * DR + k] *= qi; skk[tt * DR + k] *= ki; }
    }
    __syncthreads();
    for (int tt = 0; tt < nb; ++tt) {
      const float* gs = sa + tt * DR + r0;
      const float* ks = skk + tt * DR + r0;
      const float* qs = sq + tt * DR + r0;
      float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
      for (int i = 0; i < RP; i += 4) {
        const float4 g4 = *reinterpret_cast<const float4*>(&gs[i]);
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[i]);
        S[i] *= g4.x; S[i + 1] *= g4.y; S[i + 2] *= g4.z; S[i + 3] *= g4.w;
        p0 = fmaf(S[i], k4.x, p0); p1 = fmaf(S[i + 1], k4.y, p1);
        p2 = fmaf(S[i + 2], k4.z, p2); p3 = fmaf(S[i + 3], k4.w, p3);
      }
      float sk = (p0 + p1) + (p2 + p3);
#pragma unroll
      for (int o = 1; o < PARTS; o <<= 1) sk += __shfl_xor_sync(0xffffffffu, sk, o);
      const float u = sbeta[tt] * (sv[tt * nc + jc] - sk);
      p0 = p1 = p2 = p3 = 0.0f;
#pragma unroll
      for (int i = 0; i < RP; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[i]);
        const float4 q4 = *reinterpret_cast<const float4*>(&qs[i]);
        S[i] = fmaf(k4.x, u, S[i]); S[i + 1] = fmaf(k4.y, u, S[i + 1]);
        S[i + 2] = fmaf(k4.z, u, S[i + 2]); S[i + 3] = fmaf(k4.w, u, S[i + 3]);
        p0 = fmaf(S[i], q4.x, p0); p1 = fmaf(S[i + 1], q4.y, p1);
        p2 = fmaf(S[i + 2], q4.z, p2); p3 = fmaf(S[i + 3], q4.w, p3);
      }
      float ov = (p0 + p1) + (p2 + p3);
#pragma unroll
      for (int o = 1; o < PARTS; o <<= 1) ov += __shfl_xor_sync(0xffffffffu, ov, o);
      if (tid % PARTS == 0) so[tt * nc + jc] = ov;
    }
    __syncthreads();
    for (int tt = warp; tt < nb; tt += nwarps) {               // output norm and gate: one warp per token
      float o2 = 0.0f;
      for (int k = lane; k < vdim; k += 32) o2 = fmaf(so[tt * nc + k], so[tt * nc + k], o2);
      o2 = warp_sum(o2);
      const float inv = 1.0f / sqrtf(o2 / (float)vdim + eps);
      for (int k = lane; k < vdim; k += 32)
        out[(size_t)(start + j0 + tt) * ldo + h * vdim + k] =
            from_f<AT>(so[tt * nc + k] * inv * to_f(norm_w[k]) * sigmoid_f(sg[tt * nc + k]));
    }
  }
  if (col) {
#pragma unroll
    for (int i = 0; i < RP; ++i)
      if (r0 + i < dim) st[(size_t)(r0 + i) * vdim + jc] = S[i];
  }
}

// ---- sampling: argmax, or Gumbel-max at a temperature with a counter-based generator ---------------------------------------------
__device__ __forceinline__ uint32_t mix32(uint64_t key, uint32_t ctr) {
  uint64_t z = key + 0x9E3779B97F4A7C15ull * (uint64_t)(ctr + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return (uint32_t)((z ^ (z >> 31)) >> 32);
}
__global__ void sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature, uint64_t seed,
                              int* __restrict__ out) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  const int r = blockIdx.x;
  const float temp = temperature ? temperature[r] : 0.0f;
  float best = -INFINITY;
  int besti = 0x7fffffff;
  for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
    float s = logits[(size_t)r * vocab + v];
    if (temp > 0.0f) {
      const float uu = ((float)mix32(seed + (uint64_t)r * 0x100000001B3ull, (uint32_t)v) + 0.5f) * (1.0f / 4294967296.0f);
      s = s / temp - logf(-logf(uu));
    }
    if (s > best || (s == best && v < besti)) { best = s; besti = v; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) { bv[w] = best; bi[w] = besti; }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? bv[lane] : -INFINITY;
    besti = lane < nw ? bi[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
    }
    if (lane == 0) out[r] = besti;
  }
}

}  // namespace hy
