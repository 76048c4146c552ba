// hy_mixers.cuh — device kernels of three more mixers of the layered hybrid decoders (libjf_hybrid.so):
//   * a state-space recurrence with ONE decay per head (the scalar-decay form of the selective scan) and its gated,
//     grouped output norm;
//   * attention over a shared low-rank latent: the cache holds, per token, the normed latent and one rotated key part that
//     all heads share.  The per-head key up-projection is folded into the query and the value up-projection is applied
//     after the weighted sum, so attention itself runs over the cache rows as they are: one "key head" of size
//     rank + rot whose first `rank` dimensions are also the values (the sink-attention kernels serve it);
//   * a gated linear recurrence whose forget gate, bounded below per channel, also sets what is written.
// Same precision rule as hy_kernels.cuh: norms, angles, decays, gates, step sizes and states are fp32 (angles fp64).
#pragma once
#include "hy_kernels.cuh"
#include "jf_ptx.cuh"

namespace hy {

// ---- rotation of dimension pairs (2i, 2i + 1) -------------------------------------------------------------------------
// Frequencies come from a host-made fp64 table (any interpolation of the frequencies is already in it); the angle is
// formed and reduced in fp64, cosine and sine are multiplied by `mag` and enter the fp32 computation.
struct Rotation { const double* freq; int pairs; float mag; };

__device__ __forceinline__ void rotation_row(const Rotation& r, int pos, float* cs /* [2 * pairs] in shared memory */) {
  for (int i = threadIdx.x; i < r.pairs; i += blockDim.x) {
    double s, c;
    sincos((double)pos * r.freq[i], &s, &c);
    cs[2 * i] = (float)c * r.mag;
    cs[2 * i + 1] = (float)s * r.mag;
  }
}

// ---- state-space recurrence, one decay per head ----------------------------------------------------------------------------
// Per head h (group g = h / (heads / groups)), channel p, state n:
//   dt = softplus(dt_raw_h + dt_bias_h) ; S[p, n] <- exp(-exp(A_log_h) dt) S[p, n] + dt x_p B_n ; y_p = sum_n S[p, n] C_n + D_h x_p
// L lanes share a channel, each holding NPER CONSECUTIVE states in registers (state sizes up to NPER * L; B and C are
// staged zero-padded to that size, so the inner loop has no bounds checks and reads them four at a time).  xbc [T, ldx]:
// x at column 0 (heads * vdim), B at col_b, C at col_c (groups * nstate each), after convolution and activation.
// state [slot][heads * vdim][nstate] fp32.  y leaves in fp32 (it enters a norm).  Inputs of HY_SSD_TB tokens (fewer for 256 states and more) are staged per
// block as fp32; a block's 128 / L channels lie in one head.  Per token a thread spends about 3.5 instructions per state
// plus a short shuffle tree: measured, the per-token overhead (indices, conversions, bounds, a 5-step tree for 4 states)
// was four fifths of an earlier one-state-per-lane layout's instructions.
constexpr int HY_SSD_TB = 32;
template <typename AT, int NPER, int L>
__global__ void __launch_bounds__(128) ssd_scan_kernel(Batch b, const AT* __restrict__ xbc, int ldx, int col_b, int col_c,
                                                       const AT* __restrict__ dt_raw, int lddt, const float* __restrict__ dt_bias,
                                                       const float* __restrict__ A_log, const float* __restrict__ D, int heads,
                                                       int vdim, int nstate, int groups, int blocks_per_head,
                                                       float* __restrict__ state, float* __restrict__ y, int ldy) {
  constexpr int NP = NPER * L, PB = 128 / L, TB = NP >= 512 ? HY_SSD_TB / 4 : NP >= 256 ? HY_SSD_TB / 2 : HY_SSD_TB;
  __shared__ __align__(16) float sB[TB * NP];
  __shared__ __align__(16) float sC[TB * NP];
  __shared__ float sx[TB * PB];
  __shared__ float sdt[TB], sdec[TB];
  const int e = blockIdx.y;
  const int h = blockIdx.x / blocks_per_head;
  const int p0 = (blockIdx.x % blocks_per_head) * PB;
  const int g = h / (heads / groups);
  const int cl = threadIdx.x / L, sub = threadIdx.x % L, n0 = sub * NPER;
  const int p = p0 + cl;
  const bool live = p < vdim;
  const int pc = live ? p : vdim - 1;
  const int start = b.ent_start[e], cnt = b.ent_start[e + 1] - start, pos0 = b.ent_pos0[e];
  float* st = state + (((size_t)b.ent_slot[e] * heads + h) * vdim + pc) * nstate;
  float S[NPER];
#pragma unroll
  for (int i = 0; i < NPER; ++i) S[i] = (n0 + i < nstate && pos0 > 0) ? st[n0 + i] : 0.0f;
  const float rate = expf(A_log[h]), dd = D[h], bias = dt_bias[h];
  const AT* xb = xbc + col_b + g * nstate;
  const AT* xc = xbc + col_c + g * nstate;
  const AT* xx = xbc + h * vdim;
  float* yp = y + h * vdim + p;
  // long entries: the raw inputs of the NEXT batch of tokens are fetched into registers before the current batch runs
  constexpr int UB = TB * NP / 128, UX = (TB * PB + 127) / 128;
  const bool ahead = cnt > TB;
  AT rb[UB], rc[UB], rx[UX], rdt = from_f<AT>(0.0f);
  auto fetch = [&](int j0, int nb) {
#pragma unroll
    for (int u = 0; u < UB; ++u) {
      const int i = threadIdx.x + u * 128, tt = i / NP, n = i % NP;
      const bool ok = tt < nb && n < nstate;
      const size_t row = (size_t)(start + j0 + tt) * ldx;
      rb[u] = ok ? xb[row + n] : from_f<AT>(0.0f);
      rc[u] = ok ? xc[row + n] : from_f<AT>(0.0f);
    }
#pragma unroll
    for (int u = 0; u < UX; ++u) {
      const int i = threadIdx.x + u * 128, tt = i / PB, k = i % PB;
      rx[u] = tt < nb ? xx[(size_t)(start + j0 + tt) * ldx + min(p0 + k, vdim - 1)] : from_f<AT>(0.0f);
    }
    if (threadIdx.x < nb) rdt = dt_raw[(size_t)(start + j0 + threadIdx.x) * lddt + h];
  };
  if (ahead) fetch(0, min(TB, cnt));
  for (int j0 = 0; j0 < cnt; j0 += TB) {
    const int nb = min(TB, cnt - j0);
    __syncthreads();
    if (ahead) {
#pragma unroll
      for (int u = 0; u < UB; ++u) {
        const int i = threadIdx.x + u * 128;
        sB[i] = to_f(rb[u]);
        sC[i] = to_f(rc[u]);
      }
#pragma unroll
      for (int u = 0; u < UX; ++u) {
        const int i = threadIdx.x + u * 128;
        if (i < TB * PB) sx[i] = to_f(rx[u]);
      }
      if (threadIdx.x < nb) {
        const float dt = softplus_f(to_f(rdt) + bias);
        sdt[threadIdx.x] = dt;
        sdec[threadIdx.x] = expf(-rate * dt);
      }
    } else {
#pragma unroll 4
    for (int i = threadIdx.x; i < nb * NP; i += 128) {
      const int tt = i / NP, n = i % NP;
      const size_t row = (size_t)(start + j0 + tt) * ldx;
      const bool ok = n < nstate;
      sB[i] = ok ? to_f(xb[row + n]) : 0.0f;
      sC[i] = ok ? to_f(xc[row + n]) : 0.0f;
    }
    for (int i = threadIdx.x; i < nb * PB; i += 128) {
      const int tt = i / PB, k = i % PB;
      sx[i] = to_f(xx[(size_t)(start + j0 + tt) * ldx + min(p0 + k, vdim - 1)]);
    }
    if (threadIdx.x < nb) {
      const float dt = softplus_f(to_f(dt_raw[(size_t)(start + j0 + threadIdx.x) * lddt + h]) + bias);
      sdt[threadIdx.x] = dt;
      sdec[threadIdx.x] = expf(-rate * dt);
    }
    }
    __syncthreads();
    if (ahead && j0 + TB < cnt) fetch(j0 + TB, min(TB, cnt - j0 - TB));
    float* yr = yp + (size_t)(start + j0) * ldy;
    for (int tt = 0; tt < nb; ++tt, yr += ldy) {
      const float dec = sdec[tt], xv = sx[tt * PB + cl];
      const float dx = sdt[tt] * xv;
      float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
      if constexpr (NPER % 4 == 0) {
        const float4* b4 = reinterpret_cast<const float4*>(sB + tt * NP + n0);
        const float4* c4 = reinterpret_cast<const float4*>(sC + tt * NP + n0);
#pragma unroll
        for (int i = 0; i < NPER / 4; ++i) {
          const float4 bv = b4[i], cv = c4[i];
          S[4 * i] = fmaf(dec, S[4 * i], dx * bv.x);         a0 = fmaf(S[4 * i], cv.x, a0);
          S[4 * i + 1] = fmaf(dec, S[4 * i + 1], dx * bv.y); a1 = fmaf(S[4 * i + 1], cv.y, a1);
          S[4 * i + 2] = fmaf(dec, S[4 * i + 2], dx * bv.z); a2 = fmaf(S[4 * i + 2], cv.z, a2);
          S[4 * i + 3] = fmaf(dec, S[4 * i + 3], dx * bv.w); a3 = fmaf(S[4 * i + 3], cv.w, a3);
        }
      } else {
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
          S[i] = fmaf(dec, S[i], dx * sB[tt * NP + n0 + i]);
          a0 = fmaf(S[i], sC[tt * NP + n0 + i], a0);
        }
      }
      float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
      for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && sub == 0) *yr = fmaf(dd, xv, acc);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPER; ++i)
      if (n0 + i < nstate) st[n0 + i] = S[i];
  }
}

// Gate, then norm: v = y silu(z); each of `parts` equal slices of a row is divided by its own root mean square; times w.
template <typename AT>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, int ldy, const AT* __restrict__ z, int ldz,
                                        const float* __restrict__ w, int inner, int parts, float eps, AT* __restrict__ out,
                                        int ldo) {
  __shared__ float red[33];
  const int t = blockIdx.x, part = blockIdx.y, n = inner / parts, c0 = part * n;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = y[(size_t)t * ldy + c0 + c] * silu_f(to_f(z[(size_t)t * ldz + c0 + c]));
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = y[(size_t)t * ldy + c0 + c] * silu_f(to_f(z[(size_t)t * ldz + c0 + c]));
    out[(size_t)t * ldo + c0 + c] = from_f<AT>(v * inv * w[c0 + c]);
  }
}

// ---- attention over a shared latent -------------------------------------------------------------------------------------------
// After the merged down-projections (fp32, [query latent | key/value latent | raw rotated key part]):
//   query latent  -> RMS norm, weight, into cq (operand of the query up-projection);
//   key latent    -> RMS norm, weight, into the token's cache row, dimensions [0, rank);
//   rotated part  -> rotation at the token's position, into the cache row, dimensions [rank, rank + rot).
// A layer that borrows another layer's cache has no key part (own_kv = 0).  Cache: [page][slot in page][rank + rot].
template <typename AT>
__global__ void latent_prep_kernel(Batch b, const float* __restrict__ d, int ldd, int q_rank, int rank, int rot, int own_kv,
                                   const float* __restrict__ qn_w, const float* __restrict__ kn_w, float eps, Rotation r,
                                   AT* __restrict__ cq, int ldq, AT* __restrict__ cache) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  float* cs = reinterpret_cast<float*>(hy_smem);              // [2 * pairs]
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* row = d + (size_t)t * ldd;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x) cq[(size_t)t * ldq + c] = from_f<AT>(row[c] * inv * qn_w[c]);
  if (!own_kv) return;
  const int e = b.tok_ent[t], pos = b.tok_pos[t];
  AT* dst = cache + ((size_t)b.pages[(size_t)e * b.max_pages + pos / b.page_size] * b.page_size + pos % b.page_size) * (rank + rot);
  const float* kr = row + q_rank;
  ss = 0.0f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) ss = fmaf(kr[c], kr[c], ss);
  ss = block_sum(ss, red);
  inv = 1.0f / sqrtf(ss / (float)rank + eps);
  for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_f<AT>(kr[c] * inv * kn_w[c]);
  rotation_row(r, pos, cs);
  __syncthreads();
  const float* kp = kr + rank;
  for (int i = threadIdx.x; i < rot; i += blockDim.x) {
    float v = kp[i];
    if (i < 2 * r.pairs) {
      const float c = cs[i & ~1], s = cs[i | 1];
      v = (i & 1) ? fmaf(kp[i], c, kp[i - 1] * s) : fmaf(kp[i], c, -kp[i + 1] * s);
    }
    dst[rank + i] = from_f<AT>(v);
  }
}

// The query as the cache rows want it: per (token, head)  [ W_uk_h^T q_unrotated  (rank) | rotated q part (rot) ].
// q [T, ldq] holds heads of [dim | rot]; w_uk [H * dim, rank] row-major (thread r walks a column: coalesced across r).
// A block serves HY_LAT_TB tokens of one head and 128 output dimensions, so a weight element is read once per 8 tokens.
constexpr int HY_LAT_TB = 8;
// fold == 0: only the rotated part is written (a few-row step folds the key up-projection with head_rows_kernel).
template <typename AT, typename WT>
__global__ void __launch_bounds__(128) latent_query_kernel(Batch b, const AT* __restrict__ q, int ldq, const WT* __restrict__ w_uk,
                                                           int H, int dim, int rot, int rank, int fold, Rotation r,
                                                           AT* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  float* qs = reinterpret_cast<float*>(hy_smem);              // [TB][dim]
  float* cs = qs + HY_LAT_TB * dim;                           // [2 * pairs] of one token at a time
  const int t0 = blockIdx.x * HY_LAT_TB, h = blockIdx.y, nb = min(HY_LAT_TB, b.T - t0);
  for (int i = threadIdx.x; i < HY_LAT_TB * dim; i += blockDim.x) {
    const int tt = i / dim, k = i % dim;
    qs[i] = tt < nb ? to_f(q[(size_t)(t0 + tt) * ldq + h * (dim + rot) + k]) : 0.0f;
  }
  __syncthreads();
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  if (fold && c < rank) {
    float acc[HY_LAT_TB];
#pragma unroll
    for (int tt = 0; tt < HY_LAT_TB; ++tt) acc[tt] = 0.0f;
    const WT* wc = w_uk + (size_t)h * dim * rank + c;
    for (int k = 0; k < dim; ++k) {
      const float w = to_f(wc[(size_t)k * rank]);
#pragma unroll
      for (int tt = 0; tt < HY_LAT_TB; ++tt) acc[tt] = fmaf(qs[tt * dim + k], w, acc[tt]);
    }
    for (int tt = 0; tt < nb; ++tt) out[(size_t)(t0 + tt) * ldo + h * (rank + rot) + c] = from_f<AT>(acc[tt]);
  }
  if (blockIdx.z != 0) return;
  for (int tt = 0; tt < nb; ++tt) {
    __syncthreads();
    rotation_row(r, b.tok_pos[t0 + tt], cs);
    __syncthreads();
    const AT* qp = q + (size_t)(t0 + tt) * ldq + h * (dim + rot) + dim;
    for (int i = threadIdx.x; i < rot; i += blockDim.x) {
      float v = to_f(qp[i]);
      if (i < 2 * r.pairs) {
        const float cc = cs[i & ~1], ss = cs[i | 1];
        v = (i & 1) ? fmaf(v, cc, to_f(qp[i - 1]) * ss) : fmaf(v, cc, -to_f(qp[i + 1]) * ss);
      }
      out[(size_t)(t0 + tt) * ldo + h * (rank + rot) + rank + i] = from_f<AT>(v);
    }
  }
}

// The value up-projection behind the weighted sum: out[t, h, j] = sum_r w_uvT[h][r][j] o[t, h, r]  (o fp32: the weighted
// sum of latents; w_uvT is the value up-projection transposed per head at load so that thread j reads coalesced).
template <typename AT, typename WT>
__global__ void __launch_bounds__(128) latent_value_kernel(int T, const float* __restrict__ o, int ldi, const WT* __restrict__ w_uvT,
                                                           int H, int rank, int vdim, AT* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  float* os = reinterpret_cast<float*>(hy_smem);              // [TB][rank]
  const int t0 = blockIdx.x * HY_LAT_TB, h = blockIdx.y, nb = min(HY_LAT_TB, T - t0);
  for (int i = threadIdx.x; i < HY_LAT_TB * rank; i += blockDim.x) {
    const int tt = i / rank, k = i % rank;
    os[i] = tt < nb ? o[(size_t)(t0 + tt) * ldi + h * rank + k] : 0.0f;
  }
  __syncthreads();
  const int j = blockIdx.z * blockDim.x + threadIdx.x;
  if (j >= vdim) return;
  float acc[HY_LAT_TB];
#pragma unroll
  for (int tt = 0; tt < HY_LAT_TB; ++tt) acc[tt] = 0.0f;
  const WT* wc = w_uvT + (size_t)h * rank * vdim + j;
  for (int k = 0; k < rank; ++k) {
    const float w = to_f(wc[(size_t)k * vdim]);
#pragma unroll
    for (int tt = 0; tt < HY_LAT_TB; ++tt) acc[tt] = fmaf(os[tt * rank + k], w, acc[tt]);
  }
  for (int tt = 0; tt < nb; ++tt) out[(size_t)(t0 + tt) * ldo + h * vdim + j] = from_f<AT>(acc[tt]);
}

// Few rows (decode steps): out[t, h, n] = sum_k in[t, h, k] w[h][n][k] for up to 8 rows t.  One warp per (h, n) walks a
// weight row 16 bytes per lane (both per-head projections around the attention are stored [n][k] for this kernel as well),
// so the weights stream once at full width instead of one block per head walking them column by column.
template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(256) head_rows_kernel(int T, const TI* __restrict__ in, int ldi, int in_hs, const TW* __restrict__ w,
                                                        int H, int N, int K, TO* __restrict__ out, int ldo, int out_hs) {
  constexpr int VEC = 16 / sizeof(TW);
  const int lane = threadIdx.x & 31;
  const int id = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (id >= H * N) return;
  const int h = id / N, n = id % N;
  const TW* wr = w + ((size_t)h * N + n) * K;
  float acc[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) acc[t] = 0.0f;
  if (K % VEC == 0 && (reinterpret_cast<uintptr_t>(wr) & 15) == 0) {
    for (int k = lane * VEC; k < K; k += 32 * VEC) {
      const VecN<TW, VEC> wv = *reinterpret_cast<const VecN<TW, VEC>*>(wr + k);
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        if (t >= T) break;
        const TI* ir = in + (size_t)t * ldi + h * in_hs + k;
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[t] = fmaf(to_f(ir[j]), to_f(wv.v[j]), acc[t]);
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float wv = to_f(wr[k]);
#pragma unroll
      for (int t = 0; t < 8; ++t)
        if (t < T) acc[t] = fmaf(to_f(in[(size_t)t * ldi + h * in_hs + k]), wv, acc[t]);
    }
  }
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    if (t >= T) break;
    const float v = warp_sum(acc[t]);
    if (lane == 0) out[(size_t)t * ldo + h * out_hs + n] = from_f<TO>(v);
  }
}

// ---- gated linear recurrence ------------------------------------------------------------------------------------------------------
// Per head, S [dim, vdim]:  f = lower + (1 - lower) sigmoid(f_raw + f_bias)  (per key channel)
//   S <- diag(f) S + (1 - f) v^T ; o = S^T silu(q_raw) ; out = o / rms(o) * norm_w  (norm over the head's vdim).
// in [T, ld]: q_raw at col_q, f_raw at col_f (heads * dim each), v at col_v (heads * vdim).  state [slot][H][dim][vdim].
// Thread j keeps column j of S in registers (key size <= DR); inputs of HY_GLR_TB tokens are staged by the block, the
// output norms of the batch are made by one warp per token.
constexpr int HY_GLR_TB = 16;
// With 128 threads or more, the raw inputs of the NEXT 16 tokens are fetched into registers before the current 16 run and
// are activated into shared memory afterwards: one block per head leaves nothing else on its SM to hide the loads behind
// (measured: the waits for staged loads were the largest stall of the kernel).
template <typename AT, int DR>
__global__ void __launch_bounds__(DR > 64 ? 256 : 512)
glr_reg_kernel(Batch b, const AT* __restrict__ in, int ld, int col_q, int col_f, int col_v, const float* __restrict__ f_bias,
               const float* __restrict__ lower, const float* __restrict__ norm_w, int H, int dim, int vdim, float eps,
               float* __restrict__ state, AT* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  constexpr int TB = HY_GLR_TB, UQ = TB * DR / 128;            // q / f elements per thread and batch when nt >= 128
  const int nt = blockDim.x, nwarps = nt >> 5;
  float* sq = reinterpret_cast<float*>(hy_smem);               // [TB][DR] activated queries
  float* sf = sq + TB * DR;                                    // [TB][DR] forget gates
  float* sv = sf + TB * DR;                                    // [TB][nt] values
  float* so = sv + TB * nt;                                    // [TB][nt] raw read-outs
  const int h = blockIdx.x, e = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int start = b.ent_start[e], cnt = b.ent_start[e + 1] - start, pos0 = b.ent_pos0[e];
  float* st = state + ((size_t)b.ent_slot[e] * H + h) * dim * vdim;
  const bool col = tid < vdim;
  const bool ahead = nt >= 128 && cnt > TB;                   // short entries (decode steps) stage directly
  float S[DR];
#pragma unroll
  for (int i = 0; i < DR; ++i) S[i] = (col && i < dim && pos0 > 0) ? st[(size_t)i * vdim + tid] : 0.0f;
  AT rq[UQ], rf[UQ], rv[TB];
  const AT* inq = in + col_q + h * dim;
  const AT* inf = in + col_f + h * dim;
  const AT* inv = in + col_v + h * vdim + (col ? tid : 0);
  auto fetch = [&](int j0, int nb) {
#pragma unroll
    for (int u = 0; u < UQ; ++u) {
      const int i = tid + u * nt, tt = i / DR, k = i % DR;
      const bool ok = i < nb * DR && k < dim;
      const size_t row = (size_t)(start + j0 + tt) * ld;
      rq[u] = ok ? inq[row + k] : from_f<AT>(0.0f);
      rf[u] = ok ? inf[row + k] : from_f<AT>(0.0f);
    }
#pragma unroll
    for (int u = 0; u < TB; ++u) rv[u] = (u < nb && col) ? inv[(size_t)(start + j0 + u) * ld] : from_f<AT>(0.0f);
  };
  auto activate = [&](int nb) {
#pragma unroll
    for (int u = 0; u < UQ; ++u) {
      const int i = tid + u * nt, k = i % DR;
      if (i < nb * DR) {
        const bool ok = k < dim;
        const float lo = ok ? lower[h * dim + k] : 0.0f;
        sq[i] = ok ? silu_f(to_f(rq[u])) : 0.0f;
        sf[i] = ok ? fmaf(1.0f - lo, sigmoid_f(to_f(rf[u]) + f_bias[h * dim + k]), lo) : 1.0f;
      }
    }
#pragma unroll
    for (int u = 0; u < TB; ++u)
      if (u < nb) sv[u * nt + tid] = to_f(rv[u]);
  };
  if (ahead) fetch(0, min(TB, cnt));
  for (int j0 = 0; j0 < cnt; j0 += TB) {
    const int nb = min(TB, cnt - j0);
    __syncthreads();
    if (ahead) {
      activate(nb);
    } else {
      for (int i = tid; i < nb * DR; i += nt) {
        const int tt = i / DR, k = i % DR;
        const size_t t = (size_t)(start + j0 + tt);
        const bool ok = k < dim;
        sq[i] = ok ? silu_f(to_f(in[t * ld + col_q + h * dim + k])) : 0.0f;
        const float lo = ok ? lower[h * dim + k] : 0.0f;
        sf[i] = ok ? fmaf(1.0f - lo, sigmoid_f(to_f(in[t * ld + col_f + h * dim + k]) + f_bias[h * dim + k]), lo) : 1.0f;
      }
      for (int i = tid; i < nb * nt; i += nt) {
        const int tt = i / nt, k = i % nt;
        sv[i] = k < vdim ? to_f(in[(size_t)(start + j0 + tt) * ld + col_v + h * vdim + k]) : 0.0f;
      }
    }
    __syncthreads();
    if (ahead && j0 + TB < cnt) fetch(j0 + TB, min(TB, cnt - j0 - TB));
    for (int tt = 0; tt < nb; ++tt) {
      const float* fs = sf + tt * DR;
      const float* qs = sq + tt * DR;
      const float v = sv[tt * nt + tid];
      float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
      for (int i = 0; i < DR; i += 4) {                        // S <- f S + (1 - f) v, written as v + f (S - v)
        const float4 f4 = *reinterpret_cast<const float4*>(&fs[i]);
        const float4 q4 = *reinterpret_cast<const float4*>(&qs[i]);
        S[i] = fmaf(f4.x, S[i] - v, v); S[i + 1] = fmaf(f4.y, S[i + 1] - v, v);
        S[i + 2] = fmaf(f4.z, S[i + 2] - v, v); S[i + 3] = fmaf(f4.w, S[i + 3] - v, v);
        p0 = fmaf(S[i], q4.x, p0); p1 = fmaf(S[i + 1], q4.y, p1);
        p2 = fmaf(S[i + 2], q4.z, p2); p3 = fmaf(S[i + 3], q4.w, p3);
      }
      so[tt * nt + tid] = (p0 + p1) + (p2 + p3);
    }
    __syncthreads();
    for (int tt = warp; tt < nb; tt += nwarps) {
      float o2 = 0.0f;
      for (int k = lane; k < vdim; k += 32) o2 = fmaf(so[tt * nt + k], so[tt * nt + k], o2);
      o2 = warp_sum(o2);
      const float inv = 1.0f / sqrtf(o2 / (float)vdim + eps);
      for (int k = lane; k < vdim; k += 32)
        out[(size_t)(start + j0 + tt) * ldo + h * vdim + k] = from_f<AT>(so[tt * nt + k] * inv * norm_w[k]);
    }
  }
  if (col) {
#pragma unroll
    for (int i = 0; i < DR; ++i)
      if (i < dim) st[(size_t)i * vdim + tid] = S[i];
  }
}

// The same recurrence for any head size whose state fits shared memory: S [dim][vdim] in shared memory, a thread walks
// the columns j = tid, tid + blockDim, ...; one token at a time.
template <typename AT>
__global__ void __launch_bounds__(256)
glr_kernel(Batch b, const AT* __restrict__ in, int ld, int col_q, int col_f, int col_v, const float* __restrict__ f_bias,
           const float* __restrict__ lower, const float* __restrict__ norm_w, int H, int dim, int vdim, float eps,
           float* __restrict__ state, AT* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  float* S = reinterpret_cast<float*>(hy_smem);                // [dim][vdim]
  float* qs = S + (size_t)dim * vdim;                          // [dim]
  float* fs = qs + dim;                                        // [dim]
  float* os = fs + dim;                                        // [vdim]
  float* red = os + vdim;                                      // 33
  const int h = blockIdx.x, e = blockIdx.y, tid = threadIdx.x;
  const int start = b.ent_start[e], cnt = b.ent_start[e + 1] - start, pos0 = b.ent_pos0[e];
  float* st = state + ((size_t)b.ent_slot[e] * H + h) * dim * vdim;
  for (int i = tid; i < dim * vdim; i += blockDim.x) S[i] = pos0 > 0 ? st[i] : 0.0f;
  for (int j = 0; j < cnt; ++j) {
    const size_t t = (size_t)(start + j);
    __syncthreads();
    for (int k = tid; k < dim; k += blockDim.x) {
      qs[k] = silu_f(to_f(in[t * ld + col_q + h * dim + k]));
      const float lo = lower[h * dim + k];
      fs[k] = fmaf(1.0f - lo, sigmoid_f(to_f(in[t * ld + col_f + h * dim + k]) + f_bias[h * dim + k]), lo);
    }
    __syncthreads();
    float o2 = 0.0f;
    for (int c = tid; c < vdim; c += blockDim.x) {
      const float v = to_f(in[t * ld + col_v + h * vdim + c]);
      float o = 0.0f;
      for (int i = 0; i < dim; ++i) {
        const float s = fmaf(fs[i], S[(size_t)i * vdim + c] - v, v);
        S[(size_t)i * vdim + c] = s;
        o = fmaf(s, qs[i], o);
      }
      os[c] = o;
      o2 = fmaf(o, o, o2);
    }
    o2 = block_sum(o2, red);
    const float inv = 1.0f / sqrtf(o2 / (float)vdim + eps);
    for (int c = tid; c < vdim; c += blockDim.x) out[t * ldo + h * vdim + c] = from_f<AT>(os[c] * inv * norm_w[c]);
  }
  __syncthreads();
  for (int i = tid; i < dim * vdim; i += blockDim.x) st[i] = S[i];
}

// ---- matrix memory with exponential gates under a running maximum ----------------------------------------------------------------
// Per head, S [dim, vdim], n [dim], m (all zero at the start of a sequence, m too):
//   li = cap tanh((i_raw + i_bias) / cap) ; lf = logsigmoid(cap tanh((f_raw + f_bias) / cap))        (cap <= 0: no cap)
//   m' = max(lf + m, li) ; a = exp(lf + m - m') ; c = exp(li - m')
//   S <- a S + c k v^T ; n <- a n + c k ; o = S^T q / (max(|n . q|, exp(-m')) + 1e-6) ,  q = q_raw dim^(-1/2)
//   out = o / rms(o) * norm_w[head] * sigmoid(g)        (norm over the head's vdim)
// The normaliser n is carried as one more value column whose value is always one: column vdim of the state, so n . q is
// that column's read-out.  in [T, ld]: q, k at col_q, col_k (heads * dim each), v, g at col_v, col_g (heads * vdim);
// gates [T, ldg] fp32: i_raw at col_i + head, f_raw at col_f + head.  state [slot][H][dim * (vdim + 1) + 1], m last.
// Thread j keeps column j of the state in registers (key size <= DR); inputs of 16 or 32 tokens are staged by the
// block (for long entries the next batch's raw rows travel by asynchronous copies while the current one runs), the gates' scalar
// chain is replayed per token by one thread per token side by side, one warp per token makes the output norm.
__host__ __device__ constexpr int mlstm_tb(int dr) { return dr > 64 ? 16 : 32; }   // tokens per staged batch of the register kernel
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float cap_f(float z, float cap) { return cap > 0.0f ? cap * tanhf(z / cap) : z; }

template <typename AT, int DR>
__global__ void __launch_bounds__(256)
mlstm_reg_kernel(Batch b, const AT* __restrict__ in, int ld, int col_q, int col_k, int col_v, int col_g,
                 const float* __restrict__ gates, int ldg, int col_i, int col_f, const float* __restrict__ i_bias,
                 const float* __restrict__ f_bias, const float* __restrict__ norm_w, int H, int dim, int vdim, float cap,
                 float eps, int async_ok, float* __restrict__ state, AT* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  constexpr int TB = mlstm_tb(DR), CH = 16 / (int)sizeof(AT);  // elements per 16-byte copy
  const int nt = blockDim.x, nwarps = nt >> 5;
  float* sq = reinterpret_cast<float*>(hy_smem);               // [TB][DR] scaled queries
  float* sk = sq + TB * DR;                                    // [TB][DR] keys
  float* sv = sk + TB * DR;                                    // [TB][nt] values, a one in column vdim
  float* so = sv + TB * nt;                                    // [TB][nt] read-outs
  float* sgt = so + TB * nt;                                   // [TB][nt] output gates sigmoid(g)
  float* sg = sgt + TB * nt;                                   // [5][TB]: li, lf, a, c, exp(-m); then m of even / odd batches
  float* graw = sg + 5 * TB + 4;                               // [2][2][TB] raw gate pre-activations of the batch in flight
  AT* raw = reinterpret_cast<AT*>(graw + 4 * TB);              // [2][TB][2 DR + 2 nt] raw q | k | v | g rows in flight
  const int rw = 2 * DR + 2 * nt;
  const int h = blockIdx.x, e = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int start = b.ent_start[e], cnt = b.ent_start[e + 1] - start, pos0 = b.ent_pos0[e];
  const int vs = vdim + 1;
  float* st = state + ((size_t)b.ent_slot[e] * H + h) * ((size_t)dim * vs + 1);
  const bool col = tid < vs;
  // long entries: the next batch's raw rows travel to shared memory by asynchronous 16-byte copies while the current batch
  // runs (needs rows that start and end on 16-byte boundaries); short entries (decode steps) and odd sizes stage directly
  const bool ahead = async_ok && cnt > TB;
  float S[DR];
#pragma unroll
  for (int i = 0; i < DR; ++i) S[i] = (col && i < dim && pos0 > 0) ? st[(size_t)i * vs + tid] : 0.0f;
  if (tid == 0) sg[5 * TB] = pos0 > 0 ? st[(size_t)dim * vs] : 0.0f;
  const float qscale = 1.0f / sqrtf((float)dim);
  const float ib = i_bias[h], fb = f_bias[h];
  const int qc = dim / CH, vc = vdim / CH, per_tok = 2 * qc + 2 * vc;
  auto fetch = [&](int j0, int nb, int buf) {
    AT* dst = raw + (size_t)buf * TB * rw;
    for (int i = tid; i < nb * per_tok; i += nt) {
      const int tt = i / per_tok, c = i % per_tok;
      const AT* row = in + (size_t)(start + j0 + tt) * ld;
      const AT* src; AT* d = dst + (size_t)tt * rw;
      if (c < qc) { src = row + col_q + h * dim + c * CH; d += c * CH; }
      else if (c < 2 * qc) { src = row + col_k + h * dim + (c - qc) * CH; d += DR + (c - qc) * CH; }
      else if (c < 2 * qc + vc) { src = row + col_v + h * vdim + (c - 2 * qc) * CH; d += 2 * DR + (c - 2 * qc) * CH; }
      else { src = row + col_g + h * vdim + (c - 2 * qc - vc) * CH; d += 2 * DR + nt + (c - 2 * qc - vc) * CH; }
      jf::cp_async_16(d, src, 16u);
    }
    if (tid < nb) {
      jf::cp_async_4(graw + (buf * 2) * TB + tid, gates + (size_t)(start + j0 + tid) * ldg + col_i + h);
      jf::cp_async_4(graw + (buf * 2 + 1) * TB + tid, gates + (size_t)(start + j0 + tid) * ldg + col_f + h);
    }
    jf::cp_async_commit();
  };
  if (ahead) fetch(0, min(TB, cnt), 0);
  int par = 0;
  for (int j0 = 0; j0 < cnt; j0 += TB, par ^= 1) {
    const int nb = min(TB, cnt - j0);
    if (ahead) jf::cp_async_wait_all();
    __syncthreads();
    if (ahead) {
      const AT* src = raw + (size_t)par * TB * rw;
      for (int i = tid; i < nb * DR; i += nt) {
        const int tt = i / DR, k = i % DR;
        const bool ok = k < dim;
        sq[i] = ok ? to_f(src[(size_t)tt * rw + k]) * qscale : 0.0f;
        sk[i] = ok ? to_f(src[(size_t)tt * rw + DR + k]) : 0.0f;
      }
      for (int tt = 0; tt < nb; ++tt) {
        sv[tt * nt + tid] = tid < vdim ? to_f(src[(size_t)tt * rw + 2 * DR + tid]) : tid == vdim ? 1.0f : 0.0f;
        sgt[tt * nt + tid] = tid < vdim ? sigmoid_f(to_f(src[(size_t)tt * rw + 2 * DR + nt + tid])) : 0.0f;
      }
      if (tid < nb) {
        sg[tid] = cap_f(graw[(par * 2) * TB + tid] + ib, cap);
        sg[TB + tid] = log_sigmoid_f(cap_f(graw[(par * 2 + 1) * TB + tid] + fb, cap));
      }
    } else {
      for (int i = tid; i < nb * DR; i += nt) {
        const int tt = i / DR, k = i % DR;
        const size_t t = (size_t)(start + j0 + tt);
        const bool ok = k < dim;
        sq[i] = ok ? to_f(in[t * ld + col_q + h * dim + k]) * qscale : 0.0f;
        sk[i] = ok ? to_f(in[t * ld + col_k + h * dim + k]) : 0.0f;
      }
      for (int i = tid; i < nb * nt; i += nt) {
        const int tt = i / nt, k = i % nt;
        const size_t t = (size_t)(start + j0 + tt);
        sv[i] = k < vdim ? to_f(in[t * ld + col_v + h * vdim + k]) : k == vdim ? 1.0f : 0.0f;
        sgt[i] = k < vdim ? sigmoid_f(to_f(in[t * ld + col_g + h * vdim + k])) : 0.0f;
      }
      if (tid < nb) {
        const size_t t = (size_t)(start + j0 + tid);
        sg[tid] = cap_f(gates[t * ldg + col_i + h] + ib, cap);
        sg[TB + tid] = log_sigmoid_f(cap_f(gates[t * ldg + col_f + h] + fb, cap));
      }
    }
    __syncthreads();
    // the running maximum is a chain of additions and maxima: thread tt replays it up to its token (the same operations in
    // the same order as a serial walk), the exponentials of all tokens are then taken side by side
    if (tid < nb) {
      float m = sg[5 * TB + par], mp = m;
      for (int r = 0; r <= tid; ++r) { mp = m; m = fmaxf(sg[TB + r] + m, sg[r]); }
      sg[2 * TB + tid] = expf(sg[TB + tid] + mp - m);
      sg[3 * TB + tid] = expf(sg[tid] - m);
      sg[4 * TB + tid] = expf(-m);
      if (tid == nb - 1) sg[5 * TB + (par ^ 1)] = m;
    }
    if (ahead && j0 + TB < cnt) fetch(j0 + TB, min(TB, cnt - j0 - TB), par ^ 1);     // that buffer was read before the barrier above
    __syncthreads();
    for (int tt = 0; tt < nb; ++tt) {
      const float* ks = sk + tt * DR;
      const float* qs = sq + tt * DR;
      const float a = sg[2 * TB + tt];
      const float cv = sg[3 * TB + tt] * sv[tt * nt + tid];
      float p0 = 0.0f, p1 = 0.0f, p2 = 0.0f, p3 = 0.0f;
#pragma unroll
      for (int i = 0; i < DR; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[i]);
        const float4 q4 = *reinterpret_cast<const float4*>(&qs[i]);
        S[i] = fmaf(a, S[i], cv * k4.x); S[i + 1] = fmaf(a, S[i + 1], cv * k4.y);
        S[i + 2] = fmaf(a, S[i + 2], cv * k4.z); S[i + 3] = fmaf(a, S[i + 3], cv * k4.w);
        p0 = fmaf(S[i], q4.x, p0); p1 = fmaf(S[i + 1], q4.y, p1);
        p2 = fmaf(S[i + 2], q4.z, p2); p3 = fmaf(S[i + 3], q4.w, p3);
      }
      so[tt * nt + tid] = (p0 + p1) + (p2 + p3);
    }
    __syncthreads();
    for (int tt = warp; tt < nb; tt += nwarps) {
      const float den = 1.0f / (fmaxf(fabsf(so[tt * nt + vdim]), sg[4 * TB + tt]) + 1e-6f);
      float o2 = 0.0f;
      for (int k = lane; k < vdim; k += 32) { const float o = so[tt * nt + k] * den; o2 = fmaf(o, o, o2); }
      o2 = warp_sum(o2);
      const float inv = den / sqrtf(o2 / (float)vdim + eps);
      const size_t t = (size_t)(start + j0 + tt);
      for (int k = lane; k < vdim; k += 32)
        out[t * ldo + h * vdim + k] = from_f<AT>(so[tt * nt + k] * inv * norm_w[h * vdim + k] * sgt[tt * nt + k]);
    }
  }
  if (col) {
#pragma unroll
    for (int i = 0; i < DR; ++i)
      if (i < dim) st[(size_t)i * vs + tid] = S[i];
  }
  __syncthreads();
  if (tid == 0) st[(size_t)dim * vs] = sg[5 * TB + par];
}

// The same recurrence for any head size whose state fits shared memory: S [dim][vdim + 1] in shared memory, a thread walks
// the columns j = tid, tid + blockDim, ...; one token at a time.
template <typename AT>
__global__ void __launch_bounds__(256)
mlstm_kernel(Batch b, const AT* __restrict__ in, int ld, int col_q, int col_k, int col_v, int col_g,
             const float* __restrict__ gates, int ldg, int col_i, int col_f, const float* __restrict__ i_bias,
             const float* __restrict__ f_bias, const float* __restrict__ norm_w, int H, int dim, int vdim, float cap, float eps,
             float* __restrict__ state, AT* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  const int vs = vdim + 1;
  float* S = reinterpret_cast<float*>(hy_smem);                // [dim][vs]
  float* qs = S + (size_t)dim * vs;                            // [dim]
  float* ks = qs + dim;                                        // [dim]
  float* os = ks + dim;                                        // [vs]
  float* red = os + vs;                                        // 33
  const int h = blockIdx.x, e = blockIdx.y, tid = threadIdx.x;
  const int start = b.ent_start[e], cnt = b.ent_start[e + 1] - start, pos0 = b.ent_pos0[e];
  float* st = state + ((size_t)b.ent_slot[e] * H + h) * ((size_t)dim * vs + 1);
  for (int i = tid; i < dim * vs; i += blockDim.x) S[i] = pos0 > 0 ? st[i] : 0.0f;
  float m = pos0 > 0 ? st[(size_t)dim * vs] : 0.0f;            // every thread carries the scalar chain
  const float qscale = 1.0f / sqrtf((float)dim);
  for (int j = 0; j < cnt; ++j) {
    const size_t t = (size_t)(start + j);
    __syncthreads();
    for (int k = tid; k < dim; k += blockDim.x) {
      qs[k] = to_f(in[t * ld + col_q + h * dim + k]) * qscale;
      ks[k] = to_f(in[t * ld + col_k + h * dim + k]);
    }
    const float li = cap_f(gates[t * ldg + col_i + h] + i_bias[h], cap);
    const float lf = log_sigmoid_f(cap_f(gates[t * ldg + col_f + h] + f_bias[h], cap));
    const float mn = fmaxf(lf + m, li);
    const float a = expf(lf + m - mn), cc = expf(li - mn), em = expf(-mn);
    m = mn;
    __syncthreads();
    for (int c = tid; c < vs; c += blockDim.x) {
      const float v = c < vdim ? to_f(in[t * ld + col_v + h * vdim + c]) : 1.0f;
      const float cv = cc * v;
      float o = 0.0f;
      for (int i = 0; i < dim; ++i) {
        const float s = fmaf(a, S[(size_t)i * vs + c], cv * ks[i]);
        S[(size_t)i * vs + c] = s;
        o = fmaf(s, qs[i], o);
      }
      os[c] = o;
    }
    __syncthreads();
    const float den = 1.0f / (fmaxf(fabsf(os[vdim]), em) + 1e-6f);
    float o2 = 0.0f;
    for (int c = tid; c < vdim; c += blockDim.x) { const float o = os[c] * den; o2 = fmaf(o, o, o2); }
    o2 = block_sum(o2, red);
    const float inv = den / sqrtf(o2 / (float)vdim + eps);
    for (int c = tid; c < vdim; c += blockDim.x) {
      const float gt = sigmoid_f(to_f(in[t * ld + col_g + h * vdim + c]));
      out[t * ldo + h * vdim + c] = from_f<AT>(os[c] * inv * norm_w[h * vdim + c] * gt);
    }
  }
  __syncthreads();
  for (int i = tid; i < dim * vs; i += blockDim.x) st[i] = S[i];
  if (tid == 0) st[(size_t)dim * vs] = m;
}

}  // namespace hy
