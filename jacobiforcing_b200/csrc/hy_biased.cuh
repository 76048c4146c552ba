// hy_biased.cuh — pre-norm blocks with input convolutions, a per-layer token input and an average over the depth, and
// their mixer: softmax attention with capped scores, a logarithmic distance bias, a sliding window plus kept first
// tokens and a sink in the denominator (libjf_hybrid.so).
//
//   embed_pair   x = table[token] * scale + pair[(prev * a + token * b) mod n]   (row n for a request's first token; the
//                previous token of a portion's first token comes from the request's state slot)
//   stream_row   one block per token: x += m * ls * y (a sublayer's rows or the mixture of a routed feed-forward), then
//                the token input  y = P (gelu_tanh(G x) * e),  x += m * y / rms(y) * w,  then the depth average
//                (X_n <- x;  x <- sum_j a_j X_j), then the next sublayer's RMS norm into an fp32 row
//   canon        h + sum_i w[:, i] h_(t - taps + 1 + i) over the normed rows with the carried tail, into the operand type
//   prep         values blended with the first blending layer's, keys and values into their pages
//   attend       SIMT (one warp per (token, head)) or mma.sync tiles of 64 rows x 64 keys (bf16 build)
//
// Visible keys of position i: j <= i with i - j < window (window 0: all) or j < keep.  They are walked in a fixed order
// (kept first tokens outside the window by position, then the window by position) in groups / tiles aligned to absolute
// positions, so a position's result does not depend on the step's cut or on the batch.  Scores, cap, bias, softmax and
// the sink are fp32.  Cache layouts: keys [page][kv head][slot][dim], values [page][kv head][slot][vdim].
#pragma once
#include "hy_kernels.cuh"
#include "hy_attn.cuh"

namespace hy {

struct BiasedCfg {
  int H, G, dim, vdim, window, keep;
  float scale, cap;
  const float* r1; const float* r2; const float* sink;       // [H] each, fp32
};

// ---- embedding with a hashed pair table -----------------------------------------------------------------------------------------
// prev_tok [slots]: the last token each request fed.  kept: NULL or the first plane of the depth average's store.
template <typename WT>
__global__ void embed_pair_kernel(Batch b, const WT* __restrict__ table, float scale, const WT* __restrict__ pair, int buckets,
                                  int mul_prev, int mul_cur, const int* __restrict__ prev_tok, int width, float* __restrict__ x,
                                  float* __restrict__ kept) {
  const int t = blockIdx.x;
  const int tok = b.tok[t], e = b.tok_ent[t];
  long long row = -1;
  if (buckets > 0) {
    const int j = t - b.ent_start[e];
    if (j > 0 || b.ent_pos0[e] > 0) {
      const long long prev = j > 0 ? b.tok[t - 1] : prev_tok[b.ent_slot[e]];
      row = (prev * (long long)mul_prev + (long long)tok * (long long)mul_cur) % (long long)buckets;
      if (row < 0) row += buckets;
    } else {
      row = buckets;
    }
  }
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = to_f(table[(size_t)tok * width + c]) * scale;
    if (row >= 0) v += to_f(pair[(size_t)row * width + c]);
    x[(size_t)t * width + c] = v;
    if (kept) kept[(size_t)t * width + c] = v;
  }
}

// after embed_pair_kernel of the same step: the request's last token of this step
__global__ void prev_token_kernel(Batch b, int* __restrict__ prev_tok) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e < b.E) prev_tok[b.ent_slot[e]] = b.tok[b.ent_start[e + 1] - 1];
}

// ---- one token's row of the stream ------------------------------------------------------------------------------------------------
struct StreamOp {
  const float* y; int ldy;                                   // a sublayer's rows [T, ldy], or
  const float* rows; int ldr; const int* pair_row; const float* wts; int top;   // the mixture sum_k wts[t, k] rows[pair_row[t top + k]]
  const float* ls; float mult;                               // x += mult * ls * y  (ls NULL: one; y and rows NULL: nothing added)
  const void* side_gate; const void* side_proj; const float* side_norm; const void* side_table;   // side_proj: [side_dim, width]
  int side_ld, side_col0, side_dim;                          // token input: table row slice [side_col0, + side_dim)
  float* kept; size_t kept_stride; int kept_n; const float* dwa;   // kept[kept_n] <- x;  x <- sum_{j <= kept_n} dwa[j] kept[j]
  const float* next_w; float* next_out;                      // next_out[t] <- x / rms(x) * next_w  (fp32)
  float eps;
};

template <typename WT>
__global__ void __launch_bounds__(256) stream_row_kernel(Batch b, StreamOp o, int width, float* __restrict__ x) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  float* xs = reinterpret_cast<float*>(hy_smem);             // [width] the row
  float* ys = xs + width;                                    // [width] the token input's row
  float* gs = ys + width;                                    // [side_dim]
  __shared__ float red[33];
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = x[(size_t)t * width + c];
    if (o.y || o.rows) {
      float y;
      if (o.rows) {
        y = 0.0f;
        for (int k = 0; k < o.top; ++k) {
          const int i = t * o.top + k;
          y = fmaf(o.wts[i], o.rows[(size_t)(o.pair_row ? o.pair_row[i] : i) * o.ldr + c], y);
        }
      } else {
        y = o.y[(size_t)t * o.ldy + c];
      }
      v = fmaf(o.mult * (o.ls ? o.ls[c] : 1.0f), y, v);
    }
    xs[c] = v;
  }
  __syncthreads();
  if (o.side_dim > 0) {
    const WT* gate = (const WT*)o.side_gate;                 // [side_dim, width]
    const WT* projT = (const WT*)o.side_proj;                // [side_dim, width]: the projection, transposed
    const WT* erow = (const WT*)o.side_table + (size_t)b.tok[t] * o.side_ld + o.side_col0;
    constexpr int VEC = 16 / (int)sizeof(WT);
    if (width % VEC == 0) {
      // a warp owns up to four gate rows at a time; every chunk of the row read from shared memory serves all four
      for (int base = 0; base < o.side_dim; base += nw * 4) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int c = lane * VEC; c < width; c += 32 * VEC) {
          float xv[VEC];
#pragma unroll
          for (int j = 0; j < VEC; j += 4) *reinterpret_cast<float4*>(&xv[j]) = *reinterpret_cast<const float4*>(&xs[c + j]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int d = base + warp + nw * i;
            if (d < o.side_dim) {
              const VecN<WT, VEC> gv = *reinterpret_cast<const VecN<WT, VEC>*>(gate + (size_t)d * width + c);
#pragma unroll
              for (int j = 0; j < VEC; ++j) acc[i] = fmaf(xv[j], to_f(gv.v[j]), acc[i]);
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int d = base + warp + nw * i;
          const float dot = warp_sum(acc[i]);
          if (lane == 0 && d < o.side_dim) gs[d] = gelu_tanh_f(dot) * to_f(erow[d]);
        }
      }
    } else {
      for (int d = warp; d < o.side_dim; d += nw) {
        float dot = 0.0f;
        for (int c = lane; c < width; c += 32) dot = fmaf(xs[c], to_f(gate[(size_t)d * width + c]), dot);
        dot = warp_sum(dot);
        if (lane == 0) gs[d] = gelu_tanh_f(dot) * to_f(erow[d]);
      }
    }
    __syncthreads();
    float ss = 0.0f;
    if (width % 4 == 0) {
      for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
        float y[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int d = 0; d < o.side_dim; ++d) {
          const VecN<WT, 4> pv = *reinterpret_cast<const VecN<WT, 4>*>(projT + (size_t)d * width + c);
          const float g = gs[d];
#pragma unroll
          for (int j = 0; j < 4; ++j) y[j] = fmaf(to_f(pv.v[j]), g, y[j]);
        }
        *reinterpret_cast<float4*>(&ys[c]) = make_float4(y[0], y[1], y[2], y[3]);
#pragma unroll
        for (int j = 0; j < 4; ++j) ss = fmaf(y[j], y[j], ss);
      }
    } else {
      for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float y = 0.0f;
        for (int d = 0; d < o.side_dim; ++d) y = fmaf(to_f(projT[(size_t)d * width + c]), gs[d], y);
        ys[c] = y;
        ss = fmaf(y, y, ss);
      }
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)width + o.eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = fmaf(o.mult * o.side_norm[c], ys[c] * inv, xs[c]);
  }
  if (o.kept) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      const float own = xs[c];
      o.kept[(size_t)o.kept_n * o.kept_stride + (size_t)t * width + c] = own;
      float a = 0.0f;
      for (int j = 0; j < o.kept_n; ++j) a = fmaf(o.dwa[j], o.kept[(size_t)j * o.kept_stride + (size_t)t * width + c], a);
      xs[c] = fmaf(o.dwa[o.kept_n], own, a);
    }
  }
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {    // a thread reads back only what it wrote itself
    const float v = xs[c];
    x[(size_t)t * width + c] = v;
    ss = fmaf(v, v, ss);
  }
  if (!o.next_w) return;
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + o.eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) o.next_out[(size_t)t * width + c] = xs[c] * inv * o.next_w[c];
}

// ---- a sublayer's input: the normed row plus its causal convolution over time ------------------------------------------------------
// hn [T, width] fp32 normed rows; w [taps, width] fp32 (tap-major; last tap = the current token); state [slot][taps - 1][width] fp32 =
// the request's last taps - 1 normed rows.  taps == 0: the normed row passes as it is.
template <typename AT, int CH>
__global__ void canon_kernel(Batch b, const float* __restrict__ hn, int width, int taps, const float* __restrict__ w,
                             const float* __restrict__ state, AT* __restrict__ out) {
  struct alignas(4 * CH) Row { float v[CH]; };                        // CH consecutive channels per thread (width % CH == 0)
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * CH;
  if (c >= width) return;
  Row acc = *reinterpret_cast<const Row*>(hn + (size_t)t * width + c);
  if (taps > 0) {
    const int e = b.tok_ent[t];
    const int start = b.ent_start[e], pos0 = b.ent_pos0[e], j = t - start;
    const float* st = state + (size_t)b.ent_slot[e] * (taps - 1) * width;
    for (int i = 0; i < taps; ++i) {
      const int src = j - (taps - 1) + i;
      const float* row = src >= 0 ? hn + (size_t)(start + src) * width : pos0 + src >= 0 ? st + (size_t)(taps - 1 + src) * width : nullptr;
      if (!row) continue;
      const Row r = *reinterpret_cast<const Row*>(row + c), wv = *reinterpret_cast<const Row*>(w + (size_t)i * width + c);
#pragma unroll
      for (int k = 0; k < CH; ++k) acc.v[k] = fmaf(wv.v[k], r.v[k], acc.v[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < CH; ++k) out[(size_t)t * width + c + k] = from_f<AT>(acc.v[k]);
}

// ---- values blended with the first blending layer's; keys and values into their pages ----------------------------------------------
// mix: 0 = values as projected; 1 = this is the first blending layer: its values also go to vfirst [T, ldvf]; 2 = v <-
// (1 - lambda) v + lambda vfirst[t].  What is cached is the blended value.
template <typename AT>
__global__ void __launch_bounds__(128) biased_prep_kernel(Batch b, const AT* __restrict__ in, int ld, int col_k, int col_v, int G,
                                                          int dim, int vdim, int mix, float lambda, AT* __restrict__ vfirst, int ldvf,
                                                          AT* __restrict__ kc, AT* __restrict__ vc) {
  const int t = blockIdx.x;
  const int e = b.tok_ent[t], pos = b.tok_pos[t];
  const int page = b.pages[(size_t)e * b.max_pages + pos / b.page_size], in_page = pos % b.page_size;
  const AT* row = in + (size_t)t * ld;
  for (int i = threadIdx.x; i < G * dim; i += blockDim.x) {
    const int g = i / dim, d = i % dim;
    kc[(((size_t)page * G + g) * b.page_size + in_page) * dim + d] = row[col_k + i];
  }
  for (int i = threadIdx.x; i < G * vdim; i += blockDim.x) {
    const int g = i / vdim, d = i % vdim;
    AT v = row[col_v + i];
    if (mix == 1) vfirst[(size_t)t * ldvf + i] = v;
    else if (mix == 2) v = from_f<AT>(fmaf(lambda, to_f(vfirst[(size_t)t * ldvf + i]), (1.0f - lambda) * to_f(v)));
    vc[(((size_t)page * G + g) * b.page_size + in_page) * vdim + d] = v;
  }
}

// ---- attention, one warp per (token, query head) -------------------------------------------------------------------------------------
// The running maximum starts at the sink logit and the denominator at exp(sink - sink) = 1: the sink has no key, no value,
// no scale, no cap and no bias.
template <typename AT, typename OT>
__global__ void __launch_bounds__(128) biased_attn_kernel(Batch b, const AT* __restrict__ q, int ldq, BiasedCfg c,
                                                          const AT* __restrict__ kc, const AT* __restrict__ vc,
                                                          OT* __restrict__ out, int ldo) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = reinterpret_cast<float*>(hy_smem) + warp * c.dim;
  const int unit = blockIdx.x * 4 + warp;
  if (unit >= b.T * c.H) return;
  const int t = unit / c.H, h = unit % c.H;
  const int e = b.tok_ent[t], pos = b.tok_pos[t];
  const int g = h / (c.H / c.G);
  for (int d = lane; d < c.dim; d += 32) qs[d] = to_f(q[(size_t)t * ldq + h * c.dim + d]);
  __syncwarp();
  const int* pg = b.pages + (size_t)e * b.max_pages;
  const int w0 = c.window > 0 ? max(0, pos - c.window + 1) : 0;                     // first token of the window
  const int nk = min(c.keep, w0);                                                   // kept first tokens outside the window
  const int n = nk + pos + 1 - w0;
  const float r1 = c.r1[h], r2 = c.r2[h];
  float m = c.sink[h], l = 1.0f;
  float acc[HY_ATT_MAXD];
#pragma unroll
  for (int i = 0; i < HY_ATT_MAXD; ++i) acc[i] = 0.0f;
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int idx = i0 + lane;
    float s = -INFINITY;
    if (idx < n) {
      const int j = idx < nk ? idx : w0 + idx - nk;
      const AT* kr = kc + (((size_t)pg[j / b.page_size] * c.G + g) * b.page_size + j % b.page_size) * c.dim;
      float dot = 0.0f;
      for (int d = 0; d < c.dim; ++d) dot = fmaf(qs[d], to_f(kr[d]), dot);
      s = dot * c.scale;
      if (c.cap > 0.0f) s = c.cap * tanhf(s / c.cap);
      s -= r1 * log1pf(r2 * (float)(pos - j));
    }
    const float mn = fmaxf(m, warp_max(s));
    const float corr = expf(m - mn);
    const float p = idx < n ? expf(s - mn) : 0.0f;
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int i = 0; i < HY_ATT_MAXD; ++i) acc[i] *= corr;
    const int cnt = min(32, n - i0);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int ix = i0 + jj, j = ix < nk ? ix : w0 + ix - nk;
      const AT* vr = vc + (((size_t)pg[j / b.page_size] * c.G + g) * b.page_size + j % b.page_size) * c.vdim;
#pragma unroll
      for (int i = 0; i < HY_ATT_MAXD; ++i) {
        const int d = lane + 32 * i;
        if (d < c.vdim) acc[i] = fmaf(pj, to_f(vr[d]), acc[i]);
      }
    }
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < HY_ATT_MAXD; ++i) {
    const int d = lane + 32 * i;
    if (d < c.vdim) out[(size_t)t * ldo + h * c.vdim + d] = from_f<OT>(acc[i] * inv);
  }
}

// ---- the same attention on tensor cores (bf16 build) ----------------------------------------------------------------------------
// Work unit = (entry, key head, tile of 64 query rows); rows are (token, query head of the group) pairs, token-major, so
// the heads that share a key head share every tile that is loaded.  A unit walks tiles of 64 keys aligned to absolute
// positions: first the tiles of kept first tokens that lie before its first window tile, then the tiles from the first
// row's window to the last row's position; each row masks what it does not see.  S = Q K^T by mma.sync m16n8k16 (bf16
// operands, fp32 accumulators); scale, cap, distance bias and the online softmax in fp32; O += P V with P split into a
// bf16 head and a bf16 remainder (the weights stay 32-bit in effect).  The sink joins the denominator at the end.  Key and
// value rows are zero-padded to DP columns in shared memory (dim, vdim multiples of 8, at most DP); key / value tiles are
// double buffered.  With n_splits > 1 (steps of few rows, decoding) a unit's tile list is cut into n_splits runs, each run
// leaves (maximum, denominator, unnormalised output) per row, and biased_combine_kernel merges them with the sink.  tanh and the logarithm use the fast exponential / logarithm units: 1 - 2 / (exp(2 z) + 1) and
// log(1 + r2 d), both far inside the rounding of the bf16 operands.
template <int DP>
__global__ void __launch_bounds__(128) biased_mma_kernel(Batch b, const AttnUnit* __restrict__ units, const bf16* __restrict__ q,
                                                         int ldq, BiasedCfg c, const bf16* __restrict__ kc,
                                                         const bf16* __restrict__ vc, bf16* __restrict__ out, int ldo,
                                                         int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
  constexpr int LD = DP + 8;                            // padded row (elements): ldmatrix rows fall into distinct banks
  extern __shared__ __align__(16) unsigned char hy_smem[];
  bf16* kbuf = reinterpret_cast<bf16*>(hy_smem);        // [2][64 * LD] key tiles: one in use, one in flight
  bf16* vbuf = kbuf + 2 * 64 * LD;                      // [2][64 * LD] value tiles; the query tile sits in the first one at the start
  const AttnUnit u = units[blockIdx.x];
  const int R = c.H / c.G;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int start = b.ent_start[u.entry], cnt = b.ent_start[u.entry + 1] - start, pos0 = b.ent_pos0[u.entry];
  const int rows_total = cnt * R;
  const int* pg = b.pages + (size_t)u.entry * b.max_pages;
  const int kchunks = c.dim / 8, vchunks = c.vdim / 8;
  for (int i = tid; i < 64 * (DP / 8); i += 128) {
    const int r = i / (DP / 8), ch = i % (DP / 8);
    const int row = u.row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows_total && ch < kchunks)
      v = *reinterpret_cast<const uint4*>(q + (size_t)(start + row / R) * ldq + (u.kv_head * R + row % R) * c.dim + ch * 8);
    *reinterpret_cast<uint4*>(&vbuf[r * LD + ch * 8]) = v;
  }
  __syncthreads();
  uint32_t qa[DP / 16][4];
  {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk)
      jf::ldmatrix_x4(jf::smem_u32(&vbuf[r * LD + kk * 16 + (lane >> 4) * 8]), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
  }
  __syncthreads();                                       // the query tile has been read: its buffer takes value tiles now
  const int r_lo = u.row0 + warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const bool v_lo = r_lo < rows_total, v_hi = r_hi < rows_total;
  const int p_lo = v_lo ? pos0 + r_lo / R : -1, p_hi = v_hi ? pos0 + r_hi / R : -1;
  const int h_lo = u.kv_head * R + r_lo % R, h_hi = u.kv_head * R + r_hi % R;
  const float r1_lo = c.r1[h_lo], r2_lo = c.r2[h_lo], r1_hi = c.r1[h_hi], r2_hi = c.r2[h_hi];
  const bool warp_live = (u.row0 + warp * 16) < rows_total;
  const float inv_cap = c.cap > 0.0f ? 1.0f / c.cap : 0.0f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
  float o[DP / 8][4];
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
  const int last_row = min(u.row0 + 63, rows_total - 1);
  const int p_first = pos0 + u.row0 / R, p_last = pos0 + last_row / R;
  const int tok0 = c.window > 0 ? max(0, p_first - c.window + 1) / 64 * 64 : 0;                 // first window tile
  const int n_keep_tiles = min((c.keep + 63) / 64, tok0 / 64);                                  // kept tiles before it
  const int n_tiles = n_keep_tiles + (p_last / 64 - tok0 / 64 + 1);
  auto tile_j0 = [&](int it) { return it < n_keep_tiles ? it * 64 : tok0 + (it - n_keep_tiles) * 64; };
  // copies of tile `it` into buffer it & 1 (asynchronous; rows beyond the last position and columns beyond the head size are zeros)
  auto load_tile = [&](int it) {
    const int j0 = tile_j0(it);
    bf16* ks = kbuf + (it & 1) * 64 * LD;
    bf16* vs = vbuf + (it & 1) * 64 * LD;
    for (int i = tid; i < 64 * (DP / 8); i += 128) {
      const int r = i / (DP / 8), ch = i % (DP / 8);
      const int j = j0 + r;
      const bool ok = j <= p_last;
      const int jj = ok ? j : j0;
      const size_t rowi = ((size_t)pg[jj / b.page_size] * c.G + u.kv_head) * b.page_size + jj % b.page_size;
      const bool kok = ok && ch < kchunks, vok = ok && ch < vchunks;
      jf::cp_async_16(&ks[r * LD + ch * 8], kc + rowi * c.dim + (kok ? ch * 8 : 0), kok ? 16u : 0u);
      jf::cp_async_16(&vs[r * LD + ch * 8], vc + rowi * c.vdim + (vok ? ch * 8 : 0), vok ? 16u : 0u);
    }
    jf::cp_async_commit();
  };
  // key splits (steps of few rows): split s of n walks the tiles [s per, (s + 1) per) of the unit's list
  int it_lo = 0, it_hi = n_tiles;
  if (n_splits > 1) {
    const int per = (n_tiles + n_splits - 1) / n_splits;
    it_lo = min(u.split * per, n_tiles);
    it_hi = min(it_lo + per, n_tiles);
  }
  if (it_lo < it_hi) load_tile(it_lo);
  for (int it = it_lo; it < it_hi; ++it) {
    const int j0 = tile_j0(it);
    const bf16* ks = kbuf + (it & 1) * 64 * LD;
    const bf16* vs = vbuf + (it & 1) * 64 * LD;
    if (it + 1 < it_hi) { load_tile(it + 1); jf::cp_async_wait_1(); }         // the next tile flies under this tile's products
    else jf::cp_async_wait_all();
    __syncthreads();
    if (warp_live) {
    float s[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f; }
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
      if (kk * 16 >= c.dim) continue;
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b0, b1, b2, b3;
        const int key = np * 16 + (lane & 7) + (lane >> 4) * 8;
        jf::ldmatrix_x4(jf::smem_u32(&ks[key * LD + kk * 16 + ((lane >> 3) & 1) * 8]), b0, b1, b2, b3);
        jf::mma_bf16_16816(s[np * 2], qa[kk], b0, b1);
        jf::mma_bf16_16816(s[np * 2 + 1], qa[kk], b2, b3);
      }
    }
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int j = j0 + nb * 8 + (lane & 3) * 2 + cc;
        const bool see_lo = j <= p_lo && (c.window <= 0 || p_lo - j < c.window || j < c.keep);
        const bool see_hi = j <= p_hi && (c.window <= 0 || p_hi - j < c.window || j < c.keep);
        float a = s[nb][cc] * c.scale, d = s[nb][2 + cc] * c.scale;
        if (c.cap > 0.0f) {
          a = c.cap * (1.0f - __fdividef(2.0f, __expf(2.0f * a * inv_cap) + 1.0f));
          d = c.cap * (1.0f - __fdividef(2.0f, __expf(2.0f * d * inv_cap) + 1.0f));
        }
        a -= r1_lo * __logf(fmaf(r2_lo, (float)(p_lo - j), 1.0f));
        d -= r1_hi * __logf(fmaf(r2_hi, (float)(p_hi - j), 1.0f));
        s[nb][cc] = see_lo ? a : -INFINITY;
        s[nb][2 + cc] = see_hi ? d : -INFINITY;
        mx_lo = fmaxf(mx_lo, s[nb][cc]);
        mx_hi = fmaxf(mx_hi, s[nb][2 + cc]);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float ref_lo = mn_lo == -INFINITY ? 0.0f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.0f : mn_hi;
    const float c_lo = expf(m_lo - ref_lo), c_hi = expf(m_hi - ref_hi);      // m = -inf: exp(-inf) = 0
    m_lo = mn_lo; m_hi = mn_hi;
    float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        s[nb][cc] = expf(s[nb][cc] - ref_lo);
        s[nb][2 + cc] = expf(s[nb][2 + cc] - ref_hi);
        sum_lo += s[nb][cc];
        sum_hi += s[nb][2 + cc];
      }
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    l_lo = l_lo * c_lo + sum_lo;
    l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) { o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi; }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {                     // 16 keys per step
      uint32_t ph[4], pl[4];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const float* sv = s[kk * 2 + half];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const float x0 = sv[rr * 2], x1 = sv[rr * 2 + 1];
          const float h0 = jf::bf16_round(x0), h1 = jf::bf16_round(x1);
          ph[half * 2 + rr] = jf::pack_bf16x2(h0, h1);
          pl[half * 2 + rr] = jf::pack_bf16x2(x0 - h0, x1 - h1);
        }
      }
#pragma unroll
      for (int np = 0; np < DP / 16; ++np) {
        if (np * 16 >= c.vdim) continue;
        uint32_t b0, b1, b2, b3;
        const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        jf::ldmatrix_x4_trans(jf::smem_u32(&vs[key * LD + np * 16 + (lane >> 4) * 8]), b0, b1, b2, b3);
        jf::mma_bf16_16816(o[np * 2], ph, b0, b1);
        jf::mma_bf16_16816(o[np * 2], pl, b0, b1);
        jf::mma_bf16_16816(o[np * 2 + 1], ph, b2, b3);
        jf::mma_bf16_16816(o[np * 2 + 1], pl, b2, b3);
      }
    }
    }
    __syncthreads();                                     // this tile's buffer is free for the tile after the next
  }
  if (!warp_live) return;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int row = hh ? r_hi : r_lo;
    if (row >= rows_total) continue;
    const int t = start + row / R, h = hh ? h_hi : h_lo;
    if (n_splits > 1) {                                  // unnormalised partial result; the combine kernel adds the sink
      const size_t slot = ((size_t)t * c.H + h) * n_splits + u.split;
      float* pp = part_o + slot * DP;
#pragma unroll
      for (int i = 0; i < DP / 8; ++i)
        *reinterpret_cast<float2*>(pp + i * 8 + (lane & 3) * 2) = make_float2(o[i][hh * 2], o[i][hh * 2 + 1]);
      if ((lane & 3) == 0) {
        part_ml[slot * 2] = hh ? m_hi : m_lo;
        part_ml[slot * 2 + 1] = hh ? l_hi : l_lo;
      }
      continue;
    }
    // the sink: one more term in the denominator
    const float m = hh ? m_hi : m_lo, sk = c.sink[h];
    const float top = fmaxf(m, sk);
    const float f = expf(m - top);
    const float inv = f / ((hh ? l_hi : l_lo) * f + expf(sk - top));
    bf16* po = out + (size_t)t * ldo + h * c.vdim;
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) {
      const int d = i * 8 + (lane & 3) * 2;
      if (d >= c.vdim) continue;
      *reinterpret_cast<__nv_bfloat162*>(po + d) = __floats2bfloat162_rn(o[i][hh * 2] * inv, o[i][hh * 2 + 1] * inv);
    }
  }
}

// Merge the key splits of one (token, head) with the sink: one block per (token, head).  A split without keys holds a
// maximum of -inf and a denominator of zero.  part_o rows are pstride wide.
template <typename OT>
__global__ void biased_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const float* __restrict__ sink,
                                      int H, int vdim, int pstride, int n_splits, OT* __restrict__ out, int ldo) {
  const int t = blockIdx.x / H, h = blockIdx.x % H;
  const size_t slot0 = ((size_t)t * H + h) * n_splits;
  const float sk = sink[h];
  float M = sk;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(slot0 + s) * 2]);
  float L = expf(sk - M);
  for (int s = 0; s < n_splits; ++s) L += part_ml[(slot0 + s) * 2 + 1] * expf(part_ml[(slot0 + s) * 2] - M);
  const float inv = 1.0f / L;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float acc = 0.0f;
    for (int s = 0; s < n_splits; ++s) acc += part_o[(slot0 + s) * pstride + d] * expf(part_ml[(slot0 + s) * 2] - M);
    out[(size_t)t * ldo + h * vdim + d] = from_f<OT>(acc * inv);
  }
}

}  // namespace hy
