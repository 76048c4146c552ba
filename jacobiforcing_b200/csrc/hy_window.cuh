// hy_window.cuh — softmax attention over a sliding window plus pooled blocks (libjf_hybrid.so).
//
// Position i sees the tokens j with 0 <= i - j < window and, beside them, one key and one value for every block of `pool`
// tokens that lies wholly before the window: block b = positions [b pool, b pool + pool) is seen when
// b pool + pool - 1 <= i - window, so i sees the blocks 0 .. floor((i - window + 1) / pool) - 1.  A block's key is the mean
// of its keys as the cache holds them (normed and rotated), its value the mean of its cached values.  A token that has
// left the window while its block is not yet complete behind the window is not seen at all.  Tokens and blocks share one
// softmax.
//
//   prep     per token: RMS norm per head on queries and keys (one weight of the head's size shared by the heads), rotation
//            of the pairs (2i, 2i + 1) of the first rot_dims dimensions by pos * f_i, values rotated by their own position
//            over all of vdim; queries to the workspace, keys and values into their pages, and the cosines / sines that
//            turn the output back (by the query's position) into a per-token table
//   pool     the blocks that became complete with this step's tokens: means over the cached rows, into the pooled cache
//   attend   one warp per (token, query head) over [pooled blocks | window tokens], fp32 scores and weights, then the
//            output's pairs turned by minus the query's position
//
// Cache layouts: keys [page][kv head][slot][dim], values [page][kv head][slot][vdim], pooled keys / values
// [page][kv head][block slot][dim | vdim] with ceil(page_size / pool) block slots per page: a block lives in the page of
// its first token at slot (first % page_size) / pool (unique also when blocks straddle pages).  A pooled entry is written
// when its block completes and read only by positions that see the complete block, so a reused page needs no clearing.
#pragma once
#include "hy_kernels.cuh"
#include "hy_mixers.cuh"

namespace hy {

struct WindowCfg {
  int H, G, dim, vdim, window, pool, rot_dims, rot_values, qk_norm;
  float scale;
};

__host__ __device__ inline int window_block_slots(int page_size, int pool) { return (page_size + pool - 1) / pool; }

// in [T, ld]: q at col_q (H * dim), k at col_k (G * dim), v at col_v (G * vdim).  q_out [T, ldq].  vrot [T, ldv]: pairs
// (cos, sin) of the value rotation at the token's position (only with rot_values).
template <typename AT>
__global__ void __launch_bounds__(128) window_prep_kernel(Batch b, const AT* __restrict__ in, int ld, int col_q, int col_k, int col_v,
                                                          WindowCfg c, const float* __restrict__ qn, const float* __restrict__ kn,
                                                          float eps, Rotation rot, Rotation rot_v, AT* __restrict__ q_out, int ldq,
                                                          AT* __restrict__ kc, AT* __restrict__ vc, float* __restrict__ vrot, int ldv) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  float* cs = reinterpret_cast<float*>(hy_smem);               // [2 * rot.pairs]
  float* csv = cs + 2 * rot.pairs;                             // [2 * rot_v.pairs]
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int e = b.tok_ent[t], pos = b.tok_pos[t];
  rotation_row(rot, pos, cs);
  rotation_row(rot_v, pos, csv);
  __syncthreads();
  const int page = b.pages[(size_t)e * b.max_pages + pos / b.page_size], in_page = pos % b.page_size;
  const AT* row = in + (size_t)t * ld;
  for (int u = warp; u < c.H + c.G; u += nw) {
    const bool is_q = u < c.H;
    const AT* src = row + (is_q ? col_q + u * c.dim : col_k + (u - c.H) * c.dim);
    const float* nwt = is_q ? qn : kn;
    float inv = 1.0f;
    if (c.qk_norm) {
      float ss = 0.0f;
      for (int d = lane; d < c.dim; d += 32) { const float v = to_f(src[d]); ss = fmaf(v, v, ss); }
      ss = warp_sum(ss);
      inv = 1.0f / sqrtf(ss / (float)c.dim + eps);
    }
    AT* dst = is_q ? q_out + (size_t)t * ldq + u * c.dim
                   : kc + (((size_t)page * c.G + (u - c.H)) * b.page_size + in_page) * c.dim;
    for (int d = lane; d < c.dim; d += 32) {
      float y = to_f(src[d]) * inv * (c.qk_norm ? nwt[d] : 1.0f);
      if (d < c.rot_dims) {
        const float o = to_f(src[d ^ 1]) * inv * (c.qk_norm ? nwt[d ^ 1] : 1.0f);
        const float co = cs[d & ~1], si = cs[d | 1];
        y = (d & 1) ? fmaf(y, co, o * si) : fmaf(y, co, -o * si);
      }
      dst[d] = from_f<AT>(y);
    }
  }
  for (int i = threadIdx.x; i < c.G * c.vdim; i += blockDim.x) {
    const int g = i / c.vdim, d = i % c.vdim;
    float y = to_f(row[col_v + i]);
    if (c.rot_values) {
      const float o = to_f(row[col_v + (i ^ 1)]);
      const float co = csv[d & ~1], si = csv[d | 1];
      y = (d & 1) ? fmaf(y, co, o * si) : fmaf(y, co, -o * si);
    }
    vc[(((size_t)page * c.G + g) * b.page_size + in_page) * c.vdim + d] = from_f<AT>(y);
  }
  if (c.rot_values)
    for (int i = threadIdx.x; i < c.vdim; i += blockDim.x) vrot[(size_t)t * ldv + i] = csv[i];
}

// grid (blocks an entry can complete in one step, E).  Sums run over the block's positions in order, in fp32.
template <typename AT>
__global__ void __launch_bounds__(128) window_pool_kernel(Batch b, WindowCfg c, const AT* __restrict__ kc, const AT* __restrict__ vc,
                                                          AT* __restrict__ kp, AT* __restrict__ vp) {
  const int e = blockIdx.y;
  const int pos0 = b.ent_pos0[e], end = pos0 + b.ent_start[e + 1] - b.ent_start[e];
  const int blk = pos0 / c.pool + blockIdx.x;
  if (blk > end / c.pool - 1) return;
  const int first = blk * c.pool, slots = window_block_slots(b.page_size, c.pool);
  const int* pg = b.pages + (size_t)e * b.max_pages;
  const size_t pslot = ((size_t)pg[first / b.page_size] * c.G) * slots + (first % b.page_size) / c.pool;
  const float inv = 1.0f / (float)c.pool;
  const int per = c.dim + c.vdim;
  for (int i = threadIdx.x; i < c.G * per; i += blockDim.x) {
    const int g = i / per, d = i % per;
    const bool key = d < c.dim;
    const int w = key ? c.dim : c.vdim, dd = key ? d : d - c.dim;
    const AT* src = key ? kc : vc;
    float s = 0.0f;
    for (int j = first; j < first + c.pool; ++j)
      s += to_f(src[(((size_t)pg[j / b.page_size] * c.G + g) * b.page_size + j % b.page_size) * w + dd]);
    (key ? kp : vp)[(pslot + (size_t)g * slots) * w + dd] = from_f<AT>(s * inv);
  }
}

// One warp per (token, query head).  Visible rows are walked in groups of 32 in a fixed order (blocks by index, then the
// window's tokens by position), so a position's result does not depend on the step's cut or on the batch.
template <typename AT, typename OT>
__global__ void __launch_bounds__(128) window_attn_kernel(Batch b, const AT* __restrict__ q, int ldq, WindowCfg c,
                                                          const AT* __restrict__ kc, const AT* __restrict__ vc,
                                                          const AT* __restrict__ kp, const AT* __restrict__ vp,
                                                          const float* __restrict__ vrot, int ldv, OT* __restrict__ out, int ldo) {
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
  const int slots = window_block_slots(b.page_size, c.pool);
  const int nb = pos - c.window + 1 > 0 ? (pos - c.window + 1) / c.pool : 0;       // pooled blocks seen
  const int w0 = max(0, pos - c.window + 1);                                        // first token of the window
  const int n = nb + pos + 1 - w0;
  auto row_of = [&](int idx, const AT*& kr, const AT*& vr) {
    if (idx < nb) {
      const int first = idx * c.pool;
      const size_t r = ((size_t)pg[first / b.page_size] * c.G + g) * slots + (first % b.page_size) / c.pool;
      kr = kp + r * c.dim; vr = vp + r * c.vdim;
    } else {
      const int j = w0 + idx - nb;
      const size_t r = ((size_t)pg[j / b.page_size] * c.G + g) * b.page_size + j % b.page_size;
      kr = kc + r * c.dim; vr = vc + r * c.vdim;
    }
  };
  float m = -INFINITY, l = 0.0f;
  float acc[HY_ATT_MAXD];
#pragma unroll
  for (int i = 0; i < HY_ATT_MAXD; ++i) acc[i] = 0.0f;
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int idx = i0 + lane;
    float s = -INFINITY;
    if (idx < n) {
      const AT *kr, *vr;
      row_of(idx, kr, vr);
      float dot = 0.0f;
      for (int d = 0; d < c.dim; ++d) dot = fmaf(qs[d], to_f(kr[d]), dot);
      s = dot * c.scale;
    }
    const float mn = fmaxf(m, warp_max(s));
    const float corr = expf(m - mn);                                                 // m = -inf at the start: exp(-inf) = 0
    const float p = idx < n ? expf(s - mn) : 0.0f;
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int i = 0; i < HY_ATT_MAXD; ++i) acc[i] *= corr;
    const int cnt = min(32, n - i0);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const AT *kr, *vr;
      row_of(i0 + jj, kr, vr);
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
    float y = acc[i] * inv;
    const float o = __shfl_xor_sync(0xffffffffu, y, 1);                              // the pair's other half (d ^ 1)
    if (d < c.vdim) {
      if (c.rot_values) {
        const float co = vrot[(size_t)t * ldv + (d & ~1)], si = vrot[(size_t)t * ldv + (d | 1)];
        y = (d & 1) ? fmaf(y, co, -o * si) : fmaf(y, co, o * si);                    // the turn by minus the position
      }
      out[(size_t)t * ldo + h * c.vdim + d] = from_f<OT>(y);
    }
  }
}

}  // namespace hy
