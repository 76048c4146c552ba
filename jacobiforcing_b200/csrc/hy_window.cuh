// hy_window.cuh — softmax attention over a sliding window plus pooled blocks (libjf_hybrid.so).
//
// Position i sees the tokens j with 0 <= i - j < window and, beside them, one key and one value for every block of `pool`
// tokens whose last token is already behind the window: block b = positions [b pool, b pool + pool) is seen when
// b pool + pool - 1 <= i - window, so i sees the blocks 0 .. floor((i - window + 1) / pool) - 1.  Pooled rows:
// K_b = (1 / pool) sum_{j in b} K_j and V_b likewise, over the rows exactly as cached (keys after norm and rotation, values
// after their rotation).  Positions between the end of the last seen block and i - window belong to neither set.  One
// softmax runs over the union of both sets.
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
#include "hy_attn.cuh"

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

// ---- the same attention on tensor cores (bf16 build) ----------------------------------------------------------------------------
// Work unit = (entry, key head, tile of 64 query rows); rows are (token, query head of the group) pairs, token-major, so
// the heads that share a key head share every tile that is loaded.  A unit walks the pooled blocks any of its rows may
// see (tiles of 64 blocks), then the tokens from the first window of the tile to its last position (tiles of 64 keys
// aligned to absolute positions); each row masks what it does not see.  S = Q K^T by mma.sync m16n8k16 (bf16 operands,
// fp32 accumulators), online softmax in fp32, O += P V with P split into a bf16 head and a bf16 remainder (the weights
// stay 32-bit in effect).  Key and value rows are zero-padded to DP columns in shared memory (dim, vdim multiples of 8, at
// most DP).  The output is normalised, turned back by the query's position and written as the operand of the output
// projection: no key splits, since a row sees at most window + position / pool rows.  Key / value tiles are double
// buffered: the copies of the next tile are issued before the products of the current one.
template <int DP>
__global__ void __launch_bounds__(128) window_mma_kernel(Batch b, const AttnUnit* __restrict__ units, const bf16* __restrict__ q,
                                                         int ldq, WindowCfg c, const bf16* __restrict__ kc,
                                                         const bf16* __restrict__ vc, const bf16* __restrict__ kp,
                                                         const bf16* __restrict__ vp, const float* __restrict__ vrot, int ldv,
                                                         bf16* __restrict__ out, int ldo) {
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
  const int kchunks = c.dim / 8, vchunks = c.vdim / 8, slots = window_block_slots(b.page_size, c.pool);
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
  const int nb_lo = p_lo - c.window + 1 > 0 ? (p_lo - c.window + 1) / c.pool : 0;
  const int nb_hi = p_hi - c.window + 1 > 0 ? (p_hi - c.window + 1) / c.pool : 0;
  const bool warp_live = (u.row0 + warp * 16) < rows_total;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
  float o[DP / 8][4];
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
  const int last_row = min(u.row0 + 63, rows_total - 1);
  const int p_first = pos0 + u.row0 / R, p_last = pos0 + last_row / R;
  const int nb_tile = p_last - c.window + 1 > 0 ? (p_last - c.window + 1) / c.pool : 0;       // blocks the tile's last row sees
  const int tok0 = max(0, p_first - c.window + 1) / 64 * 64;                                    // first token tile
  const int n_pool_tiles = (nb_tile + 63) / 64;
  const int n_tiles = n_pool_tiles + (p_last / 64 - tok0 / 64 + 1);
  // copies of tile `it` into buffer it & 1 (asynchronous; rows beyond the range and columns beyond the head size are zeros)
  auto load_tile = [&](int it) {
    const bool pooled = it < n_pool_tiles;
    const int j0 = pooled ? it * 64 : tok0 + (it - n_pool_tiles) * 64;
    const int j_end = pooled ? nb_tile : p_last + 1;
    bf16* ks = kbuf + (it & 1) * 64 * LD;
    bf16* vs = vbuf + (it & 1) * 64 * LD;
    for (int i = tid; i < 64 * (DP / 8); i += 128) {
      const int r = i / (DP / 8), ch = i % (DP / 8);
      const int j = j0 + r;
      const bool ok = j < j_end;
      const int jj = ok ? j : j0;
      size_t rowi;
      if (pooled) {
        const int first = jj * c.pool;
        rowi = ((size_t)pg[first / b.page_size] * c.G + u.kv_head) * slots + (first % b.page_size) / c.pool;
      } else {
        rowi = ((size_t)pg[jj / b.page_size] * c.G + u.kv_head) * b.page_size + jj % b.page_size;
      }
      const bool kok = ok && ch < kchunks, vok = ok && ch < vchunks;
      jf::cp_async_16(&ks[r * LD + ch * 8], (pooled ? kp : kc) + rowi * c.dim + (kok ? ch * 8 : 0), kok ? 16u : 0u);
      jf::cp_async_16(&vs[r * LD + ch * 8], (pooled ? vp : vc) + rowi * c.vdim + (vok ? ch * 8 : 0), vok ? 16u : 0u);
    }
    jf::cp_async_commit();
  };
  load_tile(0);
  for (int it = 0; it < n_tiles; ++it) {
    const bool pooled = it < n_pool_tiles;
    const int j0 = pooled ? it * 64 : tok0 + (it - n_pool_tiles) * 64;
    const bf16* ks = kbuf + (it & 1) * 64 * LD;
    const bf16* vs = vbuf + (it & 1) * 64 * LD;
    if (it + 1 < n_tiles) { load_tile(it + 1); jf::cp_async_wait_1(); }       // the next tile flies under this tile's products
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
        const bool see_lo = pooled ? j < nb_lo : (j <= p_lo && j > p_lo - c.window);
        const bool see_hi = pooled ? j < nb_hi : (j <= p_hi && j > p_hi - c.window);
        s[nb][cc] = see_lo ? s[nb][cc] * c.scale : -INFINITY;
        s[nb][2 + cc] = see_hi ? s[nb][2 + cc] * c.scale : -INFINITY;
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
    const int t = start + row / R, h = u.kv_head * R + row % R;
    const float inv = 1.0f / (hh ? l_hi : l_lo);
    bf16* po = out + (size_t)t * ldo + h * c.vdim;
    const float* vr = vrot + (size_t)t * ldv;
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) {
      const int d = i * 8 + (lane & 3) * 2;                // an even dimension: the pair (d, d + 1) sits in this thread
      if (d >= c.vdim) continue;
      float y0 = o[i][hh * 2] * inv, y1 = o[i][hh * 2 + 1] * inv;
      if (c.rot_values) {
        const float co = vr[d], si = vr[d + 1];
        const float a0 = fmaf(y0, co, y1 * si), a1 = fmaf(y1, co, -y0 * si);          // the turn by minus the position
        y0 = a0; y1 = a1;
      }
      *reinterpret_cast<__nv_bfloat162*>(po + d) = __floats2bfloat162_rn(y0, y1);
    }
  }
}

constexpr size_t window_mma_smem(int dp) { return (size_t)4 * 64 * (dp + 8) * 2; }

}  // namespace hy
