// hy_gemm.cuh — tcgen05 matrix product of the layered hybrid decoders' prefill path (bf16 operands, fp32 accumulation in
// tensor memory):  C[t, n] = sum_k X[t, k] W[n, k].
//
// Swap-AB like the Jacobi engine's GEMMs: the WEIGHT tile is the MMA's A operand (M = 128 output features, so the
// accumulator's lanes are features and a warp's epilogue stores are contiguous along n), the token rows are the B operand
// (N = BT tokens, 128 or 256).  Weights are stored in HBM already in the K-major SWIZZLE_128B tile layout (one contiguous
// 16 KiB tile per 128 features x 64 k: one bulk copy per pipeline stage, no tensor map); the activation tile is read
// row-major with 16-byte loads by four producer warps that write it swizzled into shared memory.
//
// Warps 0-3: activation producers, then the epilogue (TMEM -> registers -> global, through GemmOut).
// Warp 4:    weight producer (one lane, cp.async.bulk + mbarrier expect_tx).
// Warp 5:    owns tensor memory; one lane issues tcgen05.mma and commits.
// Every wait is bounded: on a timeout the kernel raises the error flag, stops waiting and still frees its tensor memory.
#pragma once
#include "hy_kernels.cuh"
#include "jf_ptx.cuh"

namespace hy {

constexpr int TC_STAGES = 4;
constexpr int TC_WTILE = 128 * 64 * 2;                 // 16 KiB
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;           // try_wait probes (each blocks for a bounded time itself)

struct TcSmem {
  uint64_t full[TC_STAGES], empty[TC_STAGES], acc_full;
  uint32_t tmem_base;
  uint32_t failed;
};

__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, TcSmem* sm, int* err) {
  if (sm->failed) return false;
  for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i)
    if (jf::mbar_try_wait(bar, parity)) return true;
  sm->failed = 1;
  atomicExch(err, 1);
  return false;
}

// Grouped mode (routed experts): blockIdx.y names a tile of a list; a tile is up to BT consecutive rows [row0, ...) of the
// expert-sorted order that belong to one expert; its weight tiles start at Wt + expert * w_stride; activation rows are
// fetched through row_map (NULL: the sorted order itself).  Blocks beyond the list's length leave at once.
struct TcGroup {
  const int* meta; const int* offs; const int* tile_expert; const int* tile_row0; const int* row_map; size_t w_stride;
};

// GemmOut.act2 == 2 (gated pair): the weight rows alternate 16 gate features and the 16 up features that go with them, so
// lanes l and l + 16 of an epilogue warp hold one pair; act(gate) * up (act = GemmOut.act_kind) leaves through out1 at
// feature n / 2.
template <typename TO, int BT>
__global__ void __launch_bounds__(192) gemm_tc_kernel(const bf16* __restrict__ X, int lda, const bf16* __restrict__ Wt, int T,
                                                      int N, int K, GemmOut o, int* err, TcGroup grp) {
  extern __shared__ __align__(16) unsigned char hy_smem[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(hy_smem) + 1023) & ~(uintptr_t)1023);
  constexpr int XTILE = BT * 128;                        // BT rows of 64 bf16
  constexpr int SLOT = TC_WTILE + XTILE;
  TcSmem* sm = reinterpret_cast<TcSmem*>(base + TC_STAGES * SLOT);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128;
  int t0 = blockIdx.y * BT;
  if (grp.meta) {
    if ((int)blockIdx.y >= grp.meta[0]) return;           // the whole block, before any barrier or tensor memory exists
    const int e = grp.tile_expert[blockIdx.y];
    t0 = grp.tile_row0[blockIdx.y];
    T = grp.offs[e + 1];
    Wt += (size_t)e * grp.w_stride;
  }
  const int KT = (K + 63) / 64;
  if (threadIdx.x == 0) {
    for (int i = 0; i < TC_STAGES; ++i) { jf::mbar_init(&sm->full[i], 129); jf::mbar_init(&sm->empty[i], 1); }
    jf::mbar_init(&sm->acc_full, 1);
    sm->failed = 0;
    jf::fence_mbar_init();
  }
  if (warp == 5) jf::tmem_alloc(&sm->tmem_base, BT);
  jf::tc_fence_before();
  __syncthreads();
  jf::tc_fence_after();

  if (warp < 4) {
    // ---- activation producers ------------------------------------------------------------------------------------
    int srow[BT / 16];                                    // source row of each of this thread's loads (-1: beyond the rows)
#pragma unroll
    for (int u = 0; u < BT / 16; ++u) {
      const int t = t0 + ((threadIdx.x + u * 128) >> 3);
      srow[u] = t < T ? (grp.row_map ? grp.row_map[t] : t) : -1;
    }
    for (int kt = 0; kt < KT; ++kt) {
      const int s = kt % TC_STAGES;
      unsigned char* xt = base + s * SLOT + TC_WTILE;
      // all loads of the stage first (BT / 16 independent 16-byte loads per thread in flight), then the swizzled stores
      uint4 v[BT / 16];
#pragma unroll
      for (int u = 0; u < BT / 16; ++u) {
        const int k = kt * 64 + ((threadIdx.x + u * 128) & 7) * 8;
        v[u] = make_uint4(0, 0, 0, 0);
        if (srow[u] >= 0 && k < K) v[u] = *reinterpret_cast<const uint4*>(X + (size_t)srow[u] * lda + k);
      }
      if (!tc_wait(&sm->empty[s], ((kt / TC_STAGES) & 1) ^ 1, sm, err)) break;     // the slot is free: MMAs that read it retired
#pragma unroll
      for (int u = 0; u < BT / 16; ++u) {
        const int i = threadIdx.x + u * 128;
        const int r = i >> 3, c = i & 7;
        *reinterpret_cast<uint4*>(xt + r * 128 + ((c ^ (r & 7)) << 4)) = v[u];
      }
      jf::fence_proxy_async_smem();
      jf::mbar_arrive(&sm->full[s]);
    }
    // ---- epilogue ----------------------------------------------------------------------------------------------------
    if (tc_wait(&sm->acc_full, 0, sm, err)) {
      jf::tc_fence_after();
      const uint32_t taddr = sm->tmem_base + ((uint32_t)(warp * 32) << 16);
      const int n = n0 + warp * 32 + lane;
      for (int c0 = 0; c0 < BT; c0 += 16) {
        if (t0 + c0 >= T) break;
        uint32_t v[16];
        jf::tmem_ld16(taddr + c0, v);
        jf::tmem_ld_wait();
        if (o.act2 == 2) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float mine = __uint_as_float(v[j]);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
            const int f = ((n0 + warp * 32) >> 1) + lane;
            if (lane < 16 && f < o.split && t0 + c0 + j < T)
              ((TO*)o.out1)[(size_t)(t0 + c0 + j) * o.ld1 + f] = from_f<TO>(gated_pair_f(o.act_kind, mine, other, o.act_limit));
          }
          continue;
        }
        if (n < N) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (t0 + c0 + j < T) gemm_store<TO>(o, t0 + c0 + j, n, __uint_as_float(v[j]));
        }
      }
    }
  } else if (warp == 4) {
    // ---- weight producer -----------------------------------------------------------------------------------------------
    if (lane == 0) {
      const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(Wt) + (size_t)blockIdx.x * KT * TC_WTILE;
      for (int kt = 0; kt < KT; ++kt) {
        const int s = kt % TC_STAGES;
        if (!tc_wait(&sm->empty[s], ((kt / TC_STAGES) & 1) ^ 1, sm, err)) break;
        jf::mbar_expect_tx(&sm->full[s], TC_WTILE);
        jf::bulk_g2s(base + s * SLOT, wsrc + (size_t)kt * TC_WTILE, TC_WTILE, &sm->full[s]);
      }
    }
  } else {
    // ---- MMA issuer -----------------------------------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = jf::umma_idesc_bf16(128, BT);
      const uint32_t d0 = sm->tmem_base;
      bool ok = true;
      for (int kt = 0; kt < KT && ok; ++kt) {
        const int s = kt % TC_STAGES;
        ok = tc_wait(&sm->full[s], (kt / TC_STAGES) & 1, sm, err);
        if (!ok) break;
        jf::tc_fence_after();
        const uint32_t sa = jf::smem_u32(base + s * SLOT);
        const uint32_t sb = sa + TC_WTILE;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          jf::umma_bf16(d0, jf::umma_desc_sw128(sa + kk * 32), jf::umma_desc_sw128(sb + kk * 32), idesc, (kt > 0 || kk > 0) ? 1u : 0u);
        jf::umma_commit(&sm->empty[s]);
      }
      if (ok) jf::umma_commit(&sm->acc_full);
    }
    __syncwarp();
  }
  jf::tc_fence_before();
  __syncthreads();
  if (warp == 5) jf::tmem_dealloc(sm->tmem_base, BT);
}

constexpr size_t tc_smem_bytes(int bt) { return (size_t)TC_STAGES * (TC_WTILE + bt * 128) + sizeof(TcSmem) + 1024; }

// Host-side packer: row-major [N, K] floats -> bf16 tiles [ceil(N/128)][ceil(K/64)] of 128 x 64 in the swizzled layout.
inline void pack_tiles(const float* w, int N, int K, std::vector<uint16_t>& out) {
  const int NT = (N + 127) / 128, KT = (K + 63) / 64;
  out.assign((size_t)NT * KT * 128 * 64, 0);
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const size_t tile = (size_t)(n / 128) * KT + k / 64;
      const uint32_t off = jf::sw128_offset((uint32_t)(n % 128), (uint32_t)(k % 64));
      __nv_bfloat16 b = __float2bfloat16_rn(w[(size_t)n * K + k]);
      uint16_t bits;
      memcpy(&bits, &b, 2);
      out[tile * 8192 + off / 2] = bits;
    }
}

}  // namespace hy
