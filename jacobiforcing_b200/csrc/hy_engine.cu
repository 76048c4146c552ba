// hy_engine.cu — host side of libjf_hybrid.so (include/jacobi_hybrid.h): weights by checkpoint name, merged projections,
// the paged key cache, recurrent-state slots and the step function that runs a packed batch of entries through the layers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <type_traits>
#include <map>
#include <string>
#include <vector>

#include "../../include/jacobi_hybrid.h"
#include "hy_kernels.cuh"
#include "hy_gemm.cuh"
#include "hy_attn.cuh"
#include "hy_mixers.cuh"
#include "hy_experts.cuh"
#include "hy_window.cuh"
#include "hy_biased.cuh"

namespace hy {

struct HostTensor {
  std::vector<int64_t> shape;
  std::vector<float> v;
  int64_t rows() const { return shape.empty() ? 1 : shape[0]; }
  int64_t cols() const { return shape.size() < 2 ? 1 : shape[1]; }
};

// Device tensors of one layer (WT = operand type of the build; fp32 tables where the design wants fp32).
struct LayerW {
  void* norm1 = nullptr;
  void* w_in = nullptr;   int n_in = 0;        // merged projections of the normed input [n_in, width]
  void* w_out = nullptr;  int k_out = 0;       // merged output projections [width, k_out] (concatenated along k)
  // column offsets inside the merged input projection / the merged output operand
  int c_q = 0, c_k = 0, c_g = 0, c_x = 0, c_z = 0, c_v = 0, c_b = 0, c_a1 = 0, c_g1 = 0, c_up = 0;
  int o_mix = 0, o_scan = 0, o_ff = 0;
  void* conv_qk = nullptr; void* sink = nullptr;                               // attention side
  void* conv_x = nullptr; void* conv_xb = nullptr; void* w_x = nullptr; void* w_dt = nullptr; void* dt_b = nullptr;
  float* A_neg = nullptr; void* D = nullptr;                                    // scan side
  void* conv_qkv = nullptr; void* w_a2 = nullptr; void* w_g2 = nullptr; void* A_log = nullptr; void* dt_bias = nullptr;
  void* norm_w = nullptr;                                                        // delta
  void* cache = nullptr;                                                         // key pages of this layer
  // the same matrices as swizzled 128 x 64 tiles for the tensor-core product (bf16 build)
  void* w_in_t = nullptr; void* w_out_t = nullptr; void* w_x_t = nullptr; void* w_a2_t = nullptr; void* w_g2_t = nullptr;
  float* conv_state = nullptr; float* conv_state2 = nullptr; float* rec_state = nullptr;
  // norm - sublayer - norm blocks: the four norms and two layer scales of a layer
  TanhNorm n1{}, n1b{}, n2{}, n2b{};
  float* ls1 = nullptr; float* ls2 = nullptr;
  // state-space recurrence with one decay per head
  void* m_conv_w = nullptr; void* m_conv_b = nullptr;
  float* m_dt_bias = nullptr; float* m_A_log = nullptr; float* m_D = nullptr; float* m_norm = nullptr;
  // attention over a shared latent
  float* l_qn = nullptr; float* l_kn = nullptr;
  void* w_uq = nullptr; void* w_uq_t = nullptr; void* w_uk = nullptr; void* w_uvT = nullptr;
  void* w_ukT = nullptr; void* w_uv = nullptr;            // [H][rank][dim] and [H][vdim][rank]: the few-row kernel's layouts
  Rotation rot{};
  // gated linear recurrence
  float* g_fb = nullptr; float* g_lower = nullptr; float* g_norm = nullptr;
  // routed experts: router [experts, width], gate/up [experts][2 ff][width], down [experts][width][ff]
  void* w_router = nullptr; void* w_router_t = nullptr; void* w_gu = nullptr; void* w_down = nullptr;
  // the same as swizzled tiles per expert for the tensor-core product: gate/up rows alternate in blocks of 16
  void* w_gu_t = nullptr; void* w_down_t = nullptr; size_t gu_t_stride = 0, down_t_stride = 0; int gu_rows = 0;
  // blocks normed on the sublayer's output: plain RMS weights; router bias; the shared expert; the gated dense feed-forward
  // ([gate rows | up rows] stacked, and as tiles whose rows alternate 16 gate and 16 up features)
  float* pn1 = nullptr; float* pn2 = nullptr; float* x_rb = nullptr;
  void* w_sh_up = nullptr; void* w_sh_up_t = nullptr; void* w_sh_down = nullptr; void* w_sh_down_t = nullptr;
  void* w_ff_in = nullptr; void* w_ff_in_t = nullptr; int ff_rows = 0; void* w_ff_down = nullptr; void* w_ff_down_t = nullptr;
  // window attention: query / key norm weights, the values' rotation, value pages, pooled key / value pages
  float* w_qn = nullptr; float* w_kn = nullptr; Rotation rot_v{};
  void* cache_v = nullptr; void* pool_k = nullptr; void* pool_v = nullptr;
  // matrix memory: gate biases, the output norm's weight (all heads), column of the gate pre-activations
  float* t_ib = nullptr; float* t_fb = nullptr; float* t_norm = nullptr; int c_i = 0;
  // pre-norm blocks: input convolutions of both sublayers (weights; the tails live in conv_state / conv_state2), weights of
  // the depth average, the token input's projections and norm
  float* canon1 = nullptr; float* canon2 = nullptr; float* dwa = nullptr;
  void* side_gate = nullptr; void* side_proj = nullptr; float* side_norm = nullptr;
  // biased attention: bias of the merged input projection, the heads' distance-bias numbers and sinks, the blend factor
  float* b_bias = nullptr; float* b_r1 = nullptr; float* b_r2 = nullptr; float* b_sink = nullptr; float b_lambda = 0.0f;
  int b_mix = 0;                                  // 0: values as projected, 1: the first blending layer, 2: blends with the first
};

}  // namespace hy

using namespace hy;

struct hy_engine {
  hy_model_cfg m{};
  hy_runtime_cfg rt{};
  std::vector<hy_layer_cfg> lc;
  std::map<std::string, HostTensor> host;
  std::vector<LayerW> lw;
  void* embed = nullptr; void* final_norm = nullptr; void* head = nullptr; void* head_t = nullptr; double* inv_freq = nullptr;
  float* embed_norm = nullptr;
  TanhNorm final_tanh{};
  // pre-norm blocks: hashed pair table, token-input table, the last token of each request (per state slot), normed rows,
  // the depth average's store [layers + 1][step tokens][width], the first blending layer's values of the step
  void* pair_table = nullptr; void* side_table = nullptr; int* prev_tok = nullptr;
  float* hn = nullptr; float* kept = nullptr; void* vfirst = nullptr; int ld_vf = 0;
  // routed feed-forward: choices and weights per (token, choice) pair, the sorted order, the tile list
  int* x_ids = nullptr; float* x_wts = nullptr; int* x_counts = nullptr; int* x_offs = nullptr; int* x_fill = nullptr;
  int* x_tile_e = nullptr; int* x_tile_r0 = nullptr; int* x_meta = nullptr; int* x_row_tok = nullptr; int* x_pair_row = nullptr;
  int x_max_tiles = 0;
  int* err_d = nullptr; int* err_h = nullptr;
  // per-category device times (hy_profile_enable): event pairs recorded around groups of launches
  bool prof_on = false;
  float prof_ms[HY_PROFILE_CATEGORIES] = {};
  std::vector<cudaEvent_t> ev_pool;
  struct ProfRec { int cat; cudaEvent_t a, b; };
  std::vector<ProfRec> prof_list;
  cudaEvent_t get_event() {
    if (!ev_pool.empty()) { cudaEvent_t e = ev_pool.back(); ev_pool.pop_back(); return e; }
    cudaEvent_t e; cudaEventCreate(&e); return e;
  }
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::string err;
  int64_t launches = 0;
  float last_ms = 0.0f;
  int64_t bytes_w = 0, bytes_cache = 0, bytes_state = 0, bytes_ws = 0;
  std::vector<void*> allocs;
  bool finalized = false;
  // workspace
  float* x = nullptr; void* hbuf = nullptr; void* pin = nullptr; void* cat = nullptr; void* cv = nullptr;
  float* f1 = nullptr; float* f2 = nullptr; void* hw = nullptr; float* logits = nullptr; int* sampled = nullptr;
  float* temp_d = nullptr;
  int ld_pin = 0, ld_cat = 0, ld_cv = 0, ld_f1 = 0, ld_f2 = 0;
  int* meta_d = nullptr; int* meta_h = nullptr; size_t meta_words = 0;
  // tensor-core attention: work units of the step (per head layout), partial results per (row, key split)
  AttnUnit* units_d = nullptr; AttnUnit* units_h = nullptr; size_t units_cap = 0; int units_n = 0;
  int units_H = 0, units_G = 0, units_split = 0, units_ns = 0;
  float* part_o = nullptr; float* part_ml = nullptr; size_t part_rows = 0, part_dim = 0;
  const int32_t* step_start = nullptr; const int32_t* step_pos0 = nullptr;     // host views of the running step
  size_t esz() const { return m.dtype == HY_DTYPE_F32 ? 4 : 2; }
};

#define HY_CUDA(call)                                                                                   \
  do {                                                                                                  \
    cudaError_t e_ = (call);                                                                            \
    if (e_ != cudaSuccess) {                                                                            \
      h->err = std::string(#call) + ": " + cudaGetErrorString(e_);                                      \
      return HY_ERR_CUDA;                                                                               \
    }                                                                                                   \
  } while (0)

struct ProfScope {
  hy_engine* h; int cat; cudaEvent_t a{}, b{};
  ProfScope(hy_engine* h_, int cat_) : h(h_), cat(cat_) {
    if (h->prof_on) { a = h->get_event(); b = h->get_event(); cudaEventRecord(a, h->stream); }
  }
  ~ProfScope() {
    if (h->prof_on) { cudaEventRecord(b, h->stream); h->prof_list.push_back({cat, a, b}); }
  }
};

static int fail(hy_engine* h, int code, const std::string& msg) {
  h->err = msg;
  return code;
}

static int dev_alloc(hy_engine* h, void** p, size_t bytes, int64_t* counter) {
  if (bytes == 0) bytes = 16;
  HY_CUDA(cudaMalloc(p, bytes));
  h->allocs.push_back(*p);
  *counter += (int64_t)bytes;
  return HY_OK;
}

static thread_local std::string g_create_err;

extern "C" int hy_create(const hy_model_cfg* model, const hy_layer_cfg* layers, const hy_runtime_cfg* rt, hy_handle* out) {
  if (!model || !layers || !rt || !out) { g_create_err = "null argument"; return HY_ERR_INVALID; }
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    g_create_err = "no CUDA device: the hybrid engine has no CPU fallback";
    return HY_ERR_CUDA;
  }
  hy_engine* h = new hy_engine();
  h->m = *model;
  h->rt = *rt;
  h->lc.assign(layers, layers + model->n_layers);
  auto bad = [&](const std::string& s) { g_create_err = s; delete h; return HY_ERR_INVALID; };
  if (model->dtype != HY_DTYPE_BF16 && model->dtype != HY_DTYPE_F32) return bad("dtype must be bf16 or f32");
  if (rt->page_size <= 0 || rt->page_size % 16) return bad("page_size must be a positive multiple of 16");
  for (auto& c : h->lc) {
    if (c.mixer == HY_MIX_ATTN_SCAN) {
      if (c.a_vdim != c.a_dim) return bad("attention whose values are its keys needs vdim == dim");
      if (c.a_dim > 32 * HY_ATT_MAXD) return bad("attention key size above 256");
      if (c.a_kv_heads <= 0 || c.a_heads % c.a_kv_heads) return bad("attention heads must be a multiple of kv_heads");
      if (c.s_state > 256 || c.s_state <= 0) return bad("scan state size must lie in 1..256");
      if (c.a_conv > HY_MAX_TAPS || c.s_conv > HY_MAX_TAPS || c.a_conv < 1 || c.s_conv < 1) return bad("conv taps must lie in 1..16");
    } else if (c.mixer == HY_MIX_DELTA) {
      if (c.d_kv_heads <= 0 || c.d_heads % c.d_kv_heads) return bad("delta heads must be a multiple of kv_heads");
      if (c.d_dim > 1024 || c.d_vdim > 1024) return bad("delta head sizes above 1024");
      if ((size_t)c.d_dim * c.d_vdim * 4 > 200 * 1024) return bad("delta state of one head exceeds shared memory");
      if (c.d_conv > HY_MAX_TAPS || c.d_conv < 1) return bad("conv taps must lie in 1..16");
    } else if (c.mixer == HY_MIX_SSD) {
      if (c.m_heads <= 0 || c.m_vdim <= 0 || c.m_groups <= 0 || c.m_heads % c.m_groups) return bad("recurrence heads must be a multiple of its groups");
      if (c.m_state > 512 || c.m_state <= 0) return bad("recurrence state size must lie in 1..512");
      if (c.m_conv > HY_MAX_TAPS || c.m_conv < 1) return bad("conv taps must lie in 1..16");
      if (c.m_norm_groups <= 0 || (c.m_heads * c.m_vdim) % c.m_norm_groups) return bad("the output norm's parts must divide heads * vdim");
    } else if (c.mixer == HY_MIX_LATENT) {
      if (c.l_heads <= 0 || c.l_dim <= 0 || c.l_vdim <= 0 || c.l_kv_rank <= 0 || c.l_q_rank <= 0 || c.l_rot_dim < 0) return bad("latent attention sizes must be positive");
      if (c.l_kv_rank + c.l_rot_dim > 32 * HY_ATT_MAXD) return bad("latent rank + rotated size above 640");
      if (c.r_dims < 0 || c.r_dims % 2 || c.r_dims > c.l_rot_dim) return bad("rotated dimensions must be even and at most rot_dim");
      const int idx = (int)(&c - h->lc.data());
      if (c.l_kv_from >= 0) {
        if (c.l_kv_from >= idx) return bad("a borrowed latent must come from an earlier layer");
        const hy_layer_cfg& o = h->lc[c.l_kv_from];
        if (o.mixer != HY_MIX_LATENT || o.l_kv_from >= 0 || o.l_kv_rank != c.l_kv_rank || o.l_rot_dim != c.l_rot_dim)
          return bad("a borrowed latent must come from a latent-attention layer with its own down-projection and equal sizes");
      }
    } else if (c.mixer == HY_MIX_GLR) {
      if (c.g_heads <= 0 || c.g_dim <= 0 || c.g_vdim <= 0) return bad("gated linear recurrence sizes must be positive");
      if (((size_t)c.g_dim * c.g_vdim + 2 * c.g_dim + c.g_vdim + 40) * 4 > 200 * 1024 && (c.g_dim > 128 || c.g_vdim > 256))
        return bad("gated linear recurrence: the state of one head exceeds shared memory");
    } else if (c.mixer == HY_MIX_WINDOW) {
      if (c.w_heads <= 0 || c.w_kv_heads <= 0 || c.w_heads % c.w_kv_heads) return bad("window attention heads must be a multiple of kv_heads");
      if (c.w_dim <= 0 || c.w_vdim <= 0 || c.w_dim > 32 * HY_ATT_MAXD || c.w_vdim > 32 * HY_ATT_MAXD) return bad("window attention head sizes must lie in 1..640");
      if (c.w_window < 1 || c.w_pool < 1) return bad("window and pool must be at least 1");
      if (c.w_rot_dims < 0 || c.w_rot_dims % 2 || c.w_rot_dims > c.w_dim) return bad("rotated dimensions must be even and at most dim");
      if (c.w_rot_values && c.w_vdim % 2) return bad("rotated values need an even vdim");
    } else if (c.mixer == HY_MIX_MLSTM) {
      if (c.t_heads <= 0 || c.t_dim <= 0 || c.t_vdim <= 0) return bad("matrix memory sizes must be positive");
      if (((size_t)c.t_dim * (c.t_vdim + 1) + 2 * c.t_dim + c.t_vdim + 40) * 4 > 200 * 1024 &&
          (c.t_dim > 128 || c.t_vdim > 255))
        return bad("matrix memory: the state of one head exceeds shared memory");
    } else if (c.mixer == HY_MIX_BIASED) {
      if (c.b_heads <= 0 || c.b_kv_heads <= 0 || c.b_heads % c.b_kv_heads) return bad("biased attention heads must be a multiple of kv_heads");
      if (c.b_dim <= 0 || c.b_vdim <= 0 || c.b_dim > 32 * HY_ATT_MAXD || c.b_vdim > 32 * HY_ATT_MAXD) return bad("biased attention head sizes must lie in 1..640");
      if (c.b_window < 0 || c.b_keep_first < 0) return bad("window and kept first tokens must not be negative");
    } else {
      return bad("unknown mixer kind");
    }
    const int mixer_block = (c.mixer == HY_MIX_SSD || c.mixer == HY_MIX_LATENT || c.mixer == HY_MIX_GLR) ? HY_BLOCK_SANDWICH
                            : (c.mixer == HY_MIX_WINDOW || c.mixer == HY_MIX_MLSTM) ? HY_BLOCK_POSTNORM
                            : c.mixer == HY_MIX_BIASED ? HY_BLOCK_PRENORM : HY_BLOCK_PARALLEL;
    if (mixer_block != model->block_kind) return bad("this mixer does not belong to the model's block layout");
    const bool ff_fits = c.ff_kind == HY_FF_NONE || (c.ff_kind == HY_FF_RELU2 && model->block_kind == HY_BLOCK_PARALLEL) ||
                         (c.ff_kind == HY_FF_ROUTED && model->block_kind != HY_BLOCK_PARALLEL) ||
                         (c.ff_kind == HY_FF_GATED && (model->block_kind == HY_BLOCK_POSTNORM || model->block_kind == HY_BLOCK_PRENORM));
    if (!ff_fits) return bad("this feed-forward does not belong to the model's block layout");
    if (c.ff_kind == HY_FF_ROUTED) {
      if (c.x_experts <= 0 || c.x_experts > 4096 || c.x_groups <= 0 || c.x_experts % c.x_groups) return bad("experts must split into equal groups");
      if (c.x_keep < 1 || c.x_keep > c.x_groups) return bad("kept groups outside 1..groups");
      if (c.x_top < 1 || c.x_top > c.x_keep * (c.x_experts / c.x_groups)) return bad("more experts per token than the kept groups hold");
      if (c.ff <= 0) return bad("expert size must be positive");
      if (c.x_route != HY_ROUTE_SIGMOID_GROUPS && c.x_route != HY_ROUTE_TOP_SOFTMAX) return bad("unknown router kind");
      if (c.x_act < 0 || c.x_act > 2 || c.x_shared_ff < 0) return bad("unknown expert activation or negative shared size");
      if (model->block_kind == HY_BLOCK_SANDWICH && (c.x_plain || c.x_shared_ff || c.x_route || c.x_act))
        return bad("norm - sublayer - norm blocks serve gated silu experts with sigmoid scores only");
      if (model->block_kind == HY_BLOCK_POSTNORM && !c.x_plain) return bad("output-normed blocks serve experts without a gate only");
      if (model->block_kind == HY_BLOCK_PRENORM && (c.x_plain || c.x_shared_ff || c.x_route != HY_ROUTE_TOP_SOFTMAX))
        return bad("pre-norm blocks serve gated experts chosen by the largest logits only");
    }
    if (c.ff_kind == HY_FF_GATED && (c.ff <= 0 || c.ff_act < 0 || c.ff_act > 3)) return bad("gated feed-forward: size or activation");
  }
  if (model->block_kind == HY_BLOCK_PRENORM) {
    if (model->canon_taps < 0 || model->canon_taps > HY_MAX_TAPS) return bad("taps of the input convolutions must lie in 0..16");
    if (model->side_dim < 0 || model->pair_buckets < 0) return bad("negative token-input size or pair buckets");
  }
  const int want_norm = model->block_kind == HY_BLOCK_SANDWICH ? HY_NORM_TANH
                        : (model->block_kind == HY_BLOCK_POSTNORM || model->block_kind == HY_BLOCK_PRENORM) ? HY_NORM_RMS : HY_NORM_RMS_OFFSET;
  if (model->norm_kind != want_norm) return bad("block layout and norm kind do not go together");
  if (cudaSetDevice(rt->device) != cudaSuccess) return bad("cudaSetDevice failed");
  cudaStreamCreate(&h->stream);
  cudaEventCreate(&h->ev0);
  cudaEventCreate(&h->ev1);
  *out = h;
  return HY_OK;
}

extern "C" void hy_destroy(hy_handle h) {
  if (!h) return;
  cudaSetDevice(h->rt.device);
  cudaStreamSynchronize(h->stream);
  for (void* p : h->allocs) cudaFree(p);
  if (h->meta_h) cudaFreeHost(h->meta_h);
  if (h->units_h) cudaFreeHost(h->units_h);
  if (h->err_h) cudaFreeHost(h->err_h);
  cudaEventDestroy(h->ev0);
  cudaEventDestroy(h->ev1);
  cudaStreamDestroy(h->stream);
  delete h;
}

extern "C" const char* hy_last_error(hy_handle h) { return h ? h->err.c_str() : g_create_err.c_str(); }
extern "C" int64_t hy_launch_count(hy_handle h) { return h ? h->launches : 0; }
extern "C" float hy_last_step_ms(hy_handle h) { return h ? h->last_ms : 0.0f; }
extern "C" int hy_profile_enable(hy_handle h, int32_t on) {
  if (!h) return HY_ERR_INVALID;
  h->prof_on = on != 0;
  for (float& v : h->prof_ms) v = 0.0f;
  return HY_OK;
}
extern "C" int hy_profile_read(hy_handle h, float* ms) {
  if (!h || !ms) return HY_ERR_INVALID;
  for (int i = 0; i < HY_PROFILE_CATEGORIES; ++i) ms[i] = h->prof_ms[i];
  return HY_OK;
}
extern "C" int hy_memory_info(hy_handle h, int64_t* w, int64_t* c, int64_t* s, int64_t* ws) {
  if (!h) return HY_ERR_INVALID;
  if (w) *w = h->bytes_w;
  if (c) *c = h->bytes_cache;
  if (s) *s = h->bytes_state;
  if (ws) *ws = h->bytes_ws;
  return HY_OK;
}

extern "C" int hy_load_tensor(hy_handle h, const char* name, const void* data, const int64_t* shape, int32_t ndim, int32_t dtype) {
  if (!h || !name || !data) return HY_ERR_INVALID;
  if (h->finalized) return fail(h, HY_ERR_INVALID, "weights are final");
  HostTensor t;
  int64_t n = 1;
  for (int i = 0; i < ndim; ++i) { t.shape.push_back(shape[i]); n *= shape[i]; }
  t.v.resize((size_t)n);
  if (dtype == HY_DTYPE_F32) {
    memcpy(t.v.data(), data, (size_t)n * 4);
  } else if (dtype == HY_DTYPE_BF16) {
    const uint16_t* s = (const uint16_t*)data;
    for (int64_t i = 0; i < n; ++i) { uint32_t u = (uint32_t)s[i] << 16; memcpy(&t.v[(size_t)i], &u, 4); }
  } else if (dtype == HY_DTYPE_F16) {
    const __half* s = (const __half*)data;
    for (int64_t i = 0; i < n; ++i) t.v[(size_t)i] = __half2float(s[i]);
  } else if (dtype == HY_DTYPE_I32) {
    const int32_t* s = (const int32_t*)data;
    for (int64_t i = 0; i < n; ++i) t.v[(size_t)i] = (float)s[i];
  } else {
    return fail(h, HY_ERR_INVALID, "unknown tensor dtype");
  }
  h->host[name] = std::move(t);
  return HY_OK;
}

// ---- weights -------------------------------------------------------------------------------------------------------------------
namespace {

struct Builder {
  hy_engine* h;
  int rc = HY_OK;
  const HostTensor* get(const std::string& name, int64_t r, int64_t c) {
    auto it = h->host.find(name);
    if (it == h->host.end()) { if (rc == HY_OK) rc = fail(h, HY_ERR_INVALID, "missing tensor " + name); return nullptr; }
    const HostTensor& t = it->second;
    if (t.rows() != r || (c >= 0 && t.cols() != c) || (c < 0 && t.shape.size() != 1)) {
      if (rc == HY_OK) rc = fail(h, HY_ERR_INVALID, "tensor " + name + " has an unexpected shape");
      return nullptr;
    }
    return &t;
  }
  // upload as the build's operand type
  void* up(const std::vector<float>& v) {
    void* d = nullptr;
    if (rc != HY_OK) return nullptr;
    if (h->m.dtype == HY_DTYPE_F32) {
      if (dev_alloc(h, &d, v.size() * 4, &h->bytes_w) != HY_OK) { rc = HY_ERR_CUDA; return nullptr; }
      cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
    } else {
      std::vector<__nv_bfloat16> b(v.size());
      for (size_t i = 0; i < v.size(); ++i) b[i] = __float2bfloat16_rn(v[i]);
      if (dev_alloc(h, &d, v.size() * 2, &h->bytes_w) != HY_OK) { rc = HY_ERR_CUDA; return nullptr; }
      cudaMemcpy(d, b.data(), b.size() * 2, cudaMemcpyHostToDevice);
    }
    return d;
  }
  void* up_tiled(const std::vector<float>& v, int N, int K) {
    if (rc != HY_OK || h->m.dtype != HY_DTYPE_BF16) return nullptr;
    std::vector<uint16_t> t;
    pack_tiles(v.data(), N, K, t);
    void* d = nullptr;
    if (dev_alloc(h, &d, t.size() * 2, &h->bytes_w) != HY_OK) { rc = HY_ERR_CUDA; return nullptr; }
    cudaMemcpy(d, t.data(), t.size() * 2, cudaMemcpyHostToDevice);
    return d;
  }
  float* up_f32(const std::vector<float>& v) {
    void* d = nullptr;
    if (rc != HY_OK) return nullptr;
    if (dev_alloc(h, &d, v.size() * 4, &h->bytes_w) != HY_OK) { rc = HY_ERR_CUDA; return nullptr; }
    cudaMemcpy(d, v.data(), v.size() * 4, cudaMemcpyHostToDevice);
    return (float*)d;
  }
};

void stack_rows(std::vector<float>& dst, const HostTensor* t);

// Frequencies of a rotation over `dims` dimensions: base^(-2i / dims), interpolated between two wavelengths when a
// factor is given (pairs that turn more than `fast` times over `original` positions keep their frequency, pairs that
// turn fewer than `slow` times are divided by the factor, a linear ramp over the pair index lies between), and the factor
// 0.1 ln(factor) + 1 on cosine and sine.
void rotation_table(const hy_layer_cfg& c, std::vector<double>& f, float* mag) {
  const int dims = c.r_dims;
  f.resize((size_t)dims / 2);
  const double base = (double)c.r_base;
  for (int i = 0; i < dims / 2; ++i) f[(size_t)i] = pow(base, -2.0 * (double)i / (double)dims);
  *mag = 1.0f;
  if (c.r_factor > 0.0f && dims > 0) {
    const double kPi = 3.14159265358979323846;
    auto turn_dim = [&](double turns) { return (double)dims * log((double)c.r_original / (2.0 * kPi * turns)) / (2.0 * log(base)); };
    const double lo = std::max(floor(turn_dim((double)c.r_fast)), 0.0);
    const double hi = std::min(ceil(turn_dim((double)c.r_slow)), (double)(dims - 1));
    for (int i = 0; i < dims / 2; ++i) {
      const double ramp = std::min(std::max(((double)i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
      f[(size_t)i] = f[(size_t)i] / (double)c.r_factor * ramp + f[(size_t)i] * (1.0 - ramp);
    }
    *mag = (float)(0.1 * log((double)c.r_factor) + 1.0);
  }
}

struct Maxima { int in = 1, out = 1, cv = 1, f1 = 1, f2 = 1; };

bool tanh_norm_load(Builder& B, const std::string& name, int W, TanhNorm* n) {
  const HostTensor* w = B.get(name, W, -1);
  const HostTensor* b = B.get(name + ".b", W, -1);
  auto it = B.h->host.find(name + ".alpha");
  if (it == B.h->host.end() || it->second.v.size() != 1) {
    if (B.rc == HY_OK) B.rc = fail(B.h, HY_ERR_INVALID, "missing or non-scalar tensor " + name + ".alpha");
    return false;
  }
  if (!w || !b) return false;
  n->w = B.up_f32(w->v);
  n->b = B.up_f32(b->v);
  n->alpha = it->second.v[0];
  return true;
}

// Router and gated experts of a routed feed-forward ("<p>mlp.router", "<p>mlp.e<j>.gate / .up / .down"): stacked per expert
// [gate rows | up rows] and [width, ff]; for the tensor-core product also as swizzled tiles per expert whose rows
// alternate 16 gate features and the 16 up features that go with them.
int load_gated_experts(hy_engine* h, Builder& B, LayerW& L, const hy_layer_cfg& c, const std::string& p, Maxima& mx) {
  const int W = h->m.width;
  const int E = c.x_experts, ff = c.ff;
  if (auto t = B.get(p + "mlp.router", E, W)) { L.w_router = B.up(t->v); L.w_router_t = B.up_tiled(t->v, E, W); }
  std::vector<float> gu, dn;
  gu.reserve((size_t)E * 2 * ff * W);
  dn.reserve((size_t)E * W * ff);
  for (int e = 0; e < E && B.rc == HY_OK; ++e) {
    const std::string x = p + "mlp.e" + std::to_string(e) + ".";
    stack_rows(gu, B.get(x + "gate", ff, W));
    stack_rows(gu, B.get(x + "up", ff, W));
    stack_rows(dn, B.get(x + "down", W, ff));
  }
  if (B.rc != HY_OK) return B.rc;
  L.w_gu = B.up(gu);
  L.w_down = B.up(dn);
  if (h->m.dtype == HY_DTYPE_BF16 && W % 8 == 0 && ff % 8 == 0) {
    // per expert: rows [32 b, 32 b + 16) = gate features [16 b, ...), rows [32 b + 16, 32 b + 32) = the up features
    const int fb = (ff + 15) / 16, rows = fb * 32;
    std::vector<float> il((size_t)rows * W);
    std::vector<uint16_t> all, one;
    for (int e = 0; e < E; ++e) {
      std::fill(il.begin(), il.end(), 0.0f);
      const float* g = &gu[(size_t)e * 2 * ff * W];
      for (int f = 0; f < ff; ++f) {
        memcpy(&il[((size_t)(f / 16) * 32 + f % 16) * W], g + (size_t)f * W, (size_t)W * 4);
        memcpy(&il[((size_t)(f / 16) * 32 + 16 + f % 16) * W], g + (size_t)(ff + f) * W, (size_t)W * 4);
      }
      pack_tiles(il.data(), rows, W, one);
      all.insert(all.end(), one.begin(), one.end());
      L.gu_t_stride = one.size();
    }
    L.gu_rows = rows;
    if (dev_alloc(h, &L.w_gu_t, all.size() * 2, &h->bytes_w) != HY_OK) return HY_ERR_CUDA;
    cudaMemcpy(L.w_gu_t, all.data(), all.size() * 2, cudaMemcpyHostToDevice);
    all.clear();
    for (int e = 0; e < E; ++e) {
      pack_tiles(&dn[(size_t)e * W * ff], W, ff, one);
      all.insert(all.end(), one.begin(), one.end());
      L.down_t_stride = one.size();
    }
    if (dev_alloc(h, &L.w_down_t, all.size() * 2, &h->bytes_w) != HY_OK) return HY_ERR_CUDA;
    cudaMemcpy(L.w_down_t, all.data(), all.size() * 2, cudaMemcpyHostToDevice);
  }
  mx.f1 = std::max(mx.f1, E);
  mx.in = std::max(mx.in, c.x_top * ((ff + 7) & ~7));
  mx.f2 = std::max(mx.f2, c.x_top * W);
  return B.rc;
}

// One layer of a norm - sublayer - norm model: its norms and layer scales, the mixer's merged input projection, the
// mixer's small tensors, its output projection, state and cache, and the experts.
int finalize_sandwich_layer(hy_engine* h, Builder& B, size_t i, Maxima& mx) {
  const hy_layer_cfg& c = h->lc[i];
  const hy_runtime_cfg& rt = h->rt;
  LayerW& L = h->lw[i];
  const int W = h->m.width;
  const std::string p = "l" + std::to_string(i) + ".", d = p + "mix.";
  tanh_norm_load(B, p + "norm1", W, &L.n1);
  tanh_norm_load(B, p + "norm1b", W, &L.n1b);
  if (auto t = B.get(p + "ls1", W, -1)) L.ls1 = B.up_f32(t->v);
  std::vector<float> win;
  int n_in = 0, k_out = 0;
  if (c.mixer == HY_MIX_SSD) {
    const int H = c.m_heads, inner = H * c.m_vdim, GN = c.m_groups * c.m_state, C = inner + 2 * GN;
    n_in = 2 * inner + 2 * GN + H;
    stack_rows(win, B.get(d + "in", n_in, W));
    if (auto t = B.get(d + "conv", C, c.m_conv)) L.m_conv_w = B.up(t->v);
    if (auto t = B.get(d + "conv.b", C, -1)) L.m_conv_b = B.up(t->v);
    if (auto t = B.get(d + "dt_bias", H, -1)) L.m_dt_bias = B.up_f32(t->v);
    if (auto t = B.get(d + "A_log", H, -1)) L.m_A_log = B.up_f32(t->v);
    if (auto t = B.get(d + "D", H, -1)) L.m_D = B.up_f32(t->v);
    if (auto t = B.get(d + "norm", inner, -1)) L.m_norm = B.up_f32(t->v);
    k_out = inner;
    mx.in = std::max(mx.in, n_in); mx.cv = std::max(mx.cv, C); mx.f2 = std::max(mx.f2, inner);
    if (dev_alloc(h, (void**)&L.conv_state, (size_t)rt.num_slots * (c.m_conv - 1) * C * 4, &h->bytes_state)) return HY_ERR_CUDA;
    if (dev_alloc(h, (void**)&L.rec_state, (size_t)rt.num_slots * inner * c.m_state * 4, &h->bytes_state)) return HY_ERR_CUDA;
  } else if (c.mixer == HY_MIX_LATENT) {
    const int H = c.l_heads, R = c.l_kv_rank, rot = c.l_rot_dim, Dk = R + rot;
    const bool own = c.l_kv_from < 0;
    n_in = c.l_q_rank + (own ? Dk : 0);
    stack_rows(win, B.get(d + "dq", c.l_q_rank, W));
    if (own) stack_rows(win, B.get(d + "dkv", Dk, W));
    if (auto t = B.get(d + "dq.norm", c.l_q_rank, -1)) L.l_qn = B.up_f32(t->v);
    if (own) { if (auto t = B.get(d + "dkv.norm", R, -1)) L.l_kn = B.up_f32(t->v); }
    const int nq = H * (c.l_dim + rot);
    if (auto t = B.get(d + "uq", nq, c.l_q_rank)) { L.w_uq = B.up(t->v); L.w_uq_t = B.up_tiled(t->v, nq, c.l_q_rank); }
    if (auto t = B.get(d + "uk", H * c.l_dim, R)) {
      L.w_uk = B.up(t->v);
      std::vector<float> tr((size_t)H * R * c.l_dim);            // [H][rank][dim]
      for (int hh = 0; hh < H; ++hh)
        for (int k = 0; k < c.l_dim; ++k)
          for (int r = 0; r < R; ++r) tr[((size_t)hh * R + r) * c.l_dim + k] = t->v[((size_t)hh * c.l_dim + k) * R + r];
      L.w_ukT = B.up(tr);
    }
    if (auto t = B.get(d + "uv", H * c.l_vdim, R)) {
      L.w_uv = B.up(t->v);
      std::vector<float> tr((size_t)H * R * c.l_vdim);           // [H][rank][vdim]
      for (int hh = 0; hh < H; ++hh)
        for (int j = 0; j < c.l_vdim; ++j)
          for (int r = 0; r < R; ++r) tr[((size_t)hh * R + r) * c.l_vdim + j] = t->v[((size_t)hh * c.l_vdim + j) * R + r];
      L.w_uvT = B.up(tr);
    }
    if (auto t = B.get(d + "sink", H, -1)) L.sink = B.up(t->v);
    {
      std::vector<double> f;
      rotation_table(c, f, &L.rot.mag);
      void* dv = nullptr;
      if (dev_alloc(h, &dv, f.size() * 8, &h->bytes_w) != HY_OK) return HY_ERR_CUDA;
      cudaMemcpy(dv, f.data(), f.size() * 8, cudaMemcpyHostToDevice);
      L.rot.freq = (const double*)dv;
      L.rot.pairs = (int)f.size();
    }
    k_out = H * c.l_vdim;
    mx.f1 = std::max(mx.f1, n_in);
    mx.cv = std::max(mx.cv, std::max(c.l_q_rank, H * Dk));
    mx.in = std::max(mx.in, nq);
    mx.f2 = std::max(mx.f2, H * R);
    if (own) {
      if (dev_alloc(h, &L.cache, (size_t)rt.num_pages * rt.page_size * Dk * h->esz(), &h->bytes_cache)) return HY_ERR_CUDA;
    } else {
      L.cache = h->lw[(size_t)c.l_kv_from].cache;
    }
  } else {
    const int H = c.g_heads, nq = H * c.g_dim, nv = H * c.g_vdim;
    n_in = 2 * nq + nv;
    L.c_q = 0; L.c_k = nq; L.c_v = 2 * nq;
    stack_rows(win, B.get(d + "q", nq, W));
    stack_rows(win, B.get(d + "f", nq, W));
    stack_rows(win, B.get(d + "v", nv, W));
    if (auto t = B.get(d + "f.b", nq, -1)) L.g_fb = B.up_f32(t->v);
    if (auto t = B.get(d + "lower", nq, -1)) L.g_lower = B.up_f32(t->v);
    if (auto t = B.get(d + "norm", c.g_vdim, -1)) L.g_norm = B.up_f32(t->v);
    k_out = nv;
    mx.in = std::max(mx.in, n_in);
    if (dev_alloc(h, (void**)&L.rec_state, (size_t)rt.num_slots * H * c.g_dim * c.g_vdim * 4, &h->bytes_state)) return HY_ERR_CUDA;
  }
  const HostTensor* wo = B.get(d + "o", W, k_out);
  if (B.rc != HY_OK) return B.rc;
  L.n_in = n_in; L.c_up = n_in;
  L.w_in = B.up(win);
  L.w_in_t = B.up_tiled(win, n_in, W);
  L.k_out = k_out;
  L.w_out = B.up(wo->v);
  L.w_out_t = B.up_tiled(wo->v, W, k_out);
  mx.out = std::max(mx.out, k_out);
  if (c.ff_kind == HY_FF_ROUTED) {
    tanh_norm_load(B, p + "norm2", W, &L.n2);
    tanh_norm_load(B, p + "norm2b", W, &L.n2b);
    if (auto t = B.get(p + "ls2", W, -1)) L.ls2 = B.up_f32(t->v);
    if (int rc = load_gated_experts(h, B, L, c, p, mx)) return rc;
  }
  return B.rc;
}

// Rows of a [gate rows | up rows] matrix (ff each) reordered for the tensor-core product's gated epilogue: rows
// [32 b, 32 b + 16) = gate features [16 b, 16 b + 16), rows [32 b + 16, 32 b + 32) = the up features that go with them.
void interleave_gate_up(const float* gu, int ff, int W, std::vector<float>& il, int* rows) {
  const int fb = (ff + 15) / 16;
  *rows = fb * 32;
  il.assign((size_t)*rows * W, 0.0f);
  for (int f = 0; f < ff; ++f) {
    memcpy(&il[((size_t)(f / 16) * 32 + f % 16) * W], gu + (size_t)f * W, (size_t)W * 4);
    memcpy(&il[((size_t)(f / 16) * 32 + 16 + f % 16) * W], gu + (size_t)(ff + f) * W, (size_t)W * 4);
  }
}

// Gated dense feed-forward ("<p>mlp.gate / .up / .down"): [gate rows | up rows] stacked, and for the tensor-core product as
// tiles whose rows alternate 16 gate and 16 up features.
int load_gated_dense(hy_engine* h, Builder& B, LayerW& L, const hy_layer_cfg& c, const std::string& p, Maxima& mx) {
  const int W = h->m.width, ff = c.ff;
  std::vector<float> gu;
  stack_rows(gu, B.get(p + "mlp.gate", ff, W));
  stack_rows(gu, B.get(p + "mlp.up", ff, W));
  const HostTensor* dn = B.get(p + "mlp.down", W, ff);
  if (B.rc != HY_OK) return B.rc;
  L.w_ff_in = B.up(gu);
  if (h->m.dtype == HY_DTYPE_BF16 && W % 8 == 0 && ff % 8 == 0) {
    std::vector<float> il;
    interleave_gate_up(gu.data(), ff, W, il, &L.ff_rows);
    L.w_ff_in_t = B.up_tiled(il, L.ff_rows, W);
  }
  L.w_ff_down = B.up(dn->v);
  L.w_ff_down_t = B.up_tiled(dn->v, W, ff);
  mx.in = std::max(mx.in, 2 * ff);
  mx.out = std::max(mx.out, ff);
  return B.rc;
}

void* upload_rotation(hy_engine* h, const std::vector<double>& f) {
  void* dv = nullptr;
  if (dev_alloc(h, &dv, f.size() * 8, &h->bytes_w) != HY_OK) return nullptr;
  cudaMemcpy(dv, f.data(), f.size() * 8, cudaMemcpyHostToDevice);
  return dv;
}

// One layer of a model whose sublayers read the stream itself and are RMS-normed on the way back: the two norms and layer
// scales, the mixer's merged input projection with its small tensors, output projection, cache or state, and the
// feed-forward (gated dense, or routed plain experts with a router bias and a shared expert).
int finalize_postnorm_layer(hy_engine* h, Builder& B, size_t i, Maxima& mx) {
  const hy_layer_cfg& c = h->lc[i];
  const hy_runtime_cfg& rt = h->rt;
  LayerW& L = h->lw[i];
  const int W = h->m.width;
  const std::string p = "l" + std::to_string(i) + ".", d = p + "mix.";
  if (auto t = B.get(p + "norm1", W, -1)) L.pn1 = B.up_f32(t->v);
  if (auto t = B.get(p + "ls1", W, -1)) L.ls1 = B.up_f32(t->v);
  std::vector<float> win;
  int n_in = 0, k_out = 0;
  if (c.mixer == HY_MIX_WINDOW) {
    const int H = c.w_heads, G = c.w_kv_heads, D = c.w_dim, Dv = c.w_vdim;
    L.c_q = 0; L.c_k = H * D; L.c_v = H * D + G * D;
    n_in = H * D + G * D + G * Dv;
    stack_rows(win, B.get(d + "q", H * D, W));
    stack_rows(win, B.get(d + "k", G * D, W));
    stack_rows(win, B.get(d + "v", G * Dv, W));
    if (c.w_qk_norm) {
      if (auto t = B.get(d + "q.norm", D, -1)) L.w_qn = B.up_f32(t->v);
      if (auto t = B.get(d + "k.norm", D, -1)) L.w_kn = B.up_f32(t->v);
    }
    std::vector<double> f((size_t)c.w_rot_dims / 2), fv(c.w_rot_values ? (size_t)Dv / 2 : 0);
    for (size_t j = 0; j < f.size(); ++j) f[j] = pow((double)c.w_rot_base, -2.0 * (double)j / (double)c.w_rot_dims);
    for (size_t j = 0; j < fv.size(); ++j) fv[j] = pow((double)c.w_rot_base, -2.0 * (double)j / (double)Dv);
    L.rot = Rotation{(const double*)upload_rotation(h, f), (int)f.size(), 1.0f};
    L.rot_v = Rotation{(const double*)upload_rotation(h, fv), (int)fv.size(), 1.0f};
    k_out = H * Dv;
    mx.in = std::max(mx.in, n_in); mx.cv = std::max(mx.cv, H * D); mx.f1 = std::max(mx.f1, Dv);
    const size_t rows = (size_t)rt.num_pages * G * rt.page_size;
    const size_t prow = (size_t)rt.num_pages * G * window_block_slots(rt.page_size, c.w_pool);
    if (dev_alloc(h, &L.cache, rows * D * h->esz(), &h->bytes_cache)) return HY_ERR_CUDA;
    if (dev_alloc(h, &L.cache_v, rows * Dv * h->esz(), &h->bytes_cache)) return HY_ERR_CUDA;
    if (dev_alloc(h, &L.pool_k, prow * D * h->esz(), &h->bytes_cache)) return HY_ERR_CUDA;
    if (dev_alloc(h, &L.pool_v, prow * Dv * h->esz(), &h->bytes_cache)) return HY_ERR_CUDA;
  } else {
    const int H = c.t_heads, nq = H * c.t_dim, nv = H * c.t_vdim;
    L.c_q = 0; L.c_k = nq; L.c_v = 2 * nq; L.c_g = 2 * nq + nv; L.c_i = 2 * nq + 2 * nv;
    n_in = L.c_i + 2 * H;
    stack_rows(win, B.get(d + "q", nq, W));
    stack_rows(win, B.get(d + "k", nq, W));
    stack_rows(win, B.get(d + "v", nv, W));
    stack_rows(win, B.get(d + "g", nv, W));
    stack_rows(win, B.get(d + "i", H, W));
    stack_rows(win, B.get(d + "f", H, W));
    if (auto t = B.get(d + "i.b", H, -1)) L.t_ib = B.up_f32(t->v);
    if (auto t = B.get(d + "f.b", H, -1)) L.t_fb = B.up_f32(t->v);
    if (auto t = B.get(d + "norm", nv, -1)) L.t_norm = B.up_f32(t->v);
    k_out = nv;
    mx.in = std::max(mx.in, L.c_i); mx.f1 = std::max(mx.f1, 2 * H);
    const size_t per_head = (size_t)c.t_dim * (c.t_vdim + 1) + 1;
    if (dev_alloc(h, (void**)&L.rec_state, (size_t)rt.num_slots * H * per_head * 4, &h->bytes_state)) return HY_ERR_CUDA;
  }
  const HostTensor* wo = B.get(d + "o", W, k_out);
  if (B.rc != HY_OK) return B.rc;
  L.n_in = n_in; L.c_up = n_in;
  L.w_in = B.up(win);
  L.w_in_t = B.up_tiled(win, n_in, W);
  L.k_out = k_out;
  L.w_out = B.up(wo->v);
  L.w_out_t = B.up_tiled(wo->v, W, k_out);
  mx.out = std::max(mx.out, k_out);
  mx.f2 = std::max(mx.f2, W);
  if (c.ff_kind == HY_FF_NONE) return B.rc;
  if (auto t = B.get(p + "norm2", W, -1)) L.pn2 = B.up_f32(t->v);
  if (auto t = B.get(p + "ls2", W, -1)) L.ls2 = B.up_f32(t->v);
  const int ff = c.ff;
  if (c.ff_kind == HY_FF_GATED) return load_gated_dense(h, B, L, c, p, mx);
  const int E = c.x_experts;
  if (auto t = B.get(p + "mlp.router", E, W)) { L.w_router = B.up(t->v); L.w_router_t = B.up_tiled(t->v, E, W); }
  if (c.x_route == HY_ROUTE_TOP_SOFTMAX) { if (auto t = B.get(p + "mlp.router.b", E, -1)) L.x_rb = B.up_f32(t->v); }
  std::vector<float> up, dn;
  up.reserve((size_t)E * ff * W);
  dn.reserve((size_t)E * W * ff);
  for (int e = 0; e < E && B.rc == HY_OK; ++e) {
    const std::string x = p + "mlp.e" + std::to_string(e) + ".";
    stack_rows(up, B.get(x + "up", ff, W));
    stack_rows(dn, B.get(x + "down", W, ff));
  }
  if (B.rc != HY_OK) return B.rc;
  L.w_gu = B.up(up);
  L.w_down = B.up(dn);
  if (h->m.dtype == HY_DTYPE_BF16 && W % 8 == 0 && ff % 8 == 0) {
    std::vector<uint16_t> all, one;
    for (int e = 0; e < E; ++e) {
      pack_tiles(&up[(size_t)e * ff * W], ff, W, one);
      all.insert(all.end(), one.begin(), one.end());
      L.gu_t_stride = one.size();
    }
    L.gu_rows = ff;
    if (dev_alloc(h, &L.w_gu_t, all.size() * 2, &h->bytes_w) != HY_OK) return HY_ERR_CUDA;
    cudaMemcpy(L.w_gu_t, all.data(), all.size() * 2, cudaMemcpyHostToDevice);
    all.clear();
    for (int e = 0; e < E; ++e) {
      pack_tiles(&dn[(size_t)e * W * ff], W, ff, one);
      all.insert(all.end(), one.begin(), one.end());
      L.down_t_stride = one.size();
    }
    if (dev_alloc(h, &L.w_down_t, all.size() * 2, &h->bytes_w) != HY_OK) return HY_ERR_CUDA;
    cudaMemcpy(L.w_down_t, all.data(), all.size() * 2, cudaMemcpyHostToDevice);
  }
  if (c.x_shared_ff > 0) {
    const int sf = c.x_shared_ff;
    if (auto t = B.get(p + "mlp.shared.up", sf, W)) { L.w_sh_up = B.up(t->v); L.w_sh_up_t = B.up_tiled(t->v, sf, W); }
    if (auto t = B.get(p + "mlp.shared.down", W, sf)) { L.w_sh_down = B.up(t->v); L.w_sh_down_t = B.up_tiled(t->v, W, sf); }
    mx.out = std::max(mx.out, sf);
  }
  mx.f1 = std::max(mx.f1, E);
  mx.in = std::max(mx.in, c.x_top * ((ff + 7) & ~7));
  mx.f2 = std::max(mx.f2, (c.x_top + 1) * W);
  return B.rc;
}

// [width, taps] -> [taps, width]: the convolution kernel reads a tap's weights along the width
std::vector<float> tap_major(const std::vector<float>& w, int W, int taps) {
  std::vector<float> o((size_t)W * taps);
  for (int c = 0; c < W; ++c)
    for (int i = 0; i < taps; ++i) o[(size_t)i * W + c] = w[(size_t)c * taps + i];
  return o;
}

// One layer of a pre-norm model: norms, layer scales, input convolutions with their tails, the biased attention's merged
// projection with its bias, pages for keys and values, the feed-forward, the token input and the depth average's weights.
int finalize_prenorm_layer(hy_engine* h, Builder& B, size_t i, Maxima& mx) {
  const hy_layer_cfg& c = h->lc[i];
  const hy_runtime_cfg& rt = h->rt;
  LayerW& L = h->lw[i];
  const int W = h->m.width, taps = h->m.canon_taps;
  const std::string p = "l" + std::to_string(i) + ".", d = p + "mix.";
  auto scalar = [&](const std::string& name, float* out) {
    auto it = h->host.find(name);
    if (it == h->host.end() || it->second.v.size() != 1) {
      if (B.rc == HY_OK) B.rc = fail(h, HY_ERR_INVALID, "missing or non-scalar tensor " + name);
      return;
    }
    *out = it->second.v[0];
  };
  if (auto t = B.get(p + "norm1", W, -1)) L.pn1 = B.up_f32(t->v);
  if (auto t = B.get(p + "ls1", W, -1)) L.ls1 = B.up_f32(t->v);
  if (taps > 0) {
    if (auto t = B.get(p + "canon1", W, taps)) L.canon1 = B.up_f32(tap_major(t->v, W, taps));
    if (dev_alloc(h, (void**)&L.conv_state, (size_t)rt.num_slots * (taps - 1) * W * 4, &h->bytes_state)) return HY_ERR_CUDA;
  }
  if (h->m.depth_avg) { if (auto t = B.get(p + "dwa", (int64_t)i + 2, -1)) L.dwa = B.up_f32(t->v); }
  const int H = c.b_heads, G = c.b_kv_heads, D = c.b_dim, Dv = c.b_vdim;
  const int n_in = H * D + G * D + G * Dv;
  L.c_q = 0; L.c_k = H * D; L.c_v = H * D + G * D;
  std::vector<float> win, bias;
  stack_rows(win, B.get(d + "q", H * D, W));
  stack_rows(win, B.get(d + "k", G * D, W));
  stack_rows(win, B.get(d + "v", G * Dv, W));
  stack_rows(bias, B.get(d + "q.b", H * D, -1));
  stack_rows(bias, B.get(d + "k.b", G * D, -1));
  stack_rows(bias, B.get(d + "v.b", G * Dv, -1));
  if (auto t = B.get(d + "r1", H, -1)) L.b_r1 = B.up_f32(t->v);
  if (auto t = B.get(d + "r2", H, -1)) L.b_r2 = B.up_f32(t->v);
  if (auto t = B.get(d + "sink", H, -1)) L.b_sink = B.up_f32(t->v);
  if (c.b_v_mix) {
    L.b_mix = 1;
    for (size_t j = 0; j < i; ++j) if (h->lc[j].b_v_mix) L.b_mix = 2;
    if (L.b_mix == 2) scalar(d + "vmix", &L.b_lambda);
    h->ld_vf = std::max(h->ld_vf, (G * Dv + 7) & ~7);
  }
  const HostTensor* wo = B.get(d + "o", W, H * Dv);
  if (B.rc != HY_OK) return B.rc;
  L.n_in = n_in; L.c_up = n_in;
  L.w_in = B.up(win);
  L.w_in_t = B.up_tiled(win, n_in, W);
  L.b_bias = B.up_f32(bias);
  L.k_out = H * Dv;
  L.w_out = B.up(wo->v);
  L.w_out_t = B.up_tiled(wo->v, W, L.k_out);
  mx.in = std::max(mx.in, n_in); mx.out = std::max(mx.out, L.k_out); mx.f2 = std::max(mx.f2, W);
  const size_t rows = (size_t)rt.num_pages * G * rt.page_size;
  if (dev_alloc(h, &L.cache, rows * D * h->esz(), &h->bytes_cache)) return HY_ERR_CUDA;
  if (dev_alloc(h, &L.cache_v, rows * Dv * h->esz(), &h->bytes_cache)) return HY_ERR_CUDA;
  if (h->m.side_dim > 0) {
    const int sd = h->m.side_dim;
    if (auto t = B.get(p + "side.gate", sd, W)) L.side_gate = B.up(t->v);
    if (auto t = B.get(p + "side.proj", W, sd)) {           // kept transposed [sd, W]: a token's row kernel reads it along the width
      std::vector<float> tr((size_t)sd * W);
      for (int r = 0; r < W; ++r)
        for (int k = 0; k < sd; ++k) tr[(size_t)k * W + r] = t->v[(size_t)r * sd + k];
      L.side_proj = B.up(tr);
    }
    if (auto t = B.get(p + "side.norm", W, -1)) L.side_norm = B.up_f32(t->v);
  }
  if (c.ff_kind == HY_FF_NONE) return B.rc;
  if (auto t = B.get(p + "norm2", W, -1)) L.pn2 = B.up_f32(t->v);
  if (auto t = B.get(p + "ls2", W, -1)) L.ls2 = B.up_f32(t->v);
  if (taps > 0) {
    if (auto t = B.get(p + "canon2", W, taps)) L.canon2 = B.up_f32(tap_major(t->v, W, taps));
    if (dev_alloc(h, (void**)&L.conv_state2, (size_t)rt.num_slots * (taps - 1) * W * 4, &h->bytes_state)) return HY_ERR_CUDA;
  }
  if (c.ff_kind == HY_FF_GATED) return load_gated_dense(h, B, L, c, p, mx);
  return load_gated_experts(h, B, L, c, p, mx);
}

// rows of several [n_i, k] matrices stacked
void stack_rows(std::vector<float>& dst, const HostTensor* t) { if (t) dst.insert(dst.end(), t->v.begin(), t->v.end()); }

}  // namespace

extern "C" int hy_finalize(hy_handle h) {
  if (!h) return HY_ERR_INVALID;
  if (h->finalized) return HY_OK;
  HY_CUDA(cudaSetDevice(h->rt.device));
  Builder B{h};
  const int W = h->m.width, V = h->m.vocab;
  const hy_runtime_cfg& rt = h->rt;
  if (auto t = B.get("embed", V, W)) h->embed = B.up(t->v);
  if (h->m.norm_kind == HY_NORM_TANH) tanh_norm_load(B, "final.norm", W, &h->final_tanh);
  else if (auto t = B.get("final.norm", W, -1)) h->final_norm = B.up(t->v);
  if (h->m.embed_norm) { if (auto t = B.get("embed.norm", W, -1)) h->embed_norm = B.up_f32(t->v); }
  if (h->m.block_kind == HY_BLOCK_PRENORM) {
    if (h->m.pair_buckets > 0) { if (auto t = B.get("bigram", (int64_t)h->m.pair_buckets + 1, W)) h->pair_table = B.up(t->v); }
    if (h->m.side_dim > 0) { if (auto t = B.get("side.embed", V, (int64_t)h->m.side_dim * h->m.n_layers)) h->side_table = B.up(t->v); }
  }
  if (h->m.tied_head) {
    h->head = h->embed;
    if (auto t = B.get("embed", V, W)) h->head_t = B.up_tiled(t->v, V, W);
  } else if (auto t = B.get("head", V, W)) { h->head = B.up(t->v); h->head_t = B.up_tiled(t->v, V, W); }
  if (h->m.pos_kind == HY_POS_SINUSOID) {
    std::vector<double> f((W + 1) / 2);
    for (size_t i = 0; i < f.size(); ++i) f[i] = pow(10000.0, -2.0 * (double)i / (double)W);
    void* d = nullptr;
    if (dev_alloc(h, &d, f.size() * 8, &h->bytes_w) != HY_OK) return HY_ERR_CUDA;
    cudaMemcpy(d, f.data(), f.size() * 8, cudaMemcpyHostToDevice);
    h->inv_freq = (double*)d;
  }
  h->lw.resize(h->lc.size());
  int max_in = 1, max_out = 1, max_cv = 1, max_f1 = 1, max_f2 = 1;
  Maxima mx;
  for (size_t i = 0; i < h->lc.size() && B.rc == HY_OK; ++i) {
    const hy_layer_cfg& c = h->lc[i];
    LayerW& L = h->lw[i];
    if (h->m.block_kind != HY_BLOCK_PARALLEL) {
      const int rc = h->m.block_kind == HY_BLOCK_SANDWICH ? finalize_sandwich_layer(h, B, i, mx)
                     : h->m.block_kind == HY_BLOCK_POSTNORM ? finalize_postnorm_layer(h, B, i, mx) : finalize_prenorm_layer(h, B, i, mx);
      if (rc != HY_OK) return rc;
      continue;
    }
    const std::string p = "l" + std::to_string(i) + ".";
    if (auto t = B.get(p + "norm1", W, -1)) L.norm1 = B.up(t->v);
    const int ff = c.ff_kind == HY_FF_NONE ? 0 : c.ff;
    std::vector<float> win, wout;
    int n_in = 0;
    std::vector<const HostTensor*> outs;       // output projections to concatenate along k
    if (c.mixer == HY_MIX_ATTN_SCAN) {
      const std::string a = p + "mix.left.", s = p + "mix.right.";
      const int nq = c.a_heads * c.a_dim, nk = c.a_kv_heads * c.a_dim, nv = c.a_heads * c.a_vdim;
      const int R = c.s_dt_rank, N = c.s_state, I = c.s_inner;
      L.c_q = n_in; stack_rows(win, B.get(a + "q", nq, W)); n_in += nq;
      L.c_k = n_in; stack_rows(win, B.get(a + "k", nk, W)); n_in += nk;
      L.c_g = n_in; stack_rows(win, B.get(a + "g", nv, W)); n_in += nv;
      L.c_x = n_in; L.c_z = n_in + I; stack_rows(win, B.get(s + "in", 2 * I, W)); n_in += 2 * I;
      std::vector<float> cw;
      stack_rows(cw, B.get(a + "q.conv", nq, c.a_conv));
      stack_rows(cw, B.get(a + "k.conv", nk, c.a_conv));
      L.conv_qk = B.up(cw);
      if (auto t = B.get(a + "sink", c.a_heads, -1)) L.sink = B.up(t->v);
      if (auto t = B.get(s + "conv", I, c.s_conv)) L.conv_x = B.up(t->v);
      if (auto t = B.get(s + "conv.b", I, -1)) L.conv_xb = B.up(t->v);
      if (auto t = B.get(s + "x", R + 2 * N, I)) { L.w_x = B.up(t->v); L.w_x_t = B.up_tiled(t->v, R + 2 * N, I); }
      if (auto t = B.get(s + "dt", I, R)) L.w_dt = B.up(t->v);
      if (auto t = B.get(s + "dt.b", I, -1)) L.dt_b = B.up(t->v);
      if (auto t = B.get(s + "A_log", I, N)) {
        std::vector<float> an(t->v.size());
        for (size_t j = 0; j < an.size(); ++j) an[j] = -expf(t->v[j]);
        L.A_neg = B.up_f32(an);
      }
      if (auto t = B.get(s + "D", I, -1)) L.D = B.up(t->v);
      outs.push_back(B.get(a + "o", W, nv));
      outs.push_back(B.get(s + "o", W, I));
      L.o_mix = 0; L.o_scan = nv; L.o_ff = nv + I;
      max_cv = std::max(max_cv, std::max(nq + nk, I));
      max_f1 = std::max(max_f1, R + 2 * N);
      max_f2 = std::max(max_f2, I);
      // state: conv tails and the scan state, key pages
      if (dev_alloc(h, (void**)&L.conv_state, (size_t)rt.num_slots * (c.a_conv - 1) * (nq + nk) * 4, &h->bytes_state)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&L.conv_state2, (size_t)rt.num_slots * (c.s_conv - 1) * I * 4, &h->bytes_state)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&L.rec_state, (size_t)rt.num_slots * I * N * 4, &h->bytes_state)) return HY_ERR_CUDA;
      if (dev_alloc(h, &L.cache, (size_t)rt.num_pages * c.a_kv_heads * rt.page_size * c.a_dim * h->esz(), &h->bytes_cache)) return HY_ERR_CUDA;
    } else {
      const std::string d = p + "mix.";
      const int nq = c.d_kv_heads * c.d_dim, nv = c.d_heads * c.d_vdim;
      L.c_q = n_in; stack_rows(win, B.get(d + "q", nq, W)); n_in += nq;
      L.c_k = n_in; stack_rows(win, B.get(d + "k", nq, W)); n_in += nq;
      L.c_v = n_in; stack_rows(win, B.get(d + "v", nv, W)); n_in += nv;
      L.c_b = n_in; stack_rows(win, B.get(d + "b", c.d_heads, W)); n_in += c.d_heads;
      L.c_a1 = n_in; stack_rows(win, B.get(d + "a1", c.d_low_a, W)); n_in += c.d_low_a;
      L.c_g1 = n_in; stack_rows(win, B.get(d + "g1", c.d_low_g, W)); n_in += c.d_low_g;
      std::vector<float> cw;
      stack_rows(cw, B.get(d + "q.conv", nq, c.d_conv));
      stack_rows(cw, B.get(d + "k.conv", nq, c.d_conv));
      stack_rows(cw, B.get(d + "v.conv", nv, c.d_conv));
      L.conv_qkv = B.up(cw);
      if (auto t = B.get(d + "a2", c.d_heads * c.d_dim, c.d_low_a)) { L.w_a2 = B.up(t->v); L.w_a2_t = B.up_tiled(t->v, c.d_heads * c.d_dim, c.d_low_a); }
      if (auto t = B.get(d + "g2", nv, c.d_low_g)) { L.w_g2 = B.up(t->v); L.w_g2_t = B.up_tiled(t->v, nv, c.d_low_g); }
      if (auto t = B.get(d + "A_log", c.d_heads, -1)) L.A_log = B.up_f32(t->v);
      if (auto t = B.get(d + "dt_bias", c.d_heads * c.d_dim, -1)) L.dt_bias = B.up_f32(t->v);
      if (auto t = B.get(d + "norm", c.d_vdim, -1)) L.norm_w = B.up_f32(t->v);
      outs.push_back(B.get(d + "o", W, nv));
      L.o_mix = 0; L.o_scan = nv; L.o_ff = nv;
      max_cv = std::max(max_cv, 2 * nq + nv);
      max_f1 = std::max(max_f1, c.d_heads * c.d_dim);
      max_f2 = std::max(max_f2, nv);
      if (dev_alloc(h, (void**)&L.conv_state, (size_t)rt.num_slots * (c.d_conv - 1) * (2 * nq + nv) * 4, &h->bytes_state)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&L.rec_state, (size_t)rt.num_slots * c.d_heads * c.d_dim * c.d_vdim * 4, &h->bytes_state)) return HY_ERR_CUDA;
    }
    L.c_up = n_in;
    if (ff) {
      stack_rows(win, B.get(p + "mlp.up", ff, W));
      outs.push_back(B.get(p + "mlp.down", W, ff));
      n_in += ff;
    }
    if (B.rc != HY_OK) break;
    L.n_in = n_in;
    L.w_in = B.up(win);
    L.w_in_t = B.up_tiled(win, n_in, W);
    int k_out = 0;
    for (auto t : outs) k_out += (int)t->cols();
    L.k_out = k_out;
    wout.resize((size_t)W * k_out);
    int off = 0;
    for (auto t : outs) {
      const int kc = (int)t->cols();
      for (int r = 0; r < W; ++r) memcpy(&wout[(size_t)r * k_out + off], &t->v[(size_t)r * kc], (size_t)kc * 4);
      off += kc;
    }
    L.w_out = B.up(wout);
    L.w_out_t = B.up_tiled(wout, W, k_out);
    max_in = std::max(max_in, L.c_up);
    max_out = std::max(max_out, k_out);
  }
  if (B.rc != HY_OK) return B.rc;
  h->host.clear();
  max_in = std::max(max_in, mx.in); max_out = std::max(max_out, mx.out); max_cv = std::max(max_cv, mx.cv);
  max_f1 = std::max(max_f1, mx.f1); max_f2 = std::max(max_f2, mx.f2);
  // workspace
  const size_t T = (size_t)rt.max_step_tokens, es = h->esz();
  auto r8 = [](int v) { return (v + 7) & ~7; };
  h->ld_pin = r8(max_in); h->ld_cat = r8(max_out); h->ld_cv = r8(max_cv); h->ld_f1 = r8(max_f1); h->ld_f2 = r8(max_f2);
  if (dev_alloc(h, (void**)&h->x, T * W * 4, &h->bytes_ws)) return HY_ERR_CUDA;
  if (dev_alloc(h, &h->hbuf, T * W * es, &h->bytes_ws)) return HY_ERR_CUDA;
  if (dev_alloc(h, &h->pin, T * h->ld_pin * es, &h->bytes_ws)) return HY_ERR_CUDA;
  if (dev_alloc(h, &h->cat, T * h->ld_cat * es, &h->bytes_ws)) return HY_ERR_CUDA;
  if (dev_alloc(h, &h->cv, T * h->ld_cv * es, &h->bytes_ws)) return HY_ERR_CUDA;
  if (dev_alloc(h, (void**)&h->f1, T * h->ld_f1 * 4, &h->bytes_ws)) return HY_ERR_CUDA;
  if (dev_alloc(h, (void**)&h->f2, T * h->ld_f2 * 4, &h->bytes_ws)) return HY_ERR_CUDA;
  if (h->m.block_kind == HY_BLOCK_PRENORM) {
    if (dev_alloc(h, (void**)&h->hn, T * W * 4, &h->bytes_ws)) return HY_ERR_CUDA;
    if (h->m.depth_avg && dev_alloc(h, (void**)&h->kept, (h->lc.size() + 1) * T * W * 4, &h->bytes_ws)) return HY_ERR_CUDA;
    if (h->ld_vf > 0 && dev_alloc(h, &h->vfirst, T * h->ld_vf * es, &h->bytes_ws)) return HY_ERR_CUDA;
    if (dev_alloc(h, (void**)&h->prev_tok, (size_t)rt.num_slots * 4, &h->bytes_state)) return HY_ERR_CUDA;
    HY_CUDA(cudaMemset(h->prev_tok, 0, (size_t)rt.num_slots * 4));
  }
  const size_t mw = (size_t)rt.max_want;
  if (dev_alloc(h, &h->hw, mw * W * es, &h->bytes_ws)) return HY_ERR_CUDA;
  if (dev_alloc(h, (void**)&h->logits, mw * V * 4, &h->bytes_ws)) return HY_ERR_CUDA;
  if (dev_alloc(h, (void**)&h->sampled, mw * 4, &h->bytes_ws)) return HY_ERR_CUDA;
  if (dev_alloc(h, (void**)&h->temp_d, mw * 4, &h->bytes_ws)) return HY_ERR_CUDA;
  h->meta_words = 3 * T + 3 * (size_t)rt.max_step_entries + 1 + (size_t)rt.max_step_entries * rt.max_pages_per_seq + mw;
  if (dev_alloc(h, (void**)&h->meta_d, h->meta_words * 4, &h->bytes_ws)) return HY_ERR_CUDA;
  HY_CUDA(cudaMallocHost((void**)&h->meta_h, h->meta_words * 4));
  if (h->m.dtype == HY_DTYPE_BF16) {
    int maxH = 0, maxG = 0, maxD = 0;
    for (auto& c : h->lc) {
      if (c.mixer == HY_MIX_ATTN_SCAN) { maxH = std::max(maxH, c.a_heads); maxG = std::max(maxG, c.a_kv_heads); maxD = std::max(maxD, c.a_dim); }
      if (c.mixer == HY_MIX_WINDOW) { maxH = std::max(maxH, c.w_heads); maxG = std::max(maxG, c.w_kv_heads); maxD = std::max(maxD, 8); }
      if (c.mixer == HY_MIX_BIASED) {                       // partial rows of the key splits are one tile row wide
        maxH = std::max(maxH, c.b_heads); maxG = std::max(maxG, c.b_kv_heads);
        maxD = std::max(maxD, (c.b_dim <= 64 && c.b_vdim <= 64) ? 64 : 128);
      }
      if (c.mixer == HY_MIX_LATENT) {
        maxH = std::max(maxH, c.l_heads); maxG = std::max(maxG, 1);
        maxD = std::max(maxD, std::max(c.l_kv_rank + c.l_rot_dim, c.l_kv_rank <= 128 ? 128 : c.l_kv_rank <= 256 ? 256 : 512));
      }
    }
    if (maxH > 0) {
      h->part_rows = std::max<size_t>(T * maxH, 4096);
      h->part_dim = (size_t)maxD;
      h->units_cap = h->part_rows / 64 + (size_t)rt.max_step_entries * maxG * 257 + 64;
      if (dev_alloc(h, (void**)&h->part_o, h->part_rows * maxD * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->part_ml, h->part_rows * 2 * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->units_d, h->units_cap * sizeof(AttnUnit), &h->bytes_ws)) return HY_ERR_CUDA;
      HY_CUDA(cudaMallocHost((void**)&h->units_h, h->units_cap * sizeof(AttnUnit)));
    }
  }
  {
    int maxE = 0, maxTop = 0;
    for (auto& c : h->lc)
      if (c.ff_kind == HY_FF_ROUTED) { maxE = std::max(maxE, c.x_experts); maxTop = std::max(maxTop, c.x_top); }
    if (maxE > 0) {
      const size_t P = T * (size_t)maxTop;
      h->x_max_tiles = (int)(P / HY_XT) + maxE + 1;          // enough for tiles of HY_XT rows and of 128 rows
      if (dev_alloc(h, (void**)&h->x_ids, P * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->x_wts, P * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->x_row_tok, P * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->x_pair_row, P * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->x_counts, (size_t)maxE * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->x_offs, ((size_t)maxE + 1) * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->x_fill, (size_t)maxE * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->x_tile_e, (size_t)h->x_max_tiles * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->x_tile_r0, (size_t)h->x_max_tiles * 4, &h->bytes_ws)) return HY_ERR_CUDA;
      if (dev_alloc(h, (void**)&h->x_meta, 16, &h->bytes_ws)) return HY_ERR_CUDA;
      HY_CUDA(cudaMemset(h->x_counts, 0, (size_t)maxE * 4));
      HY_CUDA(cudaMemset(h->x_meta, 0, 16));
    }
  }
  if (dev_alloc(h, (void**)&h->err_d, 4, &h->bytes_ws)) return HY_ERR_CUDA;
  HY_CUDA(cudaMemset(h->err_d, 0, 4));
  HY_CUDA(cudaMallocHost((void**)&h->err_h, 4));
  *h->err_h = 0;
  HY_CUDA(cudaDeviceSynchronize());
  h->finalized = true;
  return HY_OK;
}

// ---- launches ---------------------------------------------------------------------------------------------------------------------
namespace {

template <typename TA, typename TW, typename TO>
int gemm(hy_engine* h, const TA* A, int lda, const TW* Wt, int ldw, int T, int N, int K, GemmOut o,
         const void* tiled = nullptr) {
  if (T <= 0 || N <= 0) return HY_OK;
  if (o.alpha == 0.0f) o.alpha = 1.0f;
  if constexpr (std::is_same<TA, bf16>::value && std::is_same<TW, bf16>::value) {
    const size_t rb = (size_t)((K + 7) / 8 * 8) * 2;
    const bool rows_fit = T <= 8 && rb * (T == 1 ? 1 : T == 2 ? 2 : T <= 4 ? 4 : 8) <= 200 * 1024;
    if (tiled && !rows_fit && K % 8 == 0 && lda % 8 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0) {
      static bool attr_set = false;
      if (!attr_set) {
        cudaFuncSetAttribute(gemm_tc_kernel<TO, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes(128));
        cudaFuncSetAttribute(gemm_tc_kernel<TO, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes(256));
        attr_set = true;
      }
      // 256-row tiles halve the weight traffic per row; 128-row tiles when the wider ones would leave SMs without a CTA
      if (T > 128 && (long long)((N + 127) / 128) * ((T + 255) / 256) >= 148)
        gemm_tc_kernel<TO, 256><<<dim3((N + 127) / 128, (T + 255) / 256), 192, tc_smem_bytes(256), h->stream>>>(
            A, lda, (const bf16*)tiled, T, N, K, o, h->err_d, TcGroup{});
      else
        gemm_tc_kernel<TO, 128><<<dim3((N + 127) / 128, (T + 127) / 128), 192, tc_smem_bytes(128), h->stream>>>(
            A, lda, (const bf16*)tiled, T, N, K, o, h->err_d, TcGroup{});
      h->launches++;
      return HY_OK;
    }
  }
  constexpr int VECW = 16 / (int)sizeof(TW);
  const size_t row_bytes = (size_t)((K + VECW - 1) / VECW * VECW) * sizeof(TA);
  const int want_rows = T == 1 ? 1 : T == 2 ? 2 : T <= 4 ? 4 : 8;
  if (T <= 8 && row_bytes * want_rows <= 200 * 1024) {
    int ksplit = 1;
    while (ksplit < 8 && (long long)N * ksplit < 148LL * 32 && K / (ksplit * 2) >= 512) ksplit *= 2;
    const int cpb = 8 / ksplit;
    const int blocks = std::min((N + cpb - 1) / cpb, 148 * 16);
    const int fit = (int)((200 * 1024) / row_bytes);
    static bool rows_attr = false;                        // per <TA, TW, TO>: this function is a template
    if (!rows_attr) {
      cudaFuncSetAttribute(gemm_rows_kernel<TA, TW, TO, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      cudaFuncSetAttribute(gemm_rows_kernel<TA, TW, TO, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      cudaFuncSetAttribute(gemm_rows_kernel<TA, TW, TO, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      cudaFuncSetAttribute(gemm_rows_kernel<TA, TW, TO, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      rows_attr = true;
    }
    auto launch = [&](auto kern, int rows) {
      const size_t smem = (size_t)rows * row_bytes;
      kern<<<dim3(blocks, (T + rows - 1) / rows), 256, smem, h->stream>>>(A, lda, Wt, ldw, T, N, K, ksplit, o);
    };
    if (T == 1 || fit < 2) launch(gemm_rows_kernel<TA, TW, TO, 1>, 1);
    else if (T == 2 || fit < 4) launch(gemm_rows_kernel<TA, TW, TO, 2>, 2);
    else if (T <= 4 || fit < 8) launch(gemm_rows_kernel<TA, TW, TO, 4>, 4);
    else launch(gemm_rows_kernel<TA, TW, TO, 8>, 8);
  } else {
    gemm_simt_kernel<TA, TW, TO><<<dim3((N + 63) / 64, (T + 63) / 64), 256, 0, h->stream>>>(A, lda, Wt, ldw, T, N, K, o);
  }
  h->launches++;
  return HY_OK;
}

GemmOut to_buf(void* out, int ld) { return GemmOut{out, ld, 1 << 30, nullptr, 0, 0, nullptr, 0, 1.0f}; }

// Work units of the tensor-core attention for this step and this head layout; returns false when the layout does not fit
// the kernel (the SIMT kernel serves it then).
bool attn_units(hy_engine* h, int E, int T, int H, int G, bool any_ratio = false) {
  const int R = H / G;
  if (!any_ratio && (R > 64 || 64 % R)) return false;
  if (h->units_n > 0 && h->units_H == H && h->units_G == G) return true;
  int maxctx = 1;
  for (int e = 0; e < E; ++e) maxctx = std::max(maxctx, h->step_pos0[e] + h->step_start[e + 1] - h->step_start[e]);
  const int ns_cap = (int)std::max<size_t>(1, h->part_rows / ((size_t)T * H));
  int ns = std::min(std::min((maxctx + 255) / 256, ns_cap), 256);
  const int split = ((maxctx + ns - 1) / ns + 63) / 64 * 64;
  ns = (maxctx + split - 1) / split;
  if (h->units_n > 0) cudaStreamSynchronize(h->stream);        // another layout earlier in this step still reads the list
  size_t n = 0;
  for (int e = 0; e < E; ++e) {
    const int cnt = h->step_start[e + 1] - h->step_start[e], pos0 = h->step_pos0[e], rows = cnt * R;
    for (int g = 0; g < G; ++g)
      for (int row0 = (rows - 1) / 64 * 64; row0 >= 0; row0 -= 64) {          // late rows see the most keys: start them first
        const int last_pos = pos0 + std::min(row0 + 63, rows - 1) / R;
        for (int sp = 0; sp * split <= last_pos; ++sp) {
          if (n >= h->units_cap) return false;
          h->units_h[n++] = AttnUnit{e, g, row0, sp};
        }
      }
  }
  cudaMemcpyAsync(h->units_d, h->units_h, n * sizeof(AttnUnit), cudaMemcpyHostToDevice, h->stream);
  h->units_n = (int)n; h->units_H = H; h->units_G = G; h->units_split = split; h->units_ns = ns;
  return true;
}


// Work units of the tensor-core window attention: (entry, key head, tile of 64 rows), late tiles first (they see the most).
bool window_units(hy_engine* h, int E, int H, int G) {
  const int R = H / G;
  if (h->units_n > 0 && h->units_H == H && h->units_G == G && h->units_split == -1) return true;
  if (h->units_n > 0) cudaStreamSynchronize(h->stream);        // another layout earlier in this step still reads the list
  size_t n = 0;
  for (int e = 0; e < E; ++e) {
    const int rows = (h->step_start[e + 1] - h->step_start[e]) * R;
    for (int g = 0; g < G; ++g)
      for (int row0 = (rows - 1) / 64 * 64; row0 >= 0; row0 -= 64) {
        if (n >= h->units_cap) return false;
        h->units_h[n++] = AttnUnit{e, g, row0, 0};
      }
  }
  cudaMemcpyAsync(h->units_d, h->units_h, n * sizeof(AttnUnit), cudaMemcpyHostToDevice, h->stream);
  h->units_n = (int)n; h->units_H = H; h->units_G = G; h->units_split = -1; h->units_ns = 1;
  return true;
}

// Work units of the tensor-core biased attention: (entry, key head, tile of 64 rows, key split).  Steps of few rows whose
// requests see many key tiles (decoding) cut every unit's tile list into n splits so that the SMs have work; prompts run
// unsplit.  The number of splits depends on the step only, a row's result on it only within rounding.
bool biased_units(hy_engine* h, int E, int T, int H, int G, int window, int keep, int dp) {
  const int R = H / G;
  if (h->units_n > 0 && h->units_H == H && h->units_G == G && h->units_split == -2 - window) return true;
  if (h->units_n > 0) cudaStreamSynchronize(h->stream);        // another layout earlier in this step still reads the list
  int units0 = 0, max_tiles = 1;
  for (int e = 0; e < E; ++e) {
    const int cnt = h->step_start[e + 1] - h->step_start[e], last = h->step_pos0[e] + cnt - 1;
    units0 += G * ((cnt * R + 63) / 64);
    const int seen = window > 0 ? std::min(last + 1, window + keep) : last + 1;
    max_tiles = std::max(max_tiles, seen / 64 + 2);
  }
  int ns = 1;
  if (units0 * 2 <= 148 && max_tiles >= 4 && h->part_o) {
    ns = std::min(std::min(148 / units0, (max_tiles + 1) / 2), 64);
    ns = (int)std::min<size_t>((size_t)ns, h->part_rows / ((size_t)T * H));
    if ((size_t)dp > h->part_dim) ns = 1;
    ns = std::max(ns, 1);
  }
  size_t n = 0;
  for (int e = 0; e < E; ++e) {
    const int rows = (h->step_start[e + 1] - h->step_start[e]) * R;
    for (int g = 0; g < G; ++g)
      for (int row0 = (rows - 1) / 64 * 64; row0 >= 0; row0 -= 64)
        for (int sp = 0; sp < ns; ++sp) {
          if (n >= h->units_cap) return false;
          h->units_h[n++] = AttnUnit{e, g, row0, sp};
        }
  }
  cudaMemcpyAsync(h->units_d, h->units_h, n * sizeof(AttnUnit), cudaMemcpyHostToDevice, h->stream);
  h->units_n = (int)n; h->units_H = H; h->units_G = G; h->units_split = -2 - window; h->units_ns = ns;
  return true;
}

// One layer of a norm - sublayer - norm model:  x += ls1 * n1b(mixer(n1(x)));  x += ls2 * n2b(experts(n2(x))).
// The output norms are element-wise, so they run in the epilogue of the mixer's output projection and in the experts'
// combine kernel, on the fp32 accumulators, together with the layer scale and the residual sum.
template <typename AT>
int sandwich_layer(hy_engine* h, const Batch& b, size_t li) {
  typedef AT WT;
  const hy_layer_cfg& c = h->lc[li];
  const LayerW& L = h->lw[li];
  const int W = h->m.width, T = b.T, E = b.E;
  const float eps = h->m.norm_eps;
  cudaStream_t s = h->stream;
  AT* hb = (AT*)h->hbuf; AT* pin = (AT*)h->pin; AT* cat = (AT*)h->cat; AT* cv = (AT*)h->cv;
  // the input norms are element-wise: every sublayer's epilogue also writes the NEXT sublayer's normed input, so only the
  // first layer runs a norm kernel of its own
  const bool routed = c.ff_kind == HY_FF_ROUTED;
  const bool last = li + 1 == h->lc.size();
  const TanhNorm none{};
  const TanhNorm after_mixer = routed ? L.n2 : last ? none : h->lw[li + 1].n1;
  const TanhNorm after_ff = last ? none : h->lw[li + 1].n1;
  if (li == 0) {
    ProfScope ps(h, HY_PROF_NORM);
    tanh_norm_kernel<AT><<<T, 256, 0, s>>>(h->x, nullptr, L.n1, W, hb);
    h->launches++;
  }
  if (c.mixer == HY_MIX_SSD) {
    const int H = c.m_heads, P = c.m_vdim, N = c.m_state, G = c.m_groups, inner = H * P, GN = G * N, C = inner + 2 * GN;
    {
      ProfScope ps(h, HY_PROF_GEMM_IN);
      gemm<AT, WT, AT>(h, hb, W, (const WT*)L.w_in, W, T, L.n_in, W, to_buf(pin, h->ld_pin), L.w_in_t);
    }
    {
      ProfScope ps(h, HY_PROF_CONV);
      conv_kernel<AT, WT><<<dim3((C + 127) / 128, T), 128, 0, s>>>(b, pin, h->ld_pin, inner, C, c.m_conv, (const WT*)L.m_conv_w,
                                                                   (const WT*)L.m_conv_b, 1, L.conv_state, cv, h->ld_cv);
      conv_tail_kernel<AT><<<dim3((C + 127) / 128, E), 128, 0, s>>>(b, pin, h->ld_pin, inner, C, c.m_conv, L.conv_state);
      h->launches += 2;
    }
    {
      ProfScope ps(h, HY_PROF_SCAN);
      // 4 states per thread up to 16 states, 16 per thread beyond; lanes = the power of two that covers the state size
      const int nper = N <= 16 ? 4 : 16;
      int lanes = 1;
      while (lanes * nper < N) lanes <<= 1;
      const int per_block = 128 / lanes, bph = (P + per_block - 1) / per_block;
      dim3 grid(H * bph, E);
#define HY_SSD_ARGS b, cv, h->ld_cv, inner, inner + GN, pin + 2 * inner + 2 * GN, h->ld_pin, L.m_dt_bias, L.m_A_log, L.m_D, H, P, N, \
      G, bph, L.rec_state, h->f2, h->ld_f2
#define HY_SSD_CASE(NP, LL) if (nper == NP && lanes == LL) ssd_scan_kernel<AT, NP, LL><<<grid, 128, 0, s>>>(HY_SSD_ARGS)
      HY_SSD_CASE(4, 1); else HY_SSD_CASE(4, 2); else HY_SSD_CASE(4, 4);
      else HY_SSD_CASE(16, 2); else HY_SSD_CASE(16, 4); else HY_SSD_CASE(16, 8); else HY_SSD_CASE(16, 16); else HY_SSD_CASE(16, 32);
#undef HY_SSD_CASE
#undef HY_SSD_ARGS
      gated_group_norm_kernel<AT><<<dim3(T, c.m_norm_groups), 128, 0, s>>>(h->f2, h->ld_f2, pin, h->ld_pin, L.m_norm, inner,
                                                                          c.m_norm_groups, eps, cat, h->ld_cat);
      h->launches += 2;
    }
  } else if (c.mixer == HY_MIX_LATENT) {
    const int H = c.l_heads, R = c.l_kv_rank, rot = c.l_rot_dim, Dk = R + rot, dn = c.l_dim, dv = c.l_vdim;
    const int own = c.l_kv_from < 0 ? 1 : 0;
    {
      ProfScope ps(h, HY_PROF_GEMM_IN);
      gemm<AT, WT, float>(h, hb, W, (const WT*)L.w_in, W, T, L.n_in, W, to_buf(h->f1, h->ld_f1), L.w_in_t);
    }
    {
      ProfScope ps(h, HY_PROF_CONV);
      latent_prep_kernel<AT><<<T, 128, (size_t)(2 * L.rot.pairs + 2) * 4, s>>>(b, h->f1, h->ld_f1, c.l_q_rank, R, rot, own, L.l_qn,
                                                                               L.l_kn, eps, L.rot, cv, h->ld_cv, (AT*)L.cache);
      h->launches++;
    }
    {
      ProfScope ps(h, HY_PROF_SMALL_GEMM);
      gemm<AT, WT, AT>(h, cv, h->ld_cv, (const WT*)L.w_uq, c.l_q_rank, T, H * (dn + rot), c.l_q_rank, to_buf(pin, h->ld_pin), L.w_uq_t);
      const int fold = T > 8 ? 1 : 0;
      latent_query_kernel<AT, WT><<<dim3((T + HY_LAT_TB - 1) / HY_LAT_TB, H, fold ? (R + 127) / 128 : 1), 128,
                                    (size_t)(HY_LAT_TB * dn + 2 * L.rot.pairs + 2) * 4, s>>>(b, pin, h->ld_pin, (const WT*)L.w_uk, H, dn,
                                                                                             rot, R, fold, L.rot, cv, h->ld_cv);
      h->launches++;
      if (!fold) {
        head_rows_kernel<AT, WT, AT><<<(H * R + 7) / 8, 256, 0, s>>>(T, pin, h->ld_pin, dn + rot, (const WT*)L.w_ukT, H, R, dn, cv,
                                                                     h->ld_cv, Dk);
        h->launches++;
      }
    }
    {
      ProfScope ps(h, HY_PROF_ATTN);
      bool tc = false;
      if constexpr (std::is_same<AT, bf16>::value) {
        if ((Dk == 32 || Dk == 64 || Dk == 128) && h->part_o && attn_units(h, E, T, H, 1)) {
          tc = true;
#define HY_ATTN_ARGS b, h->units_d, cv, h->ld_cv, (const bf16*)L.cache, H, 1, c.l_scale, 0.0f, 1, h->units_split, h->units_ns, R, \
          h->part_o, h->part_ml
          if (Dk == 32) attn_mma_kernel<32><<<h->units_n, 128, 0, s>>>(HY_ATTN_ARGS);
          else if (Dk == 64) attn_mma_kernel<64><<<h->units_n, 128, 0, s>>>(HY_ATTN_ARGS);
          else attn_mma_kernel<128><<<h->units_n, 128, 0, s>>>(HY_ATTN_ARGS);
#undef HY_ATTN_ARGS
          attn_combine_kernel<WT, float><<<T * H, 64, 0, s>>>(b, h->part_o, h->part_ml, (const WT*)L.sink, nullptr, 0, H, Dk, R,
                                                              h->units_split, h->units_ns, 1.0f, h->f2, h->ld_f2);
          h->launches += 2;
        }
      }
      if constexpr (std::is_same<AT, bf16>::value) {
        // wide cache rows (or a head count the narrow kernel does not tile): eight warps per tile, values split by warp
        if (!tc && Dk % 8 == 0 && R <= 512 && h->part_o && attn_units(h, E, T, H, 1, true)) {
          tc = true;
          const int nt = R <= 128 ? 2 : R <= 256 ? 4 : 8, pstride = nt * 64;
          const size_t smem = attn_wide_smem(Dk);
          static bool wide_attr = false;
          if (!wide_attr) {
            cudaFuncSetAttribute(attn_wide_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_wide_smem(640));
            cudaFuncSetAttribute(attn_wide_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_wide_smem(640));
            cudaFuncSetAttribute(attn_wide_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_wide_smem(640));
            wide_attr = true;
          }
#define HY_WIDE_ARGS b, h->units_d, cv, h->ld_cv, (const bf16*)L.cache, H, Dk, R, c.l_scale, h->units_split, h->units_ns, pstride, \
          h->part_o, h->part_ml
          if (nt == 2) attn_wide_kernel<2><<<h->units_n, 256, smem, s>>>(HY_WIDE_ARGS);
          else if (nt == 4) attn_wide_kernel<4><<<h->units_n, 256, smem, s>>>(HY_WIDE_ARGS);
          else attn_wide_kernel<8><<<h->units_n, 256, smem, s>>>(HY_WIDE_ARGS);
#undef HY_WIDE_ARGS
          attn_combine_kernel<WT, float><<<T * H, 64, 0, s>>>(b, h->part_o, h->part_ml, (const WT*)L.sink, nullptr, 0, H, pstride, R,
                                                              h->units_split, h->units_ns, 1.0f, h->f2, h->ld_f2);
          h->launches += 2;
        }
      }
      if (!tc) {
        attn_sink_kernel<AT, WT, float><<<(T * H + 3) / 4, 128, 4 * Dk * sizeof(float), s>>>(
            b, cv, h->ld_cv, (const AT*)L.cache, (const WT*)L.sink, (const AT*)nullptr, 0, H, 1, Dk, R, c.l_scale, 0.0f, 1, 1.0f,
            h->f2, h->ld_f2);
        h->launches++;
      }
    }
    {
      ProfScope ps(h, HY_PROF_SMALL_GEMM);
      if (T <= 8)
        head_rows_kernel<float, WT, AT><<<(H * dv + 7) / 8, 256, 0, s>>>(T, h->f2, h->ld_f2, R, (const WT*)L.w_uv, H, dv, R, cat,
                                                                         h->ld_cat, dv);
      else
      latent_value_kernel<AT, WT><<<dim3((T + HY_LAT_TB - 1) / HY_LAT_TB, H, (dv + 127) / 128), 128, (size_t)HY_LAT_TB * R * 4, s>>>(
          T, h->f2, h->ld_f2, (const WT*)L.w_uvT, H, R, dv, cat, h->ld_cat);
      h->launches++;
    }
  } else {
    const int H = c.g_heads, dk = c.g_dim, dv = c.g_vdim;
    {
      ProfScope ps(h, HY_PROF_GEMM_IN);
      gemm<AT, WT, AT>(h, hb, W, (const WT*)L.w_in, W, T, L.n_in, W, to_buf(pin, h->ld_pin), L.w_in_t);
    }
    ProfScope ps(h, HY_PROF_DELTA);
    static bool glr_attr = false;
    if (!glr_attr) {
      cudaFuncSetAttribute(glr_reg_kernel<AT, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      cudaFuncSetAttribute(glr_reg_kernel<AT, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      cudaFuncSetAttribute(glr_reg_kernel<AT, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      cudaFuncSetAttribute(glr_kernel<AT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
      glr_attr = true;
    }
#define HY_GLR_ARGS b, pin, h->ld_pin, L.c_q, L.c_k, L.c_v, L.g_fb, L.g_lower, L.g_norm, H, dk, dv, eps, L.rec_state, cat, h->ld_cat
    const int nthr = std::max(((dv + 31) / 32) * 32, 32);
    auto gsm = [](int dr, int nt) { return (size_t)HY_GLR_TB * (2 * dr + 2 * nt) * 4; };
    if (dk <= 32 && nthr <= 512) glr_reg_kernel<AT, 32><<<dim3(H, E), nthr, gsm(32, nthr), s>>>(HY_GLR_ARGS);
    else if (dk <= 64 && nthr <= 512) glr_reg_kernel<AT, 64><<<dim3(H, E), nthr, gsm(64, nthr), s>>>(HY_GLR_ARGS);
    else if (dk <= 128 && nthr <= 256) glr_reg_kernel<AT, 128><<<dim3(H, E), nthr, gsm(128, nthr), s>>>(HY_GLR_ARGS);
    else glr_kernel<AT><<<dim3(H, E), 256, ((size_t)dk * dv + 2 * dk + dv + 40) * 4, s>>>(HY_GLR_ARGS);
#undef HY_GLR_ARGS
    h->launches++;
  }
  {
    ProfScope ps(h, HY_PROF_GEMM_OUT);
    GemmOut o{nullptr, 0, 0, nullptr, 0, 0, h->x, W, 1.0f, L.n1b.w, L.n1b.b, L.ls1, L.n1b.alpha,
              after_mixer.w, after_mixer.b, after_mixer.alpha, hb, std::is_same<AT, float>::value ? 1 : 0};
    gemm<AT, WT, float>(h, cat, h->ld_cat, (const WT*)L.w_out, L.k_out, T, W, L.k_out, o, L.w_out_t);
  }
  if (!routed) return HY_OK;
  const int NE = c.x_experts, top = c.x_top, ff = c.ff, P = T * top, ldh = (ff + 7) & ~7;
  const bool tc_experts = std::is_same<AT, bf16>::value && L.w_gu_t != nullptr;
  // a handful of pairs: one block row per pair; beyond that the sorted order, where pairs that share an expert share its
  // stream (measured at 8 tokens x 4 experts of 32: the tensor-core product over the sorted order is 2.5 - 5 times faster)
  static const int rows_max_env = getenv("HY_EXPERT_ROWS_MAX") ? atoi(getenv("HY_EXPERT_ROWS_MAX")) : -1;   // developer switch
  const bool few = P <= (rows_max_env >= 0 ? rows_max_env : tc_experts ? 8 : 16);
  {
    ProfScope ps(h, HY_PROF_ROUTE);
    gemm<AT, WT, float>(h, hb, W, (const WT*)L.w_router, W, T, NE, W, to_buf(h->f1, h->ld_f1), L.w_router_t);
    const RouteCfg rc{NE, top, c.x_groups, c.x_keep, c.x_scale};
    route_kernel<<<T, 32, (size_t)(NE + c.x_groups) * 4, s>>>(h->f1, h->ld_f1, rc, h->x_ids, h->x_wts, few ? nullptr : h->x_counts);
    h->launches++;
    if (!few) {
      route_offsets_kernel<<<1, 32, 0, s>>>(h->x_counts, NE, tc_experts ? 128 : HY_XT, h->x_offs, h->x_fill, h->x_tile_e,
                                            h->x_tile_r0, h->x_meta);
      route_scatter_kernel<<<(P + 255) / 256, 256, 0, s>>>(P, top, h->x_ids, h->x_offs, h->x_fill, h->x_row_tok, h->x_pair_row);
      h->launches += 2;
    }
  }
  {
    ProfScope ps(h, HY_PROF_EXPERTS);
    float* ys = h->f2;                                        // [pairs, width] fp32
    if (few) {
      static bool rows_attr = false;
      if (!rows_attr) {
        cudaFuncSetAttribute(expert_rows_kernel<AT, WT, AT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(expert_rows_kernel<AT, WT, float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        rows_attr = true;
      }
      expert_rows_kernel<AT, WT, AT, true><<<dim3(std::min((ff + 7) / 8, 256), P), 256, (size_t)W * sizeof(AT), s>>>(
          hb, W, h->x_ids, top, 1, (const WT*)L.w_gu, (size_t)2 * ff * W, ff, W, pin, ldh, 0);
      expert_rows_kernel<AT, WT, float, false><<<dim3(std::min((W + 7) / 8, 256), P), 256, (size_t)ff * sizeof(AT), s>>>(
          pin, ldh, h->x_ids, top, 0, (const WT*)L.w_down, (size_t)W * ff, W, ff, ys, W, -1);
    } else if (tc_experts) {
      if constexpr (std::is_same<AT, bf16>::value) {
        static bool attr_set = false;
        if (!attr_set) {
          cudaFuncSetAttribute(gemm_tc_kernel<bf16, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes(128));
          cudaFuncSetAttribute(gemm_tc_kernel<float, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes(128));
          attr_set = true;
        }
        const int tiles = std::min(h->x_max_tiles, P / 128 + NE + 1);
        const TcGroup g1{h->x_meta, h->x_offs, h->x_tile_e, h->x_tile_r0, h->x_row_tok, L.gu_t_stride};
        const TcGroup g2{h->x_meta, h->x_offs, h->x_tile_e, h->x_tile_r0, nullptr, L.down_t_stride};
        GemmOut o1{pin, ldh, ff, nullptr, 0, 2, nullptr, 0, 1.0f};
        gemm_tc_kernel<bf16, 128><<<dim3((L.gu_rows + 127) / 128, tiles), 192, tc_smem_bytes(128), s>>>(
            hb, W, (const bf16*)L.w_gu_t, P, L.gu_rows, W, o1, h->err_d, g1);
        GemmOut o2 = to_buf(ys, W);
        gemm_tc_kernel<float, 128><<<dim3((W + 127) / 128, tiles), 192, tc_smem_bytes(128), s>>>(
            pin, ldh, (const bf16*)L.w_down_t, P, W, ff, o2, h->err_d, g2);
      }
    } else {
      const int tiles = std::min(h->x_max_tiles, P / HY_XT + NE + 1);
      expert_gemm_simt_kernel<AT, WT, AT, true><<<dim3((ff + 63) / 64, tiles), 256, 0, s>>>(
          hb, W, h->x_row_tok, (const WT*)L.w_gu, (size_t)2 * ff * W, ff, W, h->x_offs, h->x_tile_e, h->x_tile_r0, h->x_meta, pin, ldh, 0);
      expert_gemm_simt_kernel<AT, WT, float, false><<<dim3((W + 63) / 64, tiles), 256, 0, s>>>(
          pin, ldh, nullptr, (const WT*)L.w_down, (size_t)W * ff, W, ff, h->x_offs, h->x_tile_e, h->x_tile_r0, h->x_meta, ys, W, -1);
    }
    expert_combine_kernel<AT><<<T, 256, 0, s>>>(ys, W, few ? nullptr : h->x_pair_row, h->x_wts, top, W, L.n2b, L.ls2, h->x, after_ff, hb);
    h->launches += 3;
  }
  return HY_OK;
}

// x <- x + ls * rms(y) * w for a sublayer's output y [T, ldy] (or the mixture of expert rows), and hb <- x in the
// activation type for the next sublayer.
template <typename AT>
void post_norm_add(hy_engine* h, int T, const float* y, int ldy, const float* rows, const int* pair_row, const float* wts, int top,
                   const float* shared_rows, const float* w, const float* ls, int add) {
  const int W = h->m.width;
  static bool attr = false;                                  // per AT: this function is a template
  if (!attr) { cudaFuncSetAttribute(post_norm_add_kernel<AT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); attr = true; }
  post_norm_add_kernel<AT><<<T, 256, (size_t)W * 4, h->stream>>>(y, ldy, rows, W, pair_row, wts, top, shared_rows, w, ls, h->m.norm_eps,
                                                               W, add, h->x, (AT*)h->hbuf);
  h->launches++;
}

// One layer of a model whose sublayers read the stream itself:  x += ls1 * rms(mixer(x)) * w1;  x += ls2 * rms(ff(x)) * w2.
// The norm needs the whole row's mean square, so it cannot ride in the epilogue of the product that makes the row's
// tiles: the output projections leave fp32 rows, and one kernel per sublayer norms, scales, adds and writes the updated
// stream in both types.
template <typename AT>
int postnorm_layer(hy_engine* h, const Batch& b, size_t li) {
  typedef AT WT;
  const hy_layer_cfg& c = h->lc[li];
  const LayerW& L = h->lw[li];
  const int W = h->m.width, T = b.T, E = b.E;
  const float eps = h->m.norm_eps;
  cudaStream_t s = h->stream;
  AT* hb = (AT*)h->hbuf; AT* pin = (AT*)h->pin; AT* cat = (AT*)h->cat; AT* cv = (AT*)h->cv;
  if (c.mixer == HY_MIX_WINDOW) {
    const WindowCfg wc{c.w_heads, c.w_kv_heads, c.w_dim, c.w_vdim, c.w_window, c.w_pool, c.w_rot_dims, c.w_rot_values, c.w_qk_norm, c.w_scale};
    {
      ProfScope ps(h, HY_PROF_GEMM_IN);
      gemm<AT, WT, AT>(h, hb, W, (const WT*)L.w_in, W, T, L.n_in, W, to_buf(pin, h->ld_pin), L.w_in_t);
    }
    {
      ProfScope ps(h, HY_PROF_CONV);
      window_prep_kernel<AT><<<T, 128, (size_t)(2 * L.rot.pairs + 2 * L.rot_v.pairs + 2) * 4, s>>>(
          b, pin, h->ld_pin, L.c_q, L.c_k, L.c_v, wc, L.w_qn, L.w_kn, eps, L.rot, L.rot_v, cv, h->ld_cv, (AT*)L.cache, (AT*)L.cache_v,
          h->f1, h->ld_f1);
      int most = 0;                                           // blocks one entry completes in this step
      for (int e = 0; e < E; ++e) {
        const int p0 = h->step_pos0[e], end = p0 + h->step_start[e + 1] - h->step_start[e];
        most = std::max(most, end / c.w_pool - p0 / c.w_pool);
      }
      h->launches++;
      if (most > 0) {
        window_pool_kernel<AT><<<dim3(most, E), 128, 0, s>>>(b, wc, (const AT*)L.cache, (const AT*)L.cache_v, (AT*)L.pool_k, (AT*)L.pool_v);
        h->launches++;
      }
    }
    {
      ProfScope ps(h, HY_PROF_ATTN);
      bool tc = false;
      if constexpr (std::is_same<AT, bf16>::value) {
        // head sizes that are multiples of 8 up to 128: tensor-core tiles of 64 rows x 64 keys
        if (c.w_dim % 8 == 0 && c.w_vdim % 8 == 0 && c.w_dim <= 128 && c.w_vdim <= 128 && h->units_d &&
            window_units(h, E, c.w_heads, c.w_kv_heads)) {
          tc = true;
#define HY_WIN_ARGS b, h->units_d, cv, h->ld_cv, wc, (const bf16*)L.cache, (const bf16*)L.cache_v, (const bf16*)L.pool_k, \
          (const bf16*)L.pool_v, h->f1, h->ld_f1, cat, h->ld_cat
          static bool win_attr = false;
          if (!win_attr) {
            cudaFuncSetAttribute(window_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)window_mma_smem(64));
            cudaFuncSetAttribute(window_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)window_mma_smem(128));
            win_attr = true;
          }
          if (c.w_dim <= 64 && c.w_vdim <= 64) window_mma_kernel<64><<<h->units_n, 128, window_mma_smem(64), s>>>(HY_WIN_ARGS);
          else window_mma_kernel<128><<<h->units_n, 128, window_mma_smem(128), s>>>(HY_WIN_ARGS);
#undef HY_WIN_ARGS
        }
      }
      if (!tc)
        window_attn_kernel<AT, AT><<<(T * c.w_heads + 3) / 4, 128, 4 * c.w_dim * sizeof(float), s>>>(
            b, cv, h->ld_cv, wc, (const AT*)L.cache, (const AT*)L.cache_v, (const AT*)L.pool_k, (const AT*)L.pool_v, h->f1, h->ld_f1,
            cat, h->ld_cat);
      h->launches++;
    }
  } else {
    const int H = c.t_heads, dk = c.t_dim, dv = c.t_vdim;
    {
      ProfScope ps(h, HY_PROF_GEMM_IN);
      GemmOut o{pin, h->ld_pin, L.c_i, h->f1, h->ld_f1, 0, nullptr, 0, 1.0f};
      o.out2_f32 = 1;                                         // the gates' pre-activations stay fp32
      gemm<AT, WT, AT>(h, hb, W, (const WT*)L.w_in, W, T, L.n_in, W, o, L.w_in_t);
    }
    ProfScope ps(h, HY_PROF_DELTA);
    static bool attr = false;
    if (!attr) {
      cudaFuncSetAttribute(mlstm_reg_kernel<AT, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
      cudaFuncSetAttribute(mlstm_reg_kernel<AT, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
      cudaFuncSetAttribute(mlstm_reg_kernel<AT, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
      cudaFuncSetAttribute(mlstm_kernel<AT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
      attr = true;
    }
#define HY_MLSTM_GEN_ARGS b, pin, h->ld_pin, L.c_q, L.c_k, L.c_v, L.c_g, h->f1, h->ld_f1, 0, H, L.t_ib, L.t_fb, L.t_norm, H, dk, dv, \
    c.t_gate_cap, eps, L.rec_state, cat, h->ld_cat
#define HY_MLSTM_ARGS b, pin, h->ld_pin, L.c_q, L.c_k, L.c_v, L.c_g, h->f1, h->ld_f1, 0, H, L.t_ib, L.t_fb, L.t_norm, H, dk, dv, \
    c.t_gate_cap, eps, async_ok, L.rec_state, cat, h->ld_cat
    const int nthr = ((dv + 1 + 31) / 32) * 32;               // one thread per value column and one for the normaliser
    // rows of q, k, v, g that start and end on 16-byte boundaries may travel by asynchronous copies
    const int ch = 16 / (int)sizeof(AT);
    const int async_ok = (dk % ch == 0 && dv % ch == 0 && h->ld_pin % ch == 0 && L.c_k % ch == 0 && L.c_v % ch == 0 && L.c_g % ch == 0) ? 1 : 0;
    auto msm = [](int dr, int nt) {
      const size_t tb = (size_t)mlstm_tb(dr);
      return (tb * (2 * dr + 3 * nt) + 9 * tb + 4) * 4 + 2 * tb * (2 * dr + 2 * nt) * sizeof(AT);
    };
    if (dk <= 32 && nthr <= 256 && msm(32, nthr) <= 220 * 1024) mlstm_reg_kernel<AT, 32><<<dim3(H, E), nthr, msm(32, nthr), s>>>(HY_MLSTM_ARGS);
    else if (dk <= 64 && nthr <= 256 && msm(64, nthr) <= 220 * 1024) mlstm_reg_kernel<AT, 64><<<dim3(H, E), nthr, msm(64, nthr), s>>>(HY_MLSTM_ARGS);
    else if (dk <= 128 && nthr <= 256 && msm(128, nthr) <= 220 * 1024) mlstm_reg_kernel<AT, 128><<<dim3(H, E), nthr, msm(128, nthr), s>>>(HY_MLSTM_ARGS);
    else mlstm_kernel<AT><<<dim3(H, E), 256, ((size_t)dk * (dv + 1) + 2 * dk + dv + 1 + 40) * 4, s>>>(HY_MLSTM_GEN_ARGS);
#undef HY_MLSTM_ARGS
#undef HY_MLSTM_GEN_ARGS
    h->launches++;
  }
  {
    ProfScope ps(h, HY_PROF_GEMM_OUT);
    gemm<AT, WT, float>(h, cat, h->ld_cat, (const WT*)L.w_out, L.k_out, T, W, L.k_out, to_buf(h->f2, h->ld_f2), L.w_out_t);
  }
  {
    ProfScope ps(h, HY_PROF_NORM);
    post_norm_add<AT>(h, T, h->f2, h->ld_f2, nullptr, nullptr, nullptr, 0, nullptr, L.pn1, L.ls1, 1);
  }
  if (c.ff_kind == HY_FF_NONE) return HY_OK;
  if (c.ff_kind == HY_FF_GATED) {
    const int ff = c.ff;
    {
      ProfScope ps(h, HY_PROF_GEMM_IN);
      bool fused = false;
      if constexpr (std::is_same<AT, bf16>::value) {
        // more rows than the few-row kernel takes: the tensor-core product over gate / up rows that alternate in blocks of
        // 16, the gated activation in its epilogue
        if (T > 8 && L.w_ff_in_t && W % 8 == 0) {
          GemmOut o{cat, h->ld_cat, ff, nullptr, 0, 2, nullptr, 0, 1.0f};
          o.act_kind = c.ff_act;
          gemm<AT, WT, AT>(h, hb, W, (const WT*)nullptr, W, T, L.ff_rows, W, o, L.w_ff_in_t);
          fused = true;
        }
      }
      if (!fused) {
        gemm<AT, WT, AT>(h, hb, W, (const WT*)L.w_ff_in, W, T, 2 * ff, W, to_buf(pin, h->ld_pin));
        gated_act_kernel<AT><<<dim3((ff + 255) / 256, T), 256, 0, s>>>(pin, h->ld_pin, ff, c.ff_act, c.ff_limit, cat, h->ld_cat);
        h->launches++;
      }
    }
    {
      ProfScope ps(h, HY_PROF_GEMM_OUT);
      gemm<AT, WT, float>(h, cat, h->ld_cat, (const WT*)L.w_ff_down, ff, T, W, ff, to_buf(h->f2, h->ld_f2), L.w_ff_down_t);
    }
    ProfScope ps(h, HY_PROF_NORM);
    post_norm_add<AT>(h, T, h->f2, h->ld_f2, nullptr, nullptr, nullptr, 0, nullptr, L.pn2, L.ls2, 1);
    return HY_OK;
  }
  // routed plain experts: down(act(up x)), beside a shared expert of the same form
  const int NE = c.x_experts, top = c.x_top, ff = c.ff, P = T * top, ldh = (ff + 7) & ~7;
  const bool tc_experts = std::is_same<AT, bf16>::value && L.w_gu_t != nullptr;
  static const int rows_max_env = getenv("HY_EXPERT_ROWS_MAX") ? atoi(getenv("HY_EXPERT_ROWS_MAX")) : -1;   // developer switch
  const bool few = P <= (rows_max_env >= 0 ? rows_max_env : tc_experts ? 8 : 16);
  {
    ProfScope ps(h, HY_PROF_ROUTE);
    gemm<AT, WT, float>(h, hb, W, (const WT*)L.w_router, W, T, NE, W, to_buf(h->f1, h->ld_f1), L.w_router_t);
    if (c.x_route == HY_ROUTE_TOP_SOFTMAX) {
      route_top_kernel<<<T, 32, (size_t)NE * 4, s>>>(h->f1, h->ld_f1, L.x_rb, NE, top, h->x_ids, h->x_wts, few ? nullptr : h->x_counts);
    } else {
      const RouteCfg rc{NE, top, c.x_groups, c.x_keep, c.x_scale};
      route_kernel<<<T, 32, (size_t)(NE + c.x_groups) * 4, s>>>(h->f1, h->ld_f1, rc, h->x_ids, h->x_wts, few ? nullptr : h->x_counts);
    }
    h->launches++;
    if (!few) {
      route_offsets_kernel<<<1, 32, 0, s>>>(h->x_counts, NE, tc_experts ? 128 : HY_XT, h->x_offs, h->x_fill, h->x_tile_e,
                                            h->x_tile_r0, h->x_meta);
      route_scatter_kernel<<<(P + 255) / 256, 256, 0, s>>>(P, top, h->x_ids, h->x_offs, h->x_fill, h->x_row_tok, h->x_pair_row);
      h->launches += 2;
    }
  }
  float* ys = h->f2;                                          // [pairs (+ tokens: the shared expert's rows), width] fp32
  float* shared_rows = nullptr;
  {
    ProfScope ps(h, HY_PROF_EXPERTS);
    if (few) {
      static bool rows_attr = false;
      if (!rows_attr) {
        cudaFuncSetAttribute(expert_rows_kernel<AT, WT, AT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(expert_rows_kernel<AT, WT, float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        rows_attr = true;
      }
      expert_rows_kernel<AT, WT, AT, false><<<dim3(std::min((ff + 7) / 8, 256), P), 256, (size_t)W * sizeof(AT), s>>>(
          hb, W, h->x_ids, top, 1, (const WT*)L.w_gu, (size_t)ff * W, ff, W, pin, ldh, c.x_act);
      expert_rows_kernel<AT, WT, float, false><<<dim3(std::min((W + 7) / 8, 256), P), 256, (size_t)ff * sizeof(AT), s>>>(
          pin, ldh, h->x_ids, top, 0, (const WT*)L.w_down, (size_t)W * ff, W, ff, ys, W, -1);
    } else if (tc_experts) {
      if constexpr (std::is_same<AT, bf16>::value) {
        static bool attr_set = false;
        if (!attr_set) {
          cudaFuncSetAttribute(gemm_tc_kernel<bf16, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes(128));
          cudaFuncSetAttribute(gemm_tc_kernel<float, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes(128));
          attr_set = true;
        }
        const int tiles = std::min(h->x_max_tiles, P / 128 + NE + 1);
        const TcGroup g1{h->x_meta, h->x_offs, h->x_tile_e, h->x_tile_r0, h->x_row_tok, L.gu_t_stride};
        const TcGroup g2{h->x_meta, h->x_offs, h->x_tile_e, h->x_tile_r0, nullptr, L.down_t_stride};
        GemmOut o1 = to_buf(pin, ldh);
        o1.act2 = 3; o1.act_kind = c.x_act;
        gemm_tc_kernel<bf16, 128><<<dim3((ff + 127) / 128, tiles), 192, tc_smem_bytes(128), s>>>(
            hb, W, (const bf16*)L.w_gu_t, P, ff, W, o1, h->err_d, g1);
        GemmOut o2 = to_buf(ys, W);
        gemm_tc_kernel<float, 128><<<dim3((W + 127) / 128, tiles), 192, tc_smem_bytes(128), s>>>(
            pin, ldh, (const bf16*)L.w_down_t, P, W, ff, o2, h->err_d, g2);
      }
    } else {
      const int tiles = std::min(h->x_max_tiles, P / HY_XT + NE + 1);
      expert_gemm_simt_kernel<AT, WT, AT, false><<<dim3((ff + 63) / 64, tiles), 256, 0, s>>>(
          hb, W, h->x_row_tok, (const WT*)L.w_gu, (size_t)ff * W, ff, W, h->x_offs, h->x_tile_e, h->x_tile_r0, h->x_meta, pin, ldh, c.x_act);
      expert_gemm_simt_kernel<AT, WT, float, false><<<dim3((W + 63) / 64, tiles), 256, 0, s>>>(
          pin, ldh, nullptr, (const WT*)L.w_down, (size_t)W * ff, W, ff, h->x_offs, h->x_tile_e, h->x_tile_r0, h->x_meta, ys, W, -1);
    }
    h->launches += 2;
    if (c.x_shared_ff > 0) {
      const int sf = c.x_shared_ff;
      shared_rows = ys + (size_t)P * W;
      GemmOut o = to_buf(cat, h->ld_cat);
      o.act2 = 3; o.act_kind = c.x_act;
      gemm<AT, WT, AT>(h, hb, W, (const WT*)L.w_sh_up, W, T, sf, W, o, L.w_sh_up_t);
      gemm<AT, WT, float>(h, cat, h->ld_cat, (const WT*)L.w_sh_down, sf, T, W, sf, to_buf(shared_rows, W), L.w_sh_down_t);
    }
  }
  ProfScope ps(h, HY_PROF_NORM);
  post_norm_add<AT>(h, T, nullptr, 0, ys, few ? nullptr : h->x_pair_row, h->x_wts, top, shared_rows, L.pn2, L.ls2, 1);
  return HY_OK;
}

// Routed gated experts over the rows of hb [T, width]: router logits (fp32), the choice by the largest logits with a softmax
// over the chosen, both products grouped by expert.  Leaves one fp32 row per (token, choice) pair in h->f2 [pairs, width];
// returns whether the rows are in pair order (few pairs) or in the expert-sorted order (h->x_pair_row maps pairs to rows).
template <typename AT>
bool routed_gated_experts(hy_engine* h, int T, const AT* hb, const LayerW& L, const hy_layer_cfg& c) {
  typedef AT WT;
  const int W = h->m.width;
  cudaStream_t s = h->stream;
  AT* pin = (AT*)h->pin;
  const int NE = c.x_experts, top = c.x_top, ff = c.ff, P = T * top, ldh = (ff + 7) & ~7;
  const bool tc_experts = std::is_same<AT, bf16>::value && L.w_gu_t != nullptr;
  const bool few = P <= (tc_experts ? 8 : 16);
  {
    ProfScope ps(h, HY_PROF_ROUTE);
    gemm<AT, WT, float>(h, hb, W, (const WT*)L.w_router, W, T, NE, W, to_buf(h->f1, h->ld_f1), L.w_router_t);
    route_top_kernel<<<T, 32, (size_t)NE * 4, s>>>(h->f1, h->ld_f1, nullptr, NE, top, h->x_ids, h->x_wts, few ? nullptr : h->x_counts);
    h->launches++;
    if (!few) {
      route_offsets_kernel<<<1, 32, 0, s>>>(h->x_counts, NE, tc_experts ? 128 : HY_XT, h->x_offs, h->x_fill, h->x_tile_e,
                                            h->x_tile_r0, h->x_meta);
      route_scatter_kernel<<<(P + 255) / 256, 256, 0, s>>>(P, top, h->x_ids, h->x_offs, h->x_fill, h->x_row_tok, h->x_pair_row);
      h->launches += 2;
    }
  }
  ProfScope ps(h, HY_PROF_EXPERTS);
  float* ys = h->f2;
  if (few) {
    static bool rows_attr = false;
    if (!rows_attr) {
      cudaFuncSetAttribute(expert_rows_kernel<AT, WT, AT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      cudaFuncSetAttribute(expert_rows_kernel<AT, WT, float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      rows_attr = true;
    }
    expert_rows_kernel<AT, WT, AT, true><<<dim3(std::min((ff + 7) / 8, 256), P), 256, (size_t)W * sizeof(AT), s>>>(
        hb, W, h->x_ids, top, 1, (const WT*)L.w_gu, (size_t)2 * ff * W, ff, W, pin, ldh, c.x_act);
    expert_rows_kernel<AT, WT, float, false><<<dim3(std::min((W + 7) / 8, 256), P), 256, (size_t)ff * sizeof(AT), s>>>(
        pin, ldh, h->x_ids, top, 0, (const WT*)L.w_down, (size_t)W * ff, W, ff, ys, W, -1);
  } else if (tc_experts) {
    if constexpr (std::is_same<AT, bf16>::value) {
      static bool attr_set = false;
      if (!attr_set) {
        cudaFuncSetAttribute(gemm_tc_kernel<bf16, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes(128));
        cudaFuncSetAttribute(gemm_tc_kernel<float, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes(128));
        attr_set = true;
      }
      const int tiles = std::min(h->x_max_tiles, P / 128 + NE + 1);
      const TcGroup g1{h->x_meta, h->x_offs, h->x_tile_e, h->x_tile_r0, h->x_row_tok, L.gu_t_stride};
      const TcGroup g2{h->x_meta, h->x_offs, h->x_tile_e, h->x_tile_r0, nullptr, L.down_t_stride};
      GemmOut o1{pin, ldh, ff, nullptr, 0, 2, nullptr, 0, 1.0f};
      o1.act_kind = c.x_act;
      gemm_tc_kernel<bf16, 128><<<dim3((L.gu_rows + 127) / 128, tiles), 192, tc_smem_bytes(128), s>>>(
          hb, W, (const bf16*)L.w_gu_t, P, L.gu_rows, W, o1, h->err_d, g1);
      GemmOut o2 = to_buf(ys, W);
      gemm_tc_kernel<float, 128><<<dim3((W + 127) / 128, tiles), 192, tc_smem_bytes(128), s>>>(
          pin, ldh, (const bf16*)L.w_down_t, P, W, ff, o2, h->err_d, g2);
    }
  } else {
    const int tiles = std::min(h->x_max_tiles, P / HY_XT + NE + 1);
    expert_gemm_simt_kernel<AT, WT, AT, true><<<dim3((ff + 63) / 64, tiles), 256, 0, s>>>(
        hb, W, h->x_row_tok, (const WT*)L.w_gu, (size_t)2 * ff * W, ff, W, h->x_offs, h->x_tile_e, h->x_tile_r0, h->x_meta, pin, ldh, c.x_act);
    expert_gemm_simt_kernel<AT, WT, float, false><<<dim3((W + 63) / 64, tiles), 256, 0, s>>>(
        pin, ldh, nullptr, (const WT*)L.w_down, (size_t)W * ff, W, ff, h->x_offs, h->x_tile_e, h->x_tile_r0, h->x_meta, ys, W, -1);
  }
  h->launches += 2;
  return few;
}

template <typename WT>
void stream_row(hy_engine* h, const Batch& b, const StreamOp& o) {
  const int W = h->m.width;
  static bool attr = false;                                  // per WT: this function is a template
  if (!attr) { cudaFuncSetAttribute(stream_row_kernel<WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); attr = true; }
  stream_row_kernel<WT><<<b.T, 256, ((size_t)2 * W + (size_t)std::max(o.side_dim, 0)) * 4, h->stream>>>(b, o, W, h->x);
  h->launches++;
}

// the normed rows in h->hn through a sublayer's input convolution into the operand buffer; then the new tail
template <typename AT>
void canon_input(hy_engine* h, const Batch& b, const float* w, float* tails) {
  const int W = h->m.width, taps = h->m.canon_taps;
  if (W % 4 == 0) canon_kernel<AT, 4><<<dim3((W / 4 + 127) / 128, b.T), 128, 0, h->stream>>>(b, h->hn, W, taps, w, tails, (AT*)h->hbuf);
  else canon_kernel<AT, 1><<<dim3((W + 127) / 128, b.T), 128, 0, h->stream>>>(b, h->hn, W, taps, w, tails, (AT*)h->hbuf);
  h->launches++;
  if (taps > 1) {
    conv_tail_kernel<float><<<dim3((W + 127) / 128, b.E), 128, 0, h->stream>>>(b, h->hn, W, 0, W, taps, tails);
    h->launches++;
  }
}

// One layer of a pre-norm model.  On entry h->hn holds the layer's first normed rows (norm1 of the stream); on exit the
// next layer's.  x += m ls1 attention(c1(n1 x));  x += m ls2 ff(c2(n2 x));  token input;  depth average.
template <typename AT>
int prenorm_layer(hy_engine* h, const Batch& b, size_t li) {
  typedef AT WT;
  const hy_layer_cfg& c = h->lc[li];
  const LayerW& L = h->lw[li];
  const int W = h->m.width, T = b.T, E = b.E;
  const float eps = h->m.norm_eps, mult = h->m.resid_mult;
  cudaStream_t s = h->stream;
  AT* hb = (AT*)h->hbuf; AT* pin = (AT*)h->pin; AT* cat = (AT*)h->cat;
  const bool last = li + 1 == h->lc.size();
  {
    ProfScope ps(h, HY_PROF_CONV);
    canon_input<AT>(h, b, L.canon1, L.conv_state);
  }
  {
    ProfScope ps(h, HY_PROF_GEMM_IN);
    GemmOut o = to_buf(pin, h->ld_pin);
    o.bias = L.b_bias;
    gemm<AT, WT, AT>(h, hb, W, (const WT*)L.w_in, W, T, L.n_in, W, o, L.w_in_t);
  }
  const BiasedCfg bc{c.b_heads, c.b_kv_heads, c.b_dim, c.b_vdim, c.b_window, c.b_keep_first, c.b_scale, c.b_softcap, L.b_r1, L.b_r2, L.b_sink};
  {
    ProfScope ps(h, HY_PROF_CONV);
    biased_prep_kernel<AT><<<T, 128, 0, s>>>(b, pin, h->ld_pin, L.c_k, L.c_v, c.b_kv_heads, c.b_dim, c.b_vdim, L.b_mix, L.b_lambda,
                                             (AT*)h->vfirst, h->ld_vf, (AT*)L.cache, (AT*)L.cache_v);
    h->launches++;
  }
  {
    ProfScope ps(h, HY_PROF_ATTN);
    bool tc = false;
    if constexpr (std::is_same<AT, bf16>::value) {
      static const bool simt_only = getenv("HY_BIASED_SIMT") != nullptr;      // developer switch
      if (!simt_only && c.b_dim % 8 == 0 && c.b_vdim % 8 == 0 && c.b_dim <= 128 && c.b_vdim <= 128 && h->ld_pin % 8 == 0 && h->units_d &&
          biased_units(h, E, T, c.b_heads, c.b_kv_heads, c.b_window, c.b_keep_first, (c.b_dim <= 64 && c.b_vdim <= 64) ? 64 : 128)) {
        tc = true;
        static bool attr = false;
        if (!attr) {
          cudaFuncSetAttribute(biased_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)window_mma_smem(64));
          cudaFuncSetAttribute(biased_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)window_mma_smem(128));
          attr = true;
        }
        if (c.b_dim <= 64 && c.b_vdim <= 64)
          biased_mma_kernel<64><<<h->units_n, 128, window_mma_smem(64), s>>>(b, h->units_d, pin + L.c_q, h->ld_pin, bc, (const bf16*)L.cache,
                                                                            (const bf16*)L.cache_v, cat, h->ld_cat, h->units_ns, h->part_o, h->part_ml);
        else
          biased_mma_kernel<128><<<h->units_n, 128, window_mma_smem(128), s>>>(b, h->units_d, pin + L.c_q, h->ld_pin, bc, (const bf16*)L.cache,
                                                                              (const bf16*)L.cache_v, cat, h->ld_cat, h->units_ns, h->part_o, h->part_ml);
        if (h->units_ns > 1) {
          biased_combine_kernel<bf16><<<T * c.b_heads, 64, 0, s>>>(h->part_o, h->part_ml, L.b_sink, c.b_heads, c.b_vdim,
                                                                   (c.b_dim <= 64 && c.b_vdim <= 64) ? 64 : 128, h->units_ns, cat, h->ld_cat);
          h->launches++;
        }
      }
    }
    if (!tc)
      biased_attn_kernel<AT, AT><<<(T * c.b_heads + 3) / 4, 128, 4 * c.b_dim * sizeof(float), s>>>(
          b, pin + L.c_q, h->ld_pin, bc, (const AT*)L.cache, (const AT*)L.cache_v, cat, h->ld_cat);
    h->launches++;
  }
  {
    ProfScope ps(h, HY_PROF_GEMM_OUT);
    gemm<AT, WT, float>(h, cat, h->ld_cat, (const WT*)L.w_out, L.k_out, T, W, L.k_out, to_buf(h->f2, h->ld_f2), L.w_out_t);
  }
  // what closes the layer: the token input, the depth average and the next layer's first norm
  StreamOp tail{};
  tail.mult = mult; tail.eps = eps;
  if (h->m.side_dim > 0) {
    tail.side_gate = L.side_gate; tail.side_proj = L.side_proj; tail.side_norm = L.side_norm; tail.side_table = h->side_table;
    tail.side_ld = h->m.side_dim * h->m.n_layers; tail.side_col0 = (int)li * h->m.side_dim; tail.side_dim = h->m.side_dim;
  }
  if (h->m.depth_avg) { tail.kept = h->kept; tail.kept_stride = (size_t)h->rt.max_step_tokens * W; tail.kept_n = (int)li + 1; tail.dwa = L.dwa; }
  if (!last) { tail.next_w = h->lw[li + 1].pn1; tail.next_out = h->hn; }
  if (c.ff_kind == HY_FF_NONE) {
    ProfScope ps(h, HY_PROF_NORM);
    tail.y = h->f2; tail.ldy = h->ld_f2; tail.ls = L.ls1;
    stream_row<WT>(h, b, tail);
    return HY_OK;
  }
  {
    ProfScope ps(h, HY_PROF_NORM);
    StreamOp o{};
    o.y = h->f2; o.ldy = h->ld_f2; o.ls = L.ls1; o.mult = mult; o.eps = eps; o.next_w = L.pn2; o.next_out = h->hn;
    stream_row<WT>(h, b, o);
  }
  {
    ProfScope ps(h, HY_PROF_CONV);
    canon_input<AT>(h, b, L.canon2, L.conv_state2);
  }
  tail.ls = L.ls2;
  if (c.ff_kind == HY_FF_GATED) {
    const int ff = c.ff;
    {
      ProfScope ps(h, HY_PROF_GEMM_IN);
      bool fused = false;
      if constexpr (std::is_same<AT, bf16>::value) {
        if (T > 8 && L.w_ff_in_t && W % 8 == 0) {
          GemmOut o{cat, h->ld_cat, ff, nullptr, 0, 2, nullptr, 0, 1.0f};
          o.act_kind = c.ff_act; o.act_limit = c.ff_limit;
          gemm<AT, WT, AT>(h, hb, W, (const WT*)nullptr, W, T, L.ff_rows, W, o, L.w_ff_in_t);
          fused = true;
        }
      }
      if (!fused) {
        gemm<AT, WT, AT>(h, hb, W, (const WT*)L.w_ff_in, W, T, 2 * ff, W, to_buf(pin, h->ld_pin));
        gated_act_kernel<AT><<<dim3((ff + 255) / 256, T), 256, 0, s>>>(pin, h->ld_pin, ff, c.ff_act, c.ff_limit, cat, h->ld_cat);
        h->launches++;
      }
    }
    {
      ProfScope ps(h, HY_PROF_GEMM_OUT);
      gemm<AT, WT, float>(h, cat, h->ld_cat, (const WT*)L.w_ff_down, ff, T, W, ff, to_buf(h->f2, h->ld_f2), L.w_ff_down_t);
    }
    tail.y = h->f2; tail.ldy = h->ld_f2;
  } else {
    const bool few = routed_gated_experts<AT>(h, T, hb, L, c);
    tail.rows = h->f2; tail.ldr = W; tail.pair_row = few ? nullptr : h->x_pair_row; tail.wts = h->x_wts; tail.top = c.x_top;
  }
  ProfScope ps(h, HY_PROF_NORM);
  stream_row<WT>(h, b, tail);
  return HY_OK;
}

template <typename AT>
int run_step(hy_engine* h, const Batch& b, int n_want, const int* want_d, float* layers_out) {
  typedef AT WT;
  const int W = h->m.width, T = b.T, E = b.E;
  const float eps = h->m.norm_eps;
  cudaStream_t s = h->stream;
  AT* hb = (AT*)h->hbuf; AT* pin = (AT*)h->pin; AT* cat = (AT*)h->cat; AT* cv = (AT*)h->cv;
  {
    ProfScope ps(h, HY_PROF_NORM);
    if (h->m.block_kind == HY_BLOCK_PRENORM) {
      embed_pair_kernel<WT><<<T, 128, 0, s>>>(b, (const WT*)h->embed, h->m.emb_scale, (const WT*)h->pair_table, h->m.pair_buckets,
                                              h->m.pair_mul_prev, h->m.pair_mul_cur, h->prev_tok, W, h->x, h->kept);
      prev_token_kernel<<<(E + 127) / 128, 128, 0, s>>>(b, h->prev_tok);
      StreamOp o{};                                            // the first layer's first norm
      o.eps = eps; o.next_w = h->lw[0].pn1; o.next_out = h->hn;
      stream_row<WT>(h, b, o);
      h->launches++;
    } else {
      embed_kernel<WT><<<T, 128, 0, s>>>(b, (const WT*)h->embed, h->inv_freq, h->m.emb_scale, W, h->x);
    }
    h->launches++;
    // output-normed blocks read the stream itself: it leaves here in the activation type too, normed when the model says so
    if (h->m.block_kind == HY_BLOCK_POSTNORM) post_norm_add<AT>(h, T, h->x, W, nullptr, nullptr, nullptr, 0, nullptr, h->embed_norm, nullptr, 0);
  }
  for (size_t li = 0; li < h->lc.size(); ++li) {
    const hy_layer_cfg& c = h->lc[li];
    const LayerW& L = h->lw[li];
    if (h->m.block_kind != HY_BLOCK_PARALLEL) {
      if (h->m.block_kind == HY_BLOCK_SANDWICH) sandwich_layer<AT>(h, b, li);
      else if (h->m.block_kind == HY_BLOCK_POSTNORM) postnorm_layer<AT>(h, b, li);
      else prenorm_layer<AT>(h, b, li);
      if (layers_out) cudaMemcpyAsync(layers_out + li * (size_t)T * W, h->x, (size_t)T * W * 4, cudaMemcpyDeviceToHost, s);
      continue;
    }
    const int ff = c.ff_kind == HY_FF_NONE ? 0 : c.ff;
    {
      ProfScope ps(h, HY_PROF_NORM);
      rmsnorm_kernel<WT, AT><<<T, 256, 0, s>>>(h->x, nullptr, (const WT*)L.norm1, eps, W, 1.0f, hb);
      h->launches++;
    }
    // every projection that reads the normed input, in one product; the feed-forward's hidden part leaves activated,
    // straight into the operand of the merged output projection
    GemmOut o_in{pin, h->ld_pin, L.c_up, cat + L.o_ff, h->ld_cat, 1, nullptr, 0, 1.0f};
    {
      ProfScope ps(h, HY_PROF_GEMM_IN);
      gemm<AT, WT, AT>(h, hb, W, (const WT*)L.w_in, W, T, L.n_in, W, o_in, L.w_in_t);
    }
    if (c.mixer == HY_MIX_ATTN_SCAN) {
      const int nq = c.a_heads * c.a_dim, nk = c.a_kv_heads * c.a_dim, I = c.s_inner, N = c.s_state, R = c.s_dt_rank;
      // attention side: conv over q | k, keys into their pages, attention over the pages
      {
      ProfScope ps(h, HY_PROF_CONV);
      conv_kernel<AT, WT><<<dim3((nq + nk + 127) / 128, T), 128, 0, s>>>(b, pin, h->ld_pin, L.c_q, nq + nk, c.a_conv,
          (const WT*)L.conv_qk, (const WT*)nullptr, 0, L.conv_state, cv, h->ld_cv);
      conv_tail_kernel<AT><<<dim3((nq + nk + 127) / 128, E), 128, 0, s>>>(b, pin, h->ld_pin, L.c_q, nq + nk, c.a_conv, L.conv_state);
      cache_append_kernel<AT><<<T, 128, 0, s>>>(b, cv, h->ld_cv, nq, c.a_kv_heads, c.a_dim, (AT*)L.cache);
      }
      {
      ProfScope ps(h, HY_PROF_ATTN);
      bool tc = false;
      if constexpr (std::is_same<AT, bf16>::value) {
        if ((c.a_dim == 32 || c.a_dim == 64 || c.a_dim == 128) && h->part_o && attn_units(h, E, T, c.a_heads, c.a_kv_heads)) {
          tc = true;
#define HY_ATTN_ARGS b, h->units_d, cv, h->ld_cv, (const bf16*)L.cache, c.a_heads, c.a_kv_heads, c.a_scale, c.a_qt_coef, \
          c.a_qt_every, h->units_split, h->units_ns, c.a_dim, h->part_o, h->part_ml
          if (c.a_dim == 32) attn_mma_kernel<32><<<h->units_n, 128, 0, s>>>(HY_ATTN_ARGS);
          else if (c.a_dim == 64) attn_mma_kernel<64><<<h->units_n, 128, 0, s>>>(HY_ATTN_ARGS);
          else attn_mma_kernel<128><<<h->units_n, 128, 0, s>>>(HY_ATTN_ARGS);
#undef HY_ATTN_ARGS
          attn_combine_kernel<WT, bf16><<<T * c.a_heads, 64, 0, s>>>(b, h->part_o, h->part_ml, (const WT*)L.sink, pin + L.c_g, h->ld_pin,
              c.a_heads, c.a_dim, c.a_dim, h->units_split, h->units_ns, c.left_scale, cat + L.o_mix, h->ld_cat);
          h->launches++;
        }
      }
      if (!tc)
      attn_sink_kernel<AT, WT, AT><<<(T * c.a_heads + 3) / 4, 128, 4 * c.a_dim * sizeof(float), s>>>(
          b, cv, h->ld_cv, (const AT*)L.cache, (const WT*)L.sink, pin + L.c_g, h->ld_pin, c.a_heads, c.a_kv_heads, c.a_dim, c.a_dim,
          c.a_scale, c.a_qt_coef, c.a_qt_every, c.left_scale, cat + L.o_mix, h->ld_cat);
      }
      h->launches += 4;
      // scan side
      {
      ProfScope ps(h, HY_PROF_CONV);
      conv_kernel<AT, WT><<<dim3((I + 127) / 128, T), 128, 0, s>>>(b, pin, h->ld_pin, L.c_x, I, c.s_conv, (const WT*)L.conv_x,
                                                                   (const WT*)L.conv_xb, 1, L.conv_state2, cv, h->ld_cv);
      conv_tail_kernel<AT><<<dim3((I + 127) / 128, E), 128, 0, s>>>(b, pin, h->ld_pin, L.c_x, I, c.s_conv, L.conv_state2);
      }
      h->launches += 2;
      {
      ProfScope ps(h, HY_PROF_SMALL_GEMM);
      gemm<AT, WT, float>(h, cv, h->ld_cv, (const WT*)L.w_x, I, T, R + 2 * N, I, to_buf(h->f1, h->ld_f1), L.w_x_t);
      gemm<float, WT, float>(h, h->f1, h->ld_f1, (const WT*)L.w_dt, R, T, I, R, to_buf(h->f2, h->ld_f2));
      }
      {
        ProfScope ps(h, HY_PROF_SCAN);
        const int nper = N <= 32 ? 1 : N <= 64 ? 2 : N <= 128 ? 4 : 8;
        int lanes = 1;
        while (lanes * nper < N) lanes <<= 1;
        const int per_block = 128 / lanes;
        dim3 grid((I + per_block - 1) / per_block, E);
        const size_t smem = (size_t)HY_SCAN_TB * (2 * N + 3 * per_block) * 4;
#define HY_SCAN_ARGS b, cv, h->ld_cv, pin + L.c_z, h->ld_pin, h->f2, h->ld_f2, (const WT*)L.dt_b, h->f1, h->ld_f1, R, R + N, L.A_neg, \
        (const WT*)L.D, I, N, lanes, c.right_scale, L.rec_state, cat + L.o_scan, h->ld_cat
        if (nper == 1) scan_kernel<AT, WT, 1><<<grid, 128, smem, s>>>(HY_SCAN_ARGS);
        else if (nper == 2) scan_kernel<AT, WT, 2><<<grid, 128, smem, s>>>(HY_SCAN_ARGS);
        else if (nper == 4) scan_kernel<AT, WT, 4><<<grid, 128, smem, s>>>(HY_SCAN_ARGS);
        else scan_kernel<AT, WT, 8><<<grid, 128, smem, s>>>(HY_SCAN_ARGS);
#undef HY_SCAN_ARGS
        h->launches++;
      }
    } else {
      const int nq = c.d_kv_heads * c.d_dim, nv = c.d_heads * c.d_vdim, C = 2 * nq + nv;
      {
      ProfScope ps(h, HY_PROF_CONV);
      conv_kernel<AT, WT><<<dim3((C + 127) / 128, T), 128, 0, s>>>(b, pin, h->ld_pin, L.c_q, C, c.d_conv, (const WT*)L.conv_qkv,
                                                                   (const WT*)nullptr, 1, L.conv_state, cv, h->ld_cv);
      conv_tail_kernel<AT><<<dim3((C + 127) / 128, E), 128, 0, s>>>(b, pin, h->ld_pin, L.c_q, C, c.d_conv, L.conv_state);
      }
      h->launches += 2;
      {
      ProfScope ps(h, HY_PROF_SMALL_GEMM);
      gemm<AT, WT, float>(h, pin + L.c_a1, h->ld_pin, (const WT*)L.w_a2, c.d_low_a, T, c.d_heads * c.d_dim, c.d_low_a,
                          to_buf(h->f1, h->ld_f1), L.w_a2_t);
      gemm<AT, WT, float>(h, pin + L.c_g1, h->ld_pin, (const WT*)L.w_g2, c.d_low_g, T, nv, c.d_low_g, to_buf(h->f2, h->ld_f2),
                          L.w_g2_t);
      }
      ProfScope ps(h, HY_PROF_DELTA);
      const int threads = ((std::max(c.d_dim, c.d_vdim) + 31) / 32) * 32;
#define HY_DELTA_ARGS b, cv, h->ld_cv, 0, nq, 2 * nq, pin, h->ld_pin, L.c_b, h->f1, h->ld_f1, h->f2, h->ld_f2, \
      (const float*)L.A_log, (const float*)L.dt_bias, (const float*)L.norm_w, c.d_heads, c.d_kv_heads, c.d_dim, c.d_vdim, eps, \
      L.rec_state, cat + L.o_mix, h->ld_cat
      static bool delta_attr = false;
      if (!delta_attr) {
        cudaFuncSetAttribute(delta_reg_kernel<AT, float, 32, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        cudaFuncSetAttribute(delta_reg_kernel<AT, float, 64, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        cudaFuncSetAttribute(delta_reg_kernel<AT, float, 128, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        delta_attr = true;
      }
      // one thread per value column, whole warps
      const int nthr = std::max(((c.d_vdim + 31) / 32) * 32, 32);
      auto dsm = [](int dr, int nt) { return (size_t)HY_DELTA_TB * (3 * dr + 3 * nt + 1) * 4; };
      if (c.d_dim <= 32 && nthr <= 512)
        delta_reg_kernel<AT, float, 32, 1><<<dim3(c.d_heads, E), nthr, dsm(32, nthr), s>>>(HY_DELTA_ARGS);
      else if (c.d_dim <= 64 && nthr <= 256)
        delta_reg_kernel<AT, float, 64, 1><<<dim3(c.d_heads, E), nthr, dsm(64, nthr), s>>>(HY_DELTA_ARGS);
      else if (c.d_dim <= 128 && nthr <= 256)
        delta_reg_kernel<AT, float, 128, 1><<<dim3(c.d_heads, E), nthr, dsm(128, nthr), s>>>(HY_DELTA_ARGS);
      else {
        const size_t smem = ((size_t)c.d_dim * c.d_vdim + 3 * c.d_dim + 40) * 4;
        static bool dk_attr = false;
        if (!dk_attr) { cudaFuncSetAttribute(delta_kernel<AT, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024); dk_attr = true; }
        delta_kernel<AT, float><<<dim3(c.d_heads, E), threads, smem, s>>>(HY_DELTA_ARGS);
      }
#undef HY_DELTA_ARGS
      h->launches++;
    }
    (void)ff;
    // merged output projections, added to the residual stream
    GemmOut o_out{nullptr, 0, 0, nullptr, 0, 0, h->x, W, 1.0f};
    {
      ProfScope ps(h, HY_PROF_GEMM_OUT);
      gemm<AT, WT, float>(h, cat, h->ld_cat, (const WT*)L.w_out, L.k_out, T, W, L.k_out, o_out, L.w_out_t);
    }
    if (layers_out) {
      cudaMemcpyAsync(layers_out + li * (size_t)T * W, h->x, (size_t)T * W * 4, cudaMemcpyDeviceToHost, s);
    }
  }
  if (n_want > 0) {
    ProfScope ps(h, HY_PROF_HEAD);
    if (h->m.norm_kind == HY_NORM_TANH) tanh_norm_kernel<AT><<<n_want, 256, 0, s>>>(h->x, want_d, h->final_tanh, W, (AT*)h->hw);
    else rmsnorm_kernel<WT, AT><<<n_want, 256, 0, s>>>(h->x, want_d, (const WT*)h->final_norm, eps, W,
                                                       h->m.norm_kind == HY_NORM_RMS ? 0.0f : 1.0f, (AT*)h->hw);
    h->launches++;
    GemmOut o = to_buf(h->logits, h->m.vocab);
    o.alpha = h->m.logit_scale;
    gemm<AT, WT, float>(h, (const AT*)h->hw, W, (const WT*)h->head, W, n_want, h->m.vocab, W, o, h->head_t);
  }
  return HY_OK;
}

}  // namespace

extern "C" int hy_step(hy_handle h, int32_t n_entries, const int32_t* tokens, const int32_t* ent_start, const int32_t* ent_pos0,
                       const int32_t* ent_slot, const int32_t* pages, int32_t n_want, const int32_t* want, float* logits_out,
                       int32_t* sampled_out, const float* temperature, uint64_t seed, float* layers_out) {
  if (!h || !h->finalized) return h ? fail(h, HY_ERR_INVALID, "hy_finalize has not run") : HY_ERR_INVALID;
  if (n_entries <= 0 || !tokens || !ent_start || !ent_pos0 || !ent_slot || !pages) return fail(h, HY_ERR_INVALID, "null argument");
  const hy_runtime_cfg& rt = h->rt;
  const int E = n_entries, T = ent_start[E];
  if (E > rt.max_step_entries) return fail(h, HY_ERR_CAPACITY, "more entries than max_step_entries");
  if (T <= 0 || T > rt.max_step_tokens) return fail(h, HY_ERR_CAPACITY, "step tokens outside 1..max_step_tokens");
  if (n_want < 0 || n_want > rt.max_want) return fail(h, HY_ERR_CAPACITY, "more wanted rows than max_want");
  HY_CUDA(cudaSetDevice(rt.device));
  // host-side checks of everything a kernel will index with
  for (int e = 0; e < E; ++e) {
    const int cnt = ent_start[e + 1] - ent_start[e];
    if (cnt <= 0 || ent_pos0[e] < 0) return fail(h, HY_ERR_INVALID, "empty entry or negative position");
    if (ent_slot[e] < 0 || ent_slot[e] >= rt.num_slots) return fail(h, HY_ERR_INVALID, "state slot out of range");
    for (int f = 0; f < e; ++f)
      if (ent_slot[f] == ent_slot[e]) return fail(h, HY_ERR_INVALID, "two entries of a step share a state slot");
    const int need = (ent_pos0[e] + cnt + rt.page_size - 1) / rt.page_size;
    if (need > rt.max_pages_per_seq) return fail(h, HY_ERR_CAPACITY, "request longer than max_pages_per_seq pages");
    for (int i = 0; i < need; ++i) {
      const int pg = pages[(size_t)e * rt.max_pages_per_seq + i];
      if (pg < 0 || pg >= rt.num_pages) return fail(h, HY_ERR_INVALID, "page id out of range");
    }
  }
  for (int i = 0; i < T; ++i)
    if (tokens[i] < 0 || tokens[i] >= h->m.vocab) return fail(h, HY_ERR_INVALID, "token id outside the vocabulary");
  for (int i = 0; i < n_want; ++i)
    if (want[i] < 0 || want[i] >= T) return fail(h, HY_ERR_INVALID, "wanted row outside the step");
  // one staging block, one copy
  int* m = h->meta_h;
  int* tok = m; int* tok_ent = tok + T; int* tok_pos = tok_ent + T;
  int* es = tok_pos + T; int* ep = es + E + 1; int* esl = ep + E; int* pg = esl + E;
  int* wn = pg + (size_t)E * rt.max_pages_per_seq;
  memcpy(tok, tokens, (size_t)T * 4);
  for (int e = 0; e < E; ++e) {
    for (int t = ent_start[e]; t < ent_start[e + 1]; ++t) { tok_ent[t] = e; tok_pos[t] = ent_pos0[e] + t - ent_start[e]; }
    es[e] = ent_start[e]; ep[e] = ent_pos0[e]; esl[e] = ent_slot[e];
  }
  es[E] = T;
  memcpy(pg, pages, (size_t)E * rt.max_pages_per_seq * 4);
  if (n_want) memcpy(wn, want, (size_t)n_want * 4);
  const size_t words = (size_t)(wn - m) + n_want;
  HY_CUDA(cudaMemcpyAsync(h->meta_d, m, words * 4, cudaMemcpyHostToDevice, h->stream));
  const int* d = h->meta_d;
  Batch b;
  b.tok = d; b.tok_ent = d + T; b.tok_pos = d + 2 * T; b.ent_start = d + 3 * T; b.ent_pos0 = b.ent_start + E + 1;
  b.ent_slot = b.ent_pos0 + E; b.pages = b.ent_slot + E;
  b.T = T; b.E = E; b.max_pages = rt.max_pages_per_seq; b.page_size = rt.page_size;
  const int* want_d = b.pages + (size_t)E * rt.max_pages_per_seq;
  h->step_start = ent_start; h->step_pos0 = ent_pos0; h->units_n = 0;
  HY_CUDA(cudaEventRecord(h->ev0, h->stream));
  if (h->m.dtype == HY_DTYPE_F32) run_step<float>(h, b, n_want, want_d, layers_out);
  else run_step<__nv_bfloat16>(h, b, n_want, want_d, layers_out);
  if (n_want > 0 && sampled_out) {
    const float* td = nullptr;
    if (temperature) {
      HY_CUDA(cudaMemcpyAsync(h->temp_d, temperature, (size_t)n_want * 4, cudaMemcpyHostToDevice, h->stream));
      td = h->temp_d;
    }
    sample_kernel<<<n_want, 256, 0, h->stream>>>(h->logits, h->m.vocab, td, seed, h->sampled);
    h->launches++;
    HY_CUDA(cudaMemcpyAsync(sampled_out, h->sampled, (size_t)n_want * 4, cudaMemcpyDeviceToHost, h->stream));
  }
  HY_CUDA(cudaEventRecord(h->ev1, h->stream));
  if (n_want > 0 && logits_out)
    HY_CUDA(cudaMemcpyAsync(logits_out, h->logits, (size_t)n_want * h->m.vocab * 4, cudaMemcpyDeviceToHost, h->stream));
  HY_CUDA(cudaMemcpyAsync(h->err_h, h->err_d, 4, cudaMemcpyDeviceToHost, h->stream));
  HY_CUDA(cudaStreamSynchronize(h->stream));
  HY_CUDA(cudaGetLastError());
  if (*h->err_h) {
    *h->err_h = 0;
    cudaMemset(h->err_d, 0, 4);
    return fail(h, HY_ERR_CUDA, "a wait inside the tensor-core matrix product ran out (pipeline stalled)");
  }
  cudaEventElapsedTime(&h->last_ms, h->ev0, h->ev1);
  for (auto& r : h->prof_list) {
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, r.a, r.b);
    h->prof_ms[r.cat] += ms;
    h->ev_pool.push_back(r.a);
    h->ev_pool.push_back(r.b);
  }
  h->prof_list.clear();
  return HY_OK;
}
