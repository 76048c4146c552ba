/* jacobi_hybrid.h — C ABI of libjf_hybrid.so: layered hybrid decoders on B200.  Two block layouts over one residual
 * stream: one RMS norm per layer feeding mixer and feed-forward side by side (softmax attention with a sink whose values
 * are its keys, selective scans, gated delta rule layers, squared-ReLU feed-forward), and norm - sublayer - norm blocks
 * with element-wise tanh norms and per-channel layer scales (scalar-decay state-space recurrence, attention over a shared
 * low-rank latent with a rotated key part, gated linear recurrence, routed gated experts), and blocks whose sublayers read
 * the stream itself and are RMS-normed on the way back (attention over a sliding window plus pooled blocks with rotated
 * values, matrix memory with capped exponential gates, gated dense feed-forward, routed plain experts beside a shared one),
 * and pre-norm blocks whose sublayers read the normed stream through a short convolution over time and are followed by a
 * per-layer token input and an average over the depth (attention with capped scores, a logarithmic distance bias, a
 * window plus kept first tokens and a sink in the denominator; clamped gated dense feed-forward; routed gated experts).
 *
 * Same conventions as jacobi_b200.h: every function returns 0 or a negative status, hy_last_error(h) gives the text,
 * plain pointers and sizes only, host buffers are caller-owned, device memory belongs to the handle, one host thread per
 * handle.  There is no CPU fallback: without a CUDA device hy_create fails.
 *
 * A model is a list of layers (hy_layer_cfg) over a shared residual stream.  The host names tensors as the checkpoint
 * does ("l<i>.norm1", "l<i>.mix.left.q", ...); merging of the projections that read the same input and the layouts the
 * kernels want are made behind hy_finalize.  A step runs a batch of entries, each the next tokens of one request (a
 * portion of a prompt or a single decoded token), against the paged key cache and the request's recurrent-state slot.
 */
#ifndef JACOBI_HYBRID_H_
#define JACOBI_HYBRID_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hy_engine* hy_handle;

typedef enum { HY_OK = 0, HY_ERR_INVALID = -1, HY_ERR_CUDA = -2, HY_ERR_CAPACITY = -3, HY_ERR_UNSUPPORTED = -4 } hy_status;
typedef enum { HY_DTYPE_BF16 = 0, HY_DTYPE_F32 = 1, HY_DTYPE_F16 = 2, HY_DTYPE_I32 = 3 } hy_dtype;
typedef enum { HY_MIX_ATTN_SCAN = 0, HY_MIX_DELTA = 1, HY_MIX_SSD = 2, HY_MIX_LATENT = 3, HY_MIX_GLR = 4, HY_MIX_WINDOW = 5,
               HY_MIX_MLSTM = 6, HY_MIX_BIASED = 7 } hy_mixer_kind;
/* HY_FF_GATED: down(act(gate x) * (up x)), act = hy_act_kind in ff_act */
typedef enum { HY_FF_NONE = 0, HY_FF_RELU2 = 1, HY_FF_ROUTED = 2, HY_FF_GATED = 3 } hy_ff_kind;
/* HY_ACT_CLAMPED (gated pairs only): g = min(gate, limit), u = clamp(up, -limit, limit), g sigmoid(1.702 g) (u + 1) */
typedef enum { HY_ACT_SILU = 0, HY_ACT_GELU_TANH = 1, HY_ACT_GELU_ERF = 2, HY_ACT_CLAMPED = 3 } hy_act_kind;
/* how a routed feed-forward scores its experts: sigmoid scores, group-limited choice, weights normalised to x_scale |
 * the largest logits (plus a bias per expert), weights = softmax over the chosen logits alone */
typedef enum { HY_ROUTE_SIGMOID_GROUPS = 0, HY_ROUTE_TOP_SOFTMAX = 1 } hy_route_kind;
/* norm of the residual stream: RMS with a weight stored as an offset from one | tanh(alpha x) w + b (no statistics) |
 * RMS with a plain weight */
typedef enum { HY_NORM_RMS_OFFSET = 0, HY_NORM_TANH = 1, HY_NORM_RMS = 2 } hy_norm_kind;
/* HY_BLOCK_PARALLEL: x += mixer(n(x)) + ff(n(x)), one norm per layer.
 * HY_BLOCK_SANDWICH: x += ls1 * n1b(mixer(n1(x))), then x += ls2 * n2b(ff(n2(x))): a norm on both sides of each sublayer
 * and a per-channel layer scale.
 * HY_BLOCK_POSTNORM: x += ls1 * n1(mixer(x)), then x += ls2 * n2(ff(x)): the sublayers read the stream itself, the norm
 * (RMS, with statistics over the width) sits on the sublayer's output.
 * HY_BLOCK_PRENORM: x += m ls1 mixer(c1(n1(x))), then x += m ls2 ff(c2(n2(x))): RMS norms with plain weights on the
 * sublayers' inputs, c(h) = h + a causal convolution of h over time per channel (hy_model_cfg.canon_taps taps, 0: none),
 * m = hy_model_cfg.resid_mult; then the per-layer token input and the average over the depth when the model has them. */
typedef enum { HY_BLOCK_PARALLEL = 0, HY_BLOCK_SANDWICH = 1, HY_BLOCK_POSTNORM = 2, HY_BLOCK_PRENORM = 3 } hy_block_kind;
typedef enum { HY_POS_SINUSOID = 0, HY_POS_NONE = 1 } hy_pos_kind;   /* what is added to the scaled embedding */

typedef struct {
  int32_t mixer;                   /* hy_mixer_kind */
  /* HY_MIX_ATTN_SCAN, attention side: query heads, key heads (values are the keys), key size, value size, conv taps,
   * the query temperature 1 + qt_coef * ln(floor((p + 1) / qt_every) + 1), the score scale */
  int32_t a_heads, a_kv_heads, a_dim, a_vdim, a_conv, a_qt_every;
  float a_scale, a_qt_coef;
  /* scan side: channels, state size, rank of the step-size projection, conv taps */
  int32_t s_inner, s_state, s_dt_rank, s_conv;
  float left_scale, right_scale;   /* mixer = left_scale * attention + right_scale * scan */
  /* HY_MIX_DELTA: value heads, query/key heads, key size, value size, conv taps, inner sizes of the two-step decay and
   * gate projections (read from the tensor shapes) */
  int32_t d_heads, d_kv_heads, d_dim, d_vdim, d_conv, d_low_a, d_low_g;
  int32_t ff_kind, ff;             /* hy_ff_kind, hidden size of the feed-forward (of one expert when routed) */
  /* HY_MIX_SSD (state-space recurrence with one decay per head): heads, channels per head, state size, groups that share
   * B and C, conv taps, parts of the gated output norm */
  int32_t m_heads, m_vdim, m_state, m_groups, m_conv, m_norm_groups;
  /* HY_MIX_LATENT (attention over a shared low-rank latent): heads, unrotated and rotated query/key size per head,
   * value size, ranks of the key/value and the query latent, the layer whose cached latent is used (-1: its own),
   * the score scale; rotation over the first r_dims of the rotated part with base r_base, frequencies interpolated by
   * r_factor between the wavelengths original / r_fast and original / r_slow (r_factor <= 0: plain rotation) */
  int32_t l_heads, l_dim, l_rot_dim, l_vdim, l_kv_rank, l_q_rank, l_kv_from;
  float l_scale;
  int32_t r_dims;
  float r_base, r_factor, r_original, r_fast, r_slow;
  /* HY_MIX_GLR (gated linear recurrence, forget gate = 1 - input gate, bounded below per channel) */
  int32_t g_heads, g_dim, g_vdim;
  /* HY_FF_ROUTED: experts, experts used per token, groups of neighbouring experts, groups a token may choose from,
   * factor on the normalised weights */
  int32_t x_experts, x_top, x_groups, x_keep;
  float x_scale;
  /* more of HY_FF_ROUTED: hy_route_kind; experts without a gate (down(act(up x))); hy_act_kind of the experts; size of a
   * shared expert of the same form that every token uses with weight one (0: none).  ff_act: hy_act_kind of HY_FF_GATED */
  int32_t x_route, x_plain, x_act, x_shared_ff, ff_act;
  /* HY_MIX_WINDOW (softmax attention over a sliding window plus one pooled key / value per block of w_pool tokens that
   * has its last token behind the window): query heads, key/value heads, key size, value size, window length, block length,
   * rotated dimensions of queries and keys (pairs 2i, 2i + 1; 0: none), values rotated by their own position over all
   * of w_vdim and the output turned back by the query's (0 / 1), RMS norm per head on queries and keys (0 / 1);
   * rotation base, score scale */
  int32_t w_heads, w_kv_heads, w_dim, w_vdim, w_window, w_pool, w_rot_dims, w_rot_values, w_qk_norm;
  float w_rot_base, w_scale;
  /* HY_MIX_MLSTM (matrix memory with exponential gates under a running maximum): heads, key size, value size, the cap
   * c of both gate pre-activations (c tanh(z / c); <= 0: no cap) */
  int32_t t_heads, t_dim, t_vdim;
  float t_gate_cap;
  /* HY_MIX_BIASED (softmax attention without rotation; projections with biases): query heads, key/value heads, key size,
   * value size; position i sees j <= i with i - j < b_window (0: every j) or j < b_keep_first; b_v_mix: 1 = the values
   * are blended with the values of the first layer that says so, v <- (1 - l) v + l v_first, l = the layer's "vmix";
   * score = b_scale q.k, then b_softcap tanh(score / b_softcap) (<= 0: no cap), minus r1_h ln(1 + r2_h (i - j)); the
   * softmax's denominator also holds exp(sink_h) */
  int32_t b_heads, b_kv_heads, b_dim, b_vdim, b_window, b_keep_first, b_v_mix;
  float b_scale, b_softcap;
  float ff_limit;                  /* the limit of HY_ACT_CLAMPED in a HY_FF_GATED feed-forward */
} hy_layer_cfg;

typedef struct {
  int32_t width, vocab, n_layers;
  int32_t dtype;                   /* HY_DTYPE_BF16: bf16 operands, fp32 accumulation / state / residual; HY_DTYPE_F32: all fp32 */
  float emb_scale, logit_scale, norm_eps;
  int32_t norm_kind, block_kind, pos_kind;   /* hy_norm_kind, hy_block_kind, hy_pos_kind */
  int32_t embed_norm;              /* 1: the embedding passes through the model's norm with the weight "embed.norm" */
  int32_t tied_head;               /* 1: the output head is the embedding table (no "head" tensor) */
  /* HY_BLOCK_PRENORM: factor on every sublayer's result; taps of the input convolutions (0: none); size of the per-layer
   * token input (0: none; table "side.embed" [vocab, n_layers * side_dim]); 1: each layer's result is replaced by the
   * weighted sum of the embedding output and all layers' results so far (weights "l<i>.dwa") */
  float resid_mult;
  int32_t canon_taps, side_dim, depth_avg;
  /* hashed embedding of the (previous, current) token pair, added to the scaled embedding: row (prev * pair_mul_prev +
   * cur * pair_mul_cur) mod pair_buckets of "bigram", row pair_buckets for a request's first token (0 buckets: none) */
  int32_t pair_buckets, pair_mul_prev, pair_mul_cur;
} hy_model_cfg;

typedef struct {
  int32_t device;
  int32_t max_step_tokens;         /* tokens of all entries of one step */
  int32_t max_step_entries;
  int32_t page_size;               /* tokens per key-cache page (multiple of 16) */
  int32_t num_pages;
  int32_t max_pages_per_seq;
  int32_t num_slots;               /* recurrent-state slots (one per live request) */
  int32_t max_want;                /* rows whose logits one step may return */
} hy_runtime_cfg;

int hy_create(const hy_model_cfg* model, const hy_layer_cfg* layers, const hy_runtime_cfg* rt, hy_handle* out);
void hy_destroy(hy_handle h);
const char* hy_last_error(hy_handle h);

/* One checkpoint tensor by name (host pointer).  All tensors first, then hy_finalize. */
int hy_load_tensor(hy_handle h, const char* name, const void* data, const int64_t* shape, int32_t ndim, int32_t dtype);
int hy_finalize(hy_handle h);

/* One step.  tokens[total] holds the entries' tokens back to back; entry e covers [ent_start[e], ent_start[e+1]) and its
 * first token sits at position ent_pos0[e] of its request (the positions before it are in the cache / state already; an
 * entry with ent_pos0 == 0 starts from the empty state whatever its slot held).  pages[e * max_pages_per_seq + i] is the
 * page of tokens [i * page_size, (i + 1) * page_size).  want[n_want] are indices into tokens[]; logits_out (host, fp32,
 * [n_want, vocab]) and sampled_out (host, int32 [n_want]) may be NULL.  temperature[n_want] NULL or 0 = argmax, else a
 * draw from softmax(logits / temperature) with the counter-based generator keyed by (seed, want index).
 * layers_out: NULL, or host fp32 [n_layers, total, width] receiving the residual stream after every layer. */
int hy_step(hy_handle h, int32_t n_entries, const int32_t* tokens, const int32_t* ent_start, const int32_t* ent_pos0,
            const int32_t* ent_slot, const int32_t* pages, int32_t n_want, const int32_t* want, float* logits_out,
            int32_t* sampled_out, const float* temperature, uint64_t seed, float* layers_out);

int64_t hy_launch_count(hy_handle h);
/* Device milliseconds of the last hy_step (CUDA events on the handle's stream). */
float hy_last_step_ms(hy_handle h);
/* Bytes of device memory held: weights, cache pages, state slots, workspace. */
int hy_memory_info(hy_handle h, int64_t* weights, int64_t* cache, int64_t* state, int64_t* workspace);

/* Device time per group of kernels, summed over the steps since hy_profile_enable(h, 1): ms[HY_PROFILE_CATEGORIES]. */
enum { HY_PROF_NORM = 0, HY_PROF_GEMM_IN = 1, HY_PROF_CONV = 2, HY_PROF_ATTN = 3, HY_PROF_SMALL_GEMM = 4, HY_PROF_SCAN = 5,
       HY_PROF_DELTA = 6, HY_PROF_GEMM_OUT = 7, HY_PROF_HEAD = 8, HY_PROF_ROUTE = 9, HY_PROF_EXPERTS = 10,
       HY_PROFILE_CATEGORIES = 11 };
int hy_profile_enable(hy_handle h, int32_t on);
int hy_profile_read(hy_handle h, float* ms);

#ifdef __cplusplus
}
#endif
#endif
