// Internal interface between the translation units of the sequence-batch engine (seq_engine.cu: the
// step function, the paged cache and its slot manager; seq_kernels.cu: norms, query/key preparation,
// paged attention, router and expert kernels; seq_gemm.cu: token-block matrix products).
//
// Conventions.  A step processes T tokens of several sequences as ONE ragged batch: activations are
// [T, .] row-major with no padding, and three int32 arrays describe the rows -- tok_seq[t] (cache slot of
// the row's sequence), tok_pos[t] (its position, counted from 0 in the sequence) and, per entry of the
// step, ent_first[e] / ent_count[e] / ent_seq[e] / ent_pos0[e].  The residual stream, every norm, every
// softmax and the router are fp32 whatever the compute type; `AT` below is the activation / weight type
// of the matrix products (float, or __nv_bfloat16 with fp32 accumulation).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/kllm_seq.h"
#include "kllm_host.h"

namespace kllm {
namespace seq {

constexpr int kAttnRows = 32;   // (token, query head) rows of one attention CTA
constexpr int kAttnKeys = 64;   // keys per tile
constexpr int kAttnThreads = 128;

struct NormW {
  const float* w;
  const float* b;  // may be null: no bias
  int kind;        // KLLM_SEQ_NORM_LAYER / KLLM_SEQ_NORM_RMS
};

// Where the keys and values of one layer run live: pages of `page` tokens, [n_pages][page][kv_heads][dim].
// k_row / v_row: elements between two tokens' rows (kv_heads * dim and kv_heads * vdim when keys and values have pools
// of their own; a latent cache keeps one row per token and its values are the head of the key row: v == k, v_row == k_row).
struct PagedKV {
  void* k;
  void* v;
  const int32_t* table;  // [slots][table_stride]: page number of the i-th page of a sequence
  int table_stride;
  int page;
  int k_row, v_row;
};

struct AttnShape {
  int heads, kv_heads, dim, vdim;
  float scale;
  float temp_coef;  // query temperature 1 + coef * ln(floor((p + 1) / every) + 1); every == 0: none
  int temp_every;
  int qk_norm;      // RMS norm of each query / key head with a shared weight vector
  int gate;         // one sigmoid gate per (token, head) on the attention output
  int window;       // position i sees j with 0 <= i - j < window; 0: every earlier position
  const float* sink;  // [heads] or null: exp(sink) is added to the softmax denominator
  int q_f32;        // the queries are fp32 whatever the compute type
  int out_f32;      // the output is written in fp32 whatever the compute type
  int no_merge;     // leave the splits' partial results in the workspace: the caller merges them (latent_merge_expand)
  int keep_first;   // with a window: the first keep_first positions stay visible to every later one
  float softcap;    // score <- softcap * tanh(score / softcap) after the scale; 0: none
  // Attention maps that share values: v_share consecutive key heads read the values of ONE value head (key head g reads
  // value head g / v_share; the value rows hold kv_heads / v_share heads).  `heads` and `kv_heads` count the maps.  0: 1.
  int v_share;
};
inline __host__ __device__ int v_share_of(const AttnShape& a) { return a.v_share > 1 ? a.v_share : 1; }
// floats of one token's output gates: none, one per head, or one per output element (heads count maps; gates do not)
inline __host__ __device__ int gate_floats(const AttnShape& a) {
  const int h = a.heads / v_share_of(a);
  return a.gate == KLLM_SEQ_GATE_ELEMENT ? h * a.vdim : (a.gate ? h : 0);
}
// Rotary positions on the first `dims` coordinates of every query / key head (map).
struct RopeArgs {
  int dims;           // 0: none
  float base;         // angle of pair i = position * base^(-2 i / dims) ...
  const float* freq;  // ... or position * freq[i] when given ([dims / 2] fp32)
  float mag;          // cos and sin are multiplied by it
  int pairing;        // KLLM_SEQ_ROPE_*
};

// The activation that joins a gate row's product g and an up row's product u (see KLLM_SEQ_ACT_*).
struct GatedAct {
  int kind;
  float limit, alpha;
};
__host__ __device__ inline float gated_act(const GatedAct& a, float g, float u) {
  if (a.kind == KLLM_SEQ_ACT_CLAMP_SWIGLU) {
    g = fminf(g, a.limit);
    u = fminf(fmaxf(u, -a.limit), a.limit);
    return g / (1.0f + expf(-a.alpha * g)) * (u + 1.0f);
  }
  if (a.kind == KLLM_SEQ_ACT_RELU_GATE) return fmaxf(g, 0.f) * u;
  return g / (1.0f + expf(-g)) * u;
}

// ---- seq_kernels.cu -----------------------------------------------------------------------------------------------
// x[t] = norm(table[tokens[t]] * scale) (norm.w == null: the scaled row itself); `copy` (optional) receives the same rows
int launch_embed(int dtype, const void* table, const int32_t* tokens, float* x, float* copy, const NormW& norm, float eps,
                 float scale, int T, int width, cudaStream_t s);

// x += N(c1 y1 + s2[t] * y2 + c3 y3 + c4 y4; post) (optional; y2, y3, y4 optional; post.w == null: the sum itself);  x += add_rows[t];
// x += add (a [width] vector, optional);  out = N(x; pre) in the compute type (optional) -- in this order.  `rows` (optional) gathers: row i reads x[rows[i]], and x is then
// left untouched (only `out` is written).
// Router of a mixture of experts for the rows of `out` (optional, w_router != NULL; needs `pre`): logits z = Wr h in
// fp32 on the row just written, s = softmax(z), the `top` largest, weights s / (sum + 1e-20) * scale; shared-expert gate
// sigmoid(w_sg . h) when w_sg is given.
// kind KLLM_SEQ_ROUTER_SIGMOID: s = sigmoid(z); choice scores s + correction; with groups > 0 only experts of the
// groups_keep groups with the largest sum of their two best choice scores can be chosen; weights s * scale.
struct RouterArgs {
  const float* w_router;  // [experts][width]
  const float* w_sg;      // [width] or NULL
  int experts, top;
  float scale;
  int32_t* top_idx;       // [T, top]
  float* top_w;           // [T, top]
  float* sgate;           // [T]
  int kind;
  const float* correction;  // [experts] or NULL
  int groups, groups_keep;
  const float* bias;        // [experts] added to the logits, or NULL
};
__host__ __device__ inline size_t router_smem_floats(const RouterArgs& r) { return 2 * static_cast<size_t>(r.experts) + r.groups; }
// Token shift on the rows a norm kernel writes, for steps in which every sequence brings ONE token: the row's CTA owns
// its sequence's state.  out = h + (prev - h) * mu, prev = state[seq] (zeros at position 0); state[seq] = h.
struct ShiftArgs {
  const float* mu;     // [width] or null: no shift
  float* state;        // [slots][width]
  const int32_t* tok_seq;
  const int32_t* tok_pos;
};
struct ResidNormArgs {
  float* x;
  const float* add;
  const float* y1;
  const float* y2;
  const float* s2;
  NormW post;
  NormW pre;
  void* out;
  const int32_t* rows;
  int T, width, dtype;
  float eps;
  RouterArgs router;
  const float* add_rows;  // [T, width] added to x row by row (before `add`), optional
  float* out_f32;         // instead of `out`: the normed rows in fp32 (a token-shift kernel follows)
  ShiftArgs shift;        // inline token shift (single-token steps)
  const float* y3;        // further addends of the sum that joins x (with y1)
  const float* y4;
  float c1 = 1.0f, c3 = 1.0f, c4 = 1.0f;  // the coefficients of y1, y3, y4
  NormW n1{}, n3{};  // RMS norms of y1 and y3 on their own, before the sum (w == null: none)
};
int launch_resid_norm(const ResidNormArgs& a, cudaStream_t s);

// qkvg: [T, heads*dim + kv_heads*dim + (kv_heads / v_share)*vdim + gate_floats()] fp32 (projection output).
// Writes q [T, heads, dim] (compute type; head norm, rotation, temperature applied), the key / value rows into the pages,
// and the gates sigmoid(.) [T, gate_floats()] fp32.  qk_norm KLLM_SEQ_QKNORM_WEIGHTED norms before the rotation,
// KLLM_SEQ_QKNORM_UNIT after it.  With v_share > 1 the projection's query rows are head by head [map 0 | map 1 ...] and q
// is written map-major inside each group of heads that share keys -- head h, map m of key group g goes to index
// (g * v_share + m) * rep + h % rep, rep = query heads per key head -- so that the attention kernels find the rows of one
// key head side by side.
int launch_qk_prepare(int dtype, const AttnShape& a, const RopeArgs& rope, const float* qkvg, const float* qnorm_w,
                      const float* knorm_w, float eps, const int32_t* tok_seq, const int32_t* tok_pos, void* q, float* gates,
                      const PagedKV& kv, int T, cudaStream_t s);
// Differential attention: joins the key splits of both maps of every head (a.no_merge left them in `ws`), then
// o = a1 - lambda * a2, o / sqrt(mean(o^2) + eps) * out_scale over the head's vdim values, the output gate, and the
// conversion: out [T, (heads / 2) * vdim] in the compute type.  `a` is the shape the attention ran with (v_share == 2).
int launch_diff_merge(int dtype, const AttnShape& a, int splits, const float* ws, const float* gates, float lambda,
                      float out_scale, float eps, void* out, int T, cudaStream_t s);

// Causal softmax attention of the step's rows over their sequences' pages.  out [T, heads*vdim] (compute type).
// `splits` CTAs share the keys of a row tile; partial (max, sum, unnormalised output) go through `ws`.
size_t attention_workspace_bytes(const AttnShape& a, int T, int splits);
int launch_attention(int dtype, const AttnShape& a, const void* q, const float* gates, const PagedKV& kv,
                     int n_entries, const int32_t* ent_first, const int32_t* ent_count, const int32_t* ent_seq,
                     const int32_t* ent_pos0, int max_count, int max_ctx, int splits, float* ws, void* out, int T,
                     const int32_t* tok_seq, const int32_t* tok_pos, cudaStream_t s);

// Prompt steps in bf16 with head sizes up to 128 (multiples of 8): the same attention on the tensor cores (seq_attention_mma.cu).
// With splits == 1 it writes `out` itself (gate applied); otherwise it leaves partial results in `ws` for the merge.
bool attention_mma_usable(int dtype, const AttnShape& a, int max_count);
int launch_attention_mma(const AttnShape& a, const void* q, const float* gates, const PagedKV& kv, int n_entries,
                         const int32_t* ent_first, const int32_t* ent_count, const int32_t* ent_seq,
                         const int32_t* ent_pos0, int max_count, int splits, float* ws, void* out, cudaStream_t s);

// Token shift for steps with longer entries: out[t] = h[t] + (prev - h[t]) * mu in the compute type, prev = h[t - 1] inside
// an entry, the sequence's state (zeros at position 0) for its first row; afterwards state[seq] = the entry's last h.
int launch_token_shift(int dtype, const float* h, const float* mu, float* state, const int32_t* tok_seq,
                       const int32_t* tok_pos, const int32_t* ent_first, const int32_t* ent_count, int n_entries, void* out,
                       int T, int width, cudaStream_t s);

// ---- seq_mixers.cu: attention through a latent, linear attention, dense feed-forward activations -----------------------
struct LatentShape {
  int heads, dim, rot_dim, vdim, q_rank, kv_rank;
  int rope_dims;
  float rope_base;
};
// proj [T, q_rank + kv_rank + rot_dim + heads] fp32 -> cq [T, q_rank] (compute type, RMS-normed), the cache row
// [kv_rank normed latent | rot_dim rotated key part] of every token, gates [T, heads] = sigmoid
int launch_latent_prepare(int dtype, const LatentShape& a, const float* proj, const float* q_norm_w, const float* kv_norm_w,
                          float eps, const int32_t* tok_seq, const int32_t* tok_pos, void* cq, float* gates,
                          const PagedKV& kv, void* c_rows, float* kr_rows, int T, cudaStream_t s);
// Prompt steps that start their sequences can expand the latents of the step into per-head keys and values and run the
// tensor-core attention on them: c_rows [T, kv_rank] (compute type) and kr_rows [T, rot_dim] (fp32, rotated) are the
// step's latents as rows (optional outputs of latent_prepare); pack_q rotates and converts the queries; pack_kv joins
// W_uk c with the shared rotated part and converts W_uv c.
int launch_latent_pack_q(int dtype, const LatentShape& a, const float* q, const int32_t* tok_pos, void* out, int T,
                         cudaStream_t s);
int launch_latent_pack_kv(int dtype, const LatentShape& a, const float* kp, const float* kr, const float* vp, void* k, void* v,
                          int T, cudaStream_t s);
// q [T, heads, dim + rot_dim] fp32 -> qa [T, heads, kv_rank + rot_dim] fp32: W_uk(head)^T q_plain | rotated q_rot
int launch_latent_absorb(int dtype, const LatentShape& a, const float* q, const void* w_uk, const int32_t* tok_pos, float* qa,
                         int T, cudaStream_t s);
// Single-token steps: the merge of the key splits (sink and gate included) and W_uv in one kernel, a CTA per (token, head).
// ws: the partial results launch_attention left (AttnShape::no_merge) for value size kv_rank.
int launch_latent_merge_expand(int dtype, const LatentShape& a, int splits, const float* ws, const float* gates,
                               const float* sink, const void* w_uv, void* out, int T, cudaStream_t s);
// ol [T, heads, kv_rank] fp32 (weighted sums of latents) -> out [T, heads * vdim] compute type: W_uv(head) ol
int launch_latent_expand(int dtype, const LatentShape& a, const float* ol, const void* w_uv, void* out, int T, cudaStream_t s);

// proj [T, 2 * heads * dim + 2 * heads * vdim] fp32: q | k | v | gate rows before their activations.  Runs the recurrence
// of every entry from its sequence's state ([slots][heads][dim][vdim] fp32; zeros at position 0), writes o [T, heads * vdim]
// fp32 and the new state.
// Steps with long entries work chunk-parallel through `scratch` (linear_attention_scratch_bytes(); 0: not needed).
size_t linear_attention_scratch_bytes(int heads, int dim, int vdim, int T, int n_entries, int max_count);
int launch_linear_attention(int heads, int dim, int vdim, const float* decay, const float* proj, float* state, int n_entries,
                            const int32_t* ent_first, const int32_t* ent_count, const int32_t* ent_seq,
                            const int32_t* ent_pos0, int max_count, float* scratch, float* o, cudaStream_t s);
// out[t] = RMSnorm(o[t]; w) * sigmoid(gate rows of proj[t]) in the compute type
int launch_linear_out(int dtype, int heads, int dim, int vdim, const float* o, const float* proj, const float* norm_w, float eps,
                      void* out, int T, cudaStream_t s);
// out = act(z) element by element (z fp32 [n], out compute type): KLLM_SEQ_ACT_XIELU with (a, b), or KLLM_SEQ_ACT_RELU2
int launch_activation(int dtype, int act, float a, float b, const float* z, void* out, size_t n, cudaStream_t s);
// v *= scale (0: 1), then v <- cap * tanh(v / cap) (cap 0: none)
int launch_scale(float* v, float scale, float cap, size_t n, cudaStream_t s);

// Router: z = Wr h (fp32), s = softmax(z), the `top` largest, weights s / (sum + 1e-20) * scale; shared-expert gate
// sigmoid(w_sg . h) when w_sg is given.
int launch_router(int dtype, const void* h, const float* w_router, const float* w_sg, int experts, int top,
                  float scale, int32_t* top_idx, float* top_w, float* sgate, int T, int width, cudaStream_t s);

// Routed experts, one (token, chosen expert) pair at a time: inter[pair] = silu(Wg h) * (Wu h), then
// y[t] = sum_k w_k * Wd_k inter[t, k].  gate_up: [experts][2*ff][width] (gate rows, then up rows); down:
// [experts][width][ff].
// A shared expert can ride along in both kernels (ff > 0): it is one more pair per token, chosen always, with its own
// weights and inner size; y then holds routed + gate[t] * shared (gate NULL: 1).  Needs shared_expert_rides_along().
struct SharedExpert {
  const void* gate_up;  // [2*ff][width]
  const void* down;     // [width][ff]
  const float* gate;    // [T] or NULL
  void* inter;          // [T, ff] workspace in the compute type
  int ff;               // 0: no shared expert in these kernels
  float limit;          // its own clamp when the activation has one
};
bool shared_expert_rides_along(int top, int ff, int shared_ff);
// act KLLM_SEQ_ACT_RELU2: inter[pair] = max(Wu h, 0)^2 with gate_up = [experts][ff][width] (no shared expert then)
int launch_expert_gate_up(int dtype, const void* h, const void* gate_up, const int32_t* top_idx, void* inter, int T,
                          int top, int ff, int width, const SharedExpert& sh, const GatedAct& act, cudaStream_t s);
int launch_expert_down(int dtype, const void* inter, const void* down, const int32_t* top_idx, const float* top_w,
                       float* y, int T, int top, int ff, int width, const SharedExpert& sh, cudaStream_t s);

// y[t] = sum_k w[t, k] * yp[t * top + k]   (fp32 [T * top, width] -> [T, width])
int launch_combine_pairs(const float* yp, const float* top_w, float* y, int T, int top, int width, cudaStream_t s);

// out[t, f] = act(gu[t, f], gu[t, ff + f])   (gu fp32 [T, 2*ff], out compute type [T, ff]; silu(g) * u for KLLM_SEQ_ACT_SWIGLU)
int launch_gated_act(int dtype, const GatedAct& act, const float* gu, void* out, int T, int ff, cudaStream_t s);

// Routed experts over token blocks (prefill): rows grouped by expert.  sort_pairs builds, on the device, the list of
// pairs ordered by expert in blocks of `block` rows (padded with -1), and the expert of every block.
int launch_sort_pairs(const int32_t* top_idx, int n_pairs, int experts, int block, int32_t* counts /*[experts+1]*/,
                      int32_t* sorted_pair /*[cap]*/, int32_t* block_expert /*[cap/block]*/, int cap, cudaStream_t s);

// ---- seq_recurrent.cu: short convolutions with their state, query / key preparation behind one, selective scan, gated delta rule ----
// Where the last taps - 1 inputs of a convolution live: [slots][taps - 1][channels] fp32, row i of a sequence of length n
// holds the input at position n - (taps - 1) + i (positions below 0 are never read).
// Rows of one step: row t of an entry sees the entry's earlier rows directly and the sequence's state before them.  The CTA
// of an entry's first row also computes the entry's next taps - 2 rows (every read of the old state happens there) and then
// writes the new state; no other CTA touches the state.
struct StepRows {
  const int32_t* tok_seq;
  const int32_t* tok_pos;
  const int32_t* ent_first;
  const int32_t* ent_count;
  const int32_t* ent_pos0;
  int n_entries;
};
struct AttnPrep {
  int taps;               // 1: no convolution
  const float* conv_w;    // [(heads + kv_heads) * dim][taps]
  float* conv_state;      // [slots][taps - 1][(heads + kv_heads) * dim]
  const float* bias;      // [(heads + kv_heads) * dim] or NULL
  int rope_dims, rope_pairing;
  float rope_base;
};
// qk [T, heads*dim + kv_heads*dim] fp32 (projection output, values are the keys): bias, convolution, then the keys as they
// are go to the value pages, and the rotated queries / keys to q (compute type) and the key pages.
int launch_qk_conv_prepare(int dtype, const AttnShape& a, const AttnPrep& p, const float* qk, const StepRows& rows, void* q,
                           const PagedKV& kv, int T, cudaStream_t s);

// u [T, 2 * inner] fp32 (u | z rows of the input projection) -> uc [T, inner] fp32 and uc_ct (compute type): silu(conv(u) + b)
int launch_ssm_conv(int dtype, const kllm_seq_ssm& m, const float* uz, float* conv_state, const StepRows& rows, float* uc,
                    void* uc_ct, int T, cudaStream_t s);
// the scan over every entry from its sequence's state ([slots][inner][state] fp32, zeros at position 0):
// out[t] = y[t] * silu(z[t]) in the compute type
// Steps with long entries scan segments of an entry in parallel through `scratch` (ssm_scan_scratch_bytes(); 0: not needed).
size_t ssm_scan_scratch_bytes(const kllm_seq_ssm& m, int T, int n_entries, int max_count);
int launch_ssm_scan(int dtype, const kllm_seq_ssm& m, const float* uz, const float* uc, const float* low, float* state,
                    const StepRows& rows, const int32_t* ent_seq, int max_count, int T, float* scratch, void* out,
                    cudaStream_t s);

// proj [T, 2*kv_heads*dim + heads*vdim + heads + decay_rank + gate_rank] fp32 (q | k | v | beta | low-rank rows).
// delta_low: the low-rank rows in the compute type [T, decay_rank + gate_rank], the input of the product with w_low2 whose
// output is low2 [T, heads*dim + heads*vdim] fp32.
// delta_prepare: -> prep [T, delta_prep_row()] fp32: q | k (unit vectors, q scaled) | v | decay [heads*dim] |
// gate [heads*vdim] | beta [heads] (padded to a multiple of 4 floats)
__host__ __device__ inline int delta_prep_row(const kllm_seq_delta& m) {
  return (2 * m.kv_heads * m.dim + 2 * m.heads * m.vdim + m.heads * m.dim + m.heads + 3) & ~3;
}
int launch_delta_low(int dtype, const kllm_seq_delta& m, const float* proj, void* low, int T, cudaStream_t s);
int launch_delta_prepare(const kllm_seq_delta& m, const float* proj, const float* low2, float* conv_state, const StepRows& rows,
                         float* prep, int T, cudaStream_t s);
// the recurrence of every entry from its sequence's state ([slots][heads][dim][vdim] fp32); o [T, heads*vdim] fp32
// Steps with long entries walk segments of an entry in parallel through `scratch` (delta_rule_scratch_bytes(); 0: not needed).
size_t delta_rule_scratch_bytes(const kllm_seq_delta& m, int T, int n_entries, int max_count);
int launch_delta_rule(const kllm_seq_delta& m, const float* prep, float* state, const StepRows& rows, const int32_t* ent_seq,
                      int max_count, int T, float* scratch, float* o, cudaStream_t s);
// out[t, h] = o[t, h] / rms(o[t, h]) * norm_w * gate[t, h] in the compute type
int launch_delta_out(int dtype, const kllm_seq_delta& m, const float* o, const float* prep, float eps, void* out, int T,
                     cudaStream_t s);

// ---- seq_ssd.cu: state-space duality (one decay per head and token, a matrix state per head) ---------------------------
// proj [T, ssd_proj_row()] fp32: z | x | B | C | dt rows of the input projection.
__host__ __device__ inline int ssd_inner(const kllm_seq_ssd& m) { return m.heads * m.vdim; }
__host__ __device__ inline int ssd_conv_channels(const kllm_seq_ssd& m) { return m.heads * m.vdim + 2 * m.groups * m.state; }
__host__ __device__ inline int ssd_proj_row(const kllm_seq_ssd& m) { return 2 * m.heads * m.vdim + 2 * m.groups * m.state + m.heads; }
// xbc [T, ssd_conv_channels()] fp32 = silu(conv(x | B | C) + b); conv_state [slots][taps - 1][channels]
int launch_ssd_conv(const kllm_seq_ssd& m, const float* proj, float* conv_state, const StepRows& rows, float* xbc, int T,
                    cudaStream_t s);
// the recurrence of every entry from its sequence's state ([slots][heads][vdim][state] fp32, zeros at position 0):
// y [T, inner] fp32 (the skip d x included, ungated)
// Steps with long entries walk segments of an entry in parallel through `scratch` (ssd_scan_scratch_bytes(); 0: not needed).
size_t ssd_scan_scratch_bytes(const kllm_seq_ssd& m, int T, int n_entries, int max_count);
int launch_ssd_scan(const kllm_seq_ssd& m, const float* proj, const float* xbc, float* state, const StepRows& rows,
                    const int32_t* ent_seq, int max_count, int T, float* scratch, float* y, cudaStream_t s);
// out[t] = group-wise RMS norm of y[t] * silu(z[t]) times out_norm_w, in the compute type
int launch_ssd_out(int dtype, const kllm_seq_ssd& m, const float* y, const float* proj, float eps, void* out, int T,
                   cudaStream_t s);

// ---- seq_gemm.cu --------------------------------------------------------------------------------------------------
// out[T, N] (fp32) = a[T, K] . w[N, K]^T, a and w in the compute type, fp32 accumulation.
int gemm(int dtype, const void* a, const void* w, float* out, int T, int K, int N, cudaStream_t s);
// != 0 when a bounded wait inside a tensor-core product ran out since the last call (checked after a step's sync)
int gemm_take_error();
// Grouped form for the routed experts: block b (of `block` rows) multiplies rows a[row_of(b, i)] with the weights of
// expert block_expert[b]; see seq_gemm.cu.
struct GroupedArgs {
  const void* a;            // [*, K]
  const void* w;            // [experts][N][K]
  const int32_t* sorted_pair;   // [n_blocks * block] pair index or -1
  const int32_t* block_expert;  // [n_blocks] expert or -1
  int a_row_div;            // row of `a` for pair p is p / a_row_div (gate_up: top; down: 1)
  int n_blocks, block, K, N;
  // epilogue: 0 = out[pair, n] = acc (fp32);  1 = out[pair, f] = gated_act(acc_gate, acc_up) in the compute type (the
  // weights hold ff gate rows, then ff up rows; N = ff);  2 = out[pair, f] = max(acc, 0)^2 in the compute type
  int epilogue;
  GatedAct act;             // epilogue 1
  void* out;
  // tensor-core form (bf16): `a` is already in sorted order [n_blocks * block, K] and epilogue 1 writes its result in
  // sorted order too; `experts` sizes the weight map
  int sorted_layout;
  int experts;
};
int gemm_grouped(int dtype, const GroupedArgs& g, cudaStream_t s);
// bf16 only: can the grouped products of an expert layer (K = width, then K = ff) run on the tensor cores?
bool grouped_tensor_core_usable(int dtype, int width, int ff);
// hs[i] = a[sorted_pair[i] / div] (zero rows where sorted_pair[i] < 0), bf16, K % 8 == 0
int gather_rows_bf16(const void* a, const int32_t* sorted_pair, int div, void* out, int rows, int K, cudaStream_t s);

inline int cuda_rc(cudaError_t e) { return static_cast<int>(e); }
}  // namespace seq
}  // namespace kllm
