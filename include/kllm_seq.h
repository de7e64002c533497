/* kllm_seq.h -- C-ABI of the sequence-batch engine of kuiperllama_b200 (sm_100a).
 *
 * The single-sequence decoder of kllm_b200.h runs one position of one sequence per step.  This engine runs a STEP
 * of several sequences at once: every entry of a step brings the next tokens of one sequence (a whole prompt, or one
 * decoded token), all tokens of the step go through the layers as one ragged batch (no padding), and the keys and
 * values of every sequence live in fixed-size pages of one pool that sequences take as they grow and give back when
 * they end.  The layer stack is described by data (kllm_seq_layer), not by a model class: pre/post layer norms around
 * a token mixer and around a feed-forward, a schedule that may run a span of layers several times with the same
 * weights (each run with a cache of its own), so other model families can be described with the same pieces.
 *
 * Numerics.  compute type KLLM_SEQ_F32: every product in true fp32.  KLLM_SEQ_BF16: matrix products read bf16 weights
 * and bf16 activations and accumulate in fp32; keys / values are cached in bf16.  In both, the residual stream, the
 * norms, attention scores and softmax weights, the router and all gates are fp32.
 *
 * Same conventions as kllm_b200.h: device pointers in the descriptor, return 0 = ok, > 0 cudaError_t, < 0 KLLM_E_*.
 */
#ifndef KLLM_SEQ_H_
#define KLLM_SEQ_H_
#include "kllm_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define KLLM_SEQ_F32 0
#define KLLM_SEQ_BF16 1

#define KLLM_SEQ_MIXER_ATTENTION 1 /* softmax attention over the sequence's cached keys */
#define KLLM_SEQ_MIXER_LATENT 2    /* softmax attention through a low-rank latent: only the latent and one rotated key part are cached */
#define KLLM_SEQ_MIXER_LINEAR 3    /* linear attention with a decayed matrix state per head (no cache, a recurrent state) */
#define KLLM_SEQ_MIXER_SSM 4       /* selective scan: short convolution, input-dependent step sizes, a diagonal state per channel */
#define KLLM_SEQ_MIXER_DELTA 5     /* gated delta rule: a matrix state per head, decayed per key channel and corrected towards each value */
#define KLLM_SEQ_MIXER_SSD 6       /* state-space duality: short convolution, one input-dependent decay per head, a matrix state per head */
#define KLLM_SEQ_FF_NONE 0
#define KLLM_SEQ_FF_MOE 1   /* routed experts (softmax or sigmoid router), optional gated shared expert */
#define KLLM_SEQ_FF_DENSE 2 /* down(act(up h)) */

#define KLLM_SEQ_NORM_LAYER 0 /* (v - mean) / sqrt(var + eps) * w + b */
#define KLLM_SEQ_NORM_RMS 1   /* v / sqrt(mean(v^2) + eps) * w */
#define KLLM_SEQ_NORM_NONE 2  /* v itself (w is not read): a sublayer that reads the residual stream as it is */

/* output gate of an attention (kllm_seq_attention.gate) */
#define KLLM_SEQ_GATE_NONE 0
#define KLLM_SEQ_GATE_HEAD 1    /* one sigmoid gate per (token, head): `heads` gate rows close w_in */
#define KLLM_SEQ_GATE_ELEMENT 2 /* one sigmoid gate per output element: heads * vdim gate rows close w_in */

/* norm of every query / key head (kllm_seq_attention.qk_norm) */
#define KLLM_SEQ_QKNORM_NONE 0
#define KLLM_SEQ_QKNORM_WEIGHTED 1 /* RMS norm over dim with q_norm_w / k_norm_w, before the rotation */
#define KLLM_SEQ_QKNORM_UNIT 2     /* x / sqrt(mean(x^2) + eps) without weights, after the rotation */

/* activations of a feed-forward's inner layer */
#define KLLM_SEQ_ACT_SWIGLU 0 /* silu(gate h) * (up h): the weights hold gate rows, then up rows */
#define KLLM_SEQ_ACT_RELU2 1  /* max(up h, 0)^2 */
#define KLLM_SEQ_ACT_XIELU 2  /* z > 0: a z^2 + z / 2;  z <= 0: b (exp(z) - 1 - z) + z / 2 */
#define KLLM_SEQ_ACT_RELU_GATE 3    /* max(gate h, 0) * (up h): gate rows, then up rows */
#define KLLM_SEQ_ACT_CLAMP_SWIGLU 4 /* g = min(gate h, limit), u = clamp(up h, -limit, limit): g * sigmoid(alpha g) * (u + 1) */

#define KLLM_SEQ_ROUTER_SOFTMAX 0 /* scores = softmax(z); weights = chosen scores / their sum * scale */
#define KLLM_SEQ_ROUTER_SIGMOID 1 /* scores = sigmoid(z); chosen by score + correction, inside the best groups; weights = score * scale */
#define KLLM_SEQ_ROUTER_TOP_SOFTMAX 2 /* the largest logits are chosen; weights = softmax over the chosen logits only, * scale */

#define KLLM_SEQ_ROPE_HALVES 0 /* coordinate i is rotated with coordinate i + dims / 2 */
#define KLLM_SEQ_ROPE_PAIRS 1  /* coordinate 2i is rotated with coordinate 2i + 1 */

typedef struct kllm_seq_norm {
  const float* w; /* [width] */
  const float* b; /* [width] or NULL */
  int32_t kind;   /* KLLM_SEQ_NORM_* */
} kllm_seq_norm;

typedef struct kllm_seq_attention {
  int32_t heads, kv_heads, dim, vdim; /* query heads, key/value heads, query-key size, value size per head */
  float scale;                        /* score = (q . k) * scale */
  float temp_coef;                    /* query temperature 1 + coef * ln(floor((pos + 1) / every) + 1) ... */
  int32_t temp_every;                 /* ... 0: none */
  int32_t qk_norm;                    /* KLLM_SEQ_QKNORM_*: norm over dim of each query / key head */
  int32_t gate;                       /* KLLM_SEQ_GATE_*: sigmoid output gate; its rows close w_in */
  const void* w_in;  /* [heads*dim + kv_heads*dim + kv_heads*vdim (+ gate rows), width]: q | k | v (| gate) rows, compute type
                        (differential: 2*heads*dim query rows and 2*kv_heads*dim key rows) */
  const float* q_norm_w; /* [dim] */
  const float* k_norm_w; /* [dim] */
  const void* w_out;     /* [width, heads*vdim], compute type */
  int32_t window;        /* position i sees j <= i with i - j < window or j < keep_first; 0: every earlier position */
  int32_t keep_first;    /* the first keep_first positions stay visible behind the window (at their true positions) */
  float softcap;         /* score <- softcap * tanh(score / softcap) after the scale; 0: none */
  const float* sink;     /* [heads]: exp(sink) joins the softmax denominator (no key, no value), or NULL */
  const float* in_bias;  /* [rows of w_in] fp32 added to the projection, or NULL */
  int32_t conv_taps;     /* > 1: a causal convolution over time on every query and key channel, right after the projection
                            (zeros before the sequence's start; the last conv_taps - 1 projected rows are state of the sequence) */
  const float* conv_w;   /* [heads*dim + kv_heads*dim][conv_taps] fp32, the last column weighs the current token
                            (NULL: no filter; with conv_taps == 1 it is one weight per channel) */
  int32_t rope_dims;     /* rotary positions on the first rope_dims coordinates of every query and key head; 0: none */
  float rope_base;       /* angle of pair i = position * rope_base^(-2 i / rope_dims) */
  int32_t rope_pairing;  /* KLLM_SEQ_ROPE_* */
  int32_t values_are_keys; /* the values are the keys as they are before the rotation: w_in has no value rows, vdim == dim */
  const float* rope_freq;  /* [rope_dims / 2] fp32: angle of pair i = position * rope_freq[i] (any frequency scaling is
                              folded into this table), or NULL: rope_base^(-2 i / rope_dims) */
  float rope_mag;          /* cos and sin are multiplied by it (the rotated coordinates grow by this factor); 0 means 1 */
  /* Differential attention (!= 0): every query head and every key head holds TWO maps of `dim` coordinates, laid out
   * head by head as [map 1 | map 2]; head norms and rotation act on each map; each map is a softmax attention of its
   * own over the head's values (a1, a2), and the head's output is o = a1 - diff_lambda * a2, then
   * o / sqrt(mean(o^2) + eps) * diff_out_scale over its vdim values. */
  int32_t differential;
  float diff_lambda, diff_out_scale;
} kllm_seq_attention;

/* Attention through a latent.  Queries: cq = RMSnorm(W_dq h), q = W_uq cq, per head [dim plain | rot_dim rotated].
 * Keys / values: W_dkv h = [kv_rank | rot_dim]; c = RMSnorm(first part) is the latent, the second part, rotated, is a key
 * part shared by all heads.  Per head k = [W_uk c | rotated part], v = W_uv c.  Only c and the rotated part are cached:
 * the engine scores with W_uk^T q against c and applies W_uv after the weighted sum of latents. */
typedef struct kllm_seq_latent {
  int32_t heads, dim, rot_dim, vdim, q_rank, kv_rank;
  float scale;        /* score = (q . k) * scale */
  int32_t window;     /* position i sees j with 0 <= i - j < window; 0: all earlier positions */
  int32_t rope_dims;  /* rotary positions on the first rope_dims coordinates of the rotated part, coordinate i paired with i + rope_dims / 2 */
  float rope_base;    /* angle = position * rope_base^(-2 i / rope_dims) */
  const void* w_in;   /* [q_rank + kv_rank + rot_dim + heads, width]: W_dq | W_dkv | gate rows, compute type */
  const float* q_norm_w;  /* [q_rank] */
  const float* kv_norm_w; /* [kv_rank] */
  const void* w_uq;   /* [heads * (dim + rot_dim), q_rank] */
  const void* w_uk;   /* [heads * dim, kv_rank] */
  const void* w_uv;   /* [heads * vdim, kv_rank] */
  const float* sink;  /* [heads]: exp(sink) joins the softmax denominator (no key, no value), or NULL */
  const void* w_out;  /* [width, heads * vdim] */
} kllm_seq_latent;

/* Linear attention: q, k, v = silu(W h); per head S <- decay * S + k v^T, o = S^T q; the heads together are RMS-normed,
 * multiplied by sigmoid(W_g h) and projected.  S [dim, vdim] per head is fp32 state of the sequence. */
typedef struct kllm_seq_linear {
  int32_t heads, dim, vdim;
  const float* decay;      /* [heads], device */
  const void* w_in;        /* [2 * heads * dim + 2 * heads * vdim, width]: q | k | v | gate rows */
  const float* out_norm_w; /* [heads * vdim] */
  const void* w_out;       /* [width, heads * vdim] */
} kllm_seq_linear;

/* Selective scan.  W_in h = [u | z] (inner each); u <- silu(conv(u) + conv_b); W_x u = [low: dt_rank | B: state | C: state];
 * step d = softplus(W_dt low + dt_b) per channel; per channel c and state n: S <- exp(d_c a[c, n]) S + d_c u_c B_n;
 * y_c = sum_n S[c, n] C_n + D_c u_c; out = W_out (y * silu(z)).  S and the last conv_taps - 1 rows of u are fp32 state. */
typedef struct kllm_seq_ssm {
  int32_t inner, state, dt_rank, conv_taps;
  const void* w_in;     /* [2 * inner, width]: u rows, then z rows */
  const float* conv_w;  /* [inner][conv_taps] fp32, the last column weighs the current token */
  const float* conv_b;  /* [inner] or NULL */
  const void* w_x;      /* [dt_rank + 2 * state, inner] */
  const float* w_dt;    /* [inner, dt_rank] fp32 */
  const float* dt_b;    /* [inner] */
  const float* a;       /* [inner, state] fp32: the rates, already negative (-exp(A_log)) */
  const float* d;       /* [inner] */
  const void* w_out;    /* [width, inner] */
} kllm_seq_ssm;

/* Gated delta rule.  q, k (kv_heads x dim) and v (heads x vdim) = silu(conv(W h)); q, k <- unit vectors per head
 * (x / sqrt(sum x^2 + 1e-6)), q *= dim^-1/2; beta = sigmoid(W_b h) per head; decay g = exp(-rate_h * softplus(W_a2 (W_a1 h) +
 * dt_bias)) per head and key channel.  Per head: S <- g * S (rows); u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
 * o / rms(o) * out_norm_w * sigmoid(W_g2 (W_g1 h)), then W_out.  S [dim, vdim] per head and the last conv_taps - 1
 * projected rows are fp32 state.  Head h reads q / k head h / (heads / kv_heads). */
typedef struct kllm_seq_delta {
  int32_t heads, kv_heads, dim, vdim, conv_taps, decay_rank, gate_rank;
  const void* w_in;        /* [2 * kv_heads*dim + heads*vdim + heads + decay_rank + gate_rank, width]: q | k | v | beta | a1 | g1 rows */
  const float* conv_w;     /* [2 * kv_heads*dim + heads*vdim][conv_taps] fp32 */
  const void* w_low2;      /* [heads*dim + heads*vdim, decay_rank + gate_rank], compute type: the two second low-rank
                              projections as one product, W_a2 in the upper left block, W_g2 in the lower right, zeros elsewhere */
  const float* dt_bias;    /* [heads*dim] */
  const float* rate;       /* [heads] fp32: exp(A_log) */
  const float* out_norm_w; /* [vdim] */
  const void* w_out;       /* [width, heads*vdim] */
} kllm_seq_delta;

/* State-space duality (a selective scan whose decay is ONE number per head and token).  inner = heads * vdim.
 * W_in h = [z: inner | x: inner | B: groups*state | C: groups*state | dt: heads]; x, B and C together pass a causal
 * convolution per channel and SiLU; dt <- softplus(dt + dt_bias) (no clamp).  Head h reads B, C of group h / (heads / groups):
 * S <- exp(a_h dt) S + dt B x^T (S is state x vdim), y = S^T C + d_h x.  Then y * silu(z), an RMS norm in norm_groups
 * equal parts of inner (each part by its own root mean square) times out_norm_w, and W_out.  S and the last
 * conv_taps - 1 inputs of the convolution are fp32 state of the sequence. */
typedef struct kllm_seq_ssd {
  int32_t heads, vdim, state, groups, conv_taps, norm_groups;
  const void* w_in;        /* [2 * inner + 2 * groups * state + heads, width] */
  const float* conv_w;     /* [inner + 2 * groups * state][conv_taps] fp32, the last column weighs the current token */
  const float* conv_b;     /* [inner + 2 * groups * state] or NULL */
  const float* dt_bias;    /* [heads] */
  const float* a;          /* [heads] fp32: the rates, already negative (-exp(A_log)) */
  const float* d;          /* [heads] */
  const float* out_norm_w; /* [inner] */
  const void* w_out;       /* [width, inner] */
} kllm_seq_ssd;

typedef struct kllm_seq_dense {
  int32_t ff, act;    /* inner size; KLLM_SEQ_ACT_* (XIELU, RELU2, or RELU_GATE: then `up` holds ff gate rows followed by ff up rows) */
  float act_a, act_b; /* the two coefficients of KLLM_SEQ_ACT_XIELU */
  const void* up;     /* [ff, width] */
  const void* down;   /* [width, ff] */
} kllm_seq_dense;

typedef struct kllm_seq_moe {
  int32_t experts, top, ff; /* routed experts, chosen per token, inner size of a routed expert */
  float router_scale;       /* see KLLM_SEQ_ROUTER_* */
  const float* w_router;    /* [experts, width] fp32 */
  const void* gate_up;      /* [experts][2*ff][width]: gate rows, then up rows; compute type */
  const void* down;         /* [experts][width][ff] */
  int32_t shared_ff;        /* 0: no shared expert */
  const void* shared_gate_up; /* [2*shared_ff][width] */
  const void* shared_down;    /* [width][shared_ff] */
  const float* w_shared_gate; /* [width] fp32: the shared expert's output is scaled by sigmoid(w . h); NULL: by 1 */
  int32_t router_kind;        /* KLLM_SEQ_ROUTER_* */
  const float* correction;    /* [experts] added to the scores for the choice only (sigmoid router), or NULL */
  int32_t groups, groups_keep; /* sigmoid router: experts form `groups` equal groups of neighbours, a group scores the sum
                                  of its two largest choice scores, and only the best groups_keep groups can be chosen; 0: no groups */
  int32_t act;                /* KLLM_SEQ_ACT_SWIGLU / CLAMP_SWIGLU, or KLLM_SEQ_ACT_RELU2 (then gate_up holds [experts][ff][width]) */
  const float* router_bias;   /* [experts] fp32 added to the router's logits, or NULL */
  float act_limit, act_alpha; /* KLLM_SEQ_ACT_CLAMP_SWIGLU: the routed experts' clamp and the sigmoid's slope */
  float shared_act_limit;     /* the shared expert's clamp (same activation and slope) */
} kllm_seq_moe;

typedef struct kllm_seq_layer {
  int32_t mixer_kind; /* KLLM_SEQ_MIXER_* */
  int32_t ff_kind;    /* KLLM_SEQ_FF_* */
  /* x += post_mixer(mixer(pre_mixer(x)));  x += post_ff(ff(pre_ff(x)));  a pre-norm of kind KLLM_SEQ_NORM_NONE hands x
   * itself to the sublayer */
  kllm_seq_norm pre_mixer, post_mixer, pre_ff, post_ff;
  kllm_seq_attention attn;
  kllm_seq_moe moe;
  /* A norm without weights (w == NULL) after a sublayer means none: x += sublayer(...). */
  /* token shift: the mixer reads h + (h_prev - h) * shift instead of h = pre_mixer(x), h_prev the previous token's h
   * (zeros before the first token; the last h of a sequence is part of its state).  [width] fp32 or NULL */
  const float* shift;
  kllm_seq_latent latent;
  kllm_seq_linear linear;
  kllm_seq_dense dense;
  kllm_seq_ssm ssm;
  kllm_seq_delta delta;
  /* A second mixer of another kind beside the first (0: none): both read the same input and the mixer's output is
   * mixer_scale * first + mixer2_scale * second (the scales are read only when there is a second mixer). */
  int32_t mixer2_kind;
  float mixer_scale, mixer2_scale;
  /* != 0: the feed-forward reads the mixer's input too (pre_mixer's output; pre_ff is not used) and
   * x += mixer(...) + ff(...) in one step */
  int32_t parallel_ff;
  kllm_seq_ssd ssd;
  /* RMS norms over the model width on each mixer's own output, before the mixers' weighted sum (w == NULL: none) */
  kllm_seq_norm mixer_out_norm, mixer2_out_norm;
} kllm_seq_layer;

typedef struct kllm_seq_desc {
  int32_t dtype; /* KLLM_SEQ_F32 / KLLM_SEQ_BF16 */
  int32_t width, vocab;
  float norm_eps;
  int32_t n_layers;
  const kllm_seq_layer* layers;
  /* the order in which layers run: run r executes layer run_layer[r] with cache r; run_add[r] >= 0 adds row
   * run_add[r] of `run_vectors` ([*, width] fp32) to the residual stream right before it */
  int32_t n_runs;
  const int32_t* run_layer;
  const int32_t* run_add;
  const float* run_vectors;
  const void* embed; /* [vocab, width] compute type */
  kllm_seq_norm final_norm;
  const void* head;  /* [vocab, width] compute type */
  /* cache geometry */
  int32_t max_tokens; /* tokens all live sequences may hold together */
  int32_t max_seqs;   /* live sequences */
  int32_t page_tokens; /* tokens per page; 0: the engine's default */
  kllm_seq_norm embed_norm;  /* applied to the embedding rows (w == NULL: none) */
  const int32_t* run_embed;  /* [n_runs] or NULL: != 0 adds the embedding output (after embed_norm) to the residual stream
                                before the run, ahead of run_add's vector */
  float logit_scale;         /* logits = head(...) * logit_scale; 0 means 1 */
  float embed_scale;         /* the embedding rows are multiplied by it (before embed_norm); 0 means 1 */
  float logit_softcap;       /* logits <- cap * tanh(logits / cap), after logit_scale; 0: none */
} kllm_seq_desc;

typedef struct kllm_seq_engine kllm_seq_engine;

int kllm_seq_create(const kllm_seq_desc* desc, void* stream, kllm_seq_engine** out);
void kllm_seq_destroy(kllm_seq_engine* eng);

/* Sequences: open returns a slot; close gives its pages back to the pool. */
int kllm_seq_open(kllm_seq_engine* eng, int32_t* seq_out);
int kllm_seq_close(kllm_seq_engine* eng, int32_t seq);
int kllm_seq_length(const kllm_seq_engine* eng, int32_t seq);
int kllm_seq_free_pages(const kllm_seq_engine* eng);

/* One step.  Entry e appends counts[e] tokens (tokens_host, concatenated in entry order) to sequence seqs[e].
 * want_host lists the rows (indices into the concatenated tokens) whose logits are wanted; they are written to
 * logits_host [n_want, vocab] (fp32) and, when argmax_host is given, their greedy ids to argmax_host [n_want].
 * Blocking: returns after the results are in host memory. */
int kllm_seq_step(kllm_seq_engine* eng, int32_t n_entries, const int32_t* seqs, const int32_t* counts,
                  const int32_t* tokens_host, int32_t n_want, const int32_t* want_host, float* logits_host,
                  int32_t* argmax_host);

/* Diagnostics: the next step also copies the residual stream after every layer run to host memory
 * [n_runs, tokens of the step, width]; fusions across layer runs are switched off for that step. */
int kllm_seq_trace_residual(kllm_seq_engine* eng, float* residual_host);
/* Measurement aid: the next step records an event after each of its phases and writes the device time spent in every
 * phase class, in milliseconds, to phase_ms[KLLM_SEQ_PHASES] (summed over the layer runs). */
#define KLLM_SEQ_PHASE_NORM 0       /* embedding rows, residual + norm kernels, token shift */
#define KLLM_SEQ_PHASE_IN_PROJ 1    /* q | k | v | gate product (latent: the down-projections) */
#define KLLM_SEQ_PHASE_QK_PREPARE 2 /* head norms, temperature, rotation, cache scatter, gates; latent: + query up-projection and key absorption */
#define KLLM_SEQ_PHASE_ATTENTION 3  /* paged attention + merge of the key splits; linear attention; latent: + value expansion */
#define KLLM_SEQ_PHASE_OUT_PROJ 4
#define KLLM_SEQ_PHASE_ROUTER 5     /* residual + norms around the router and the router itself (one kernel) */
#define KLLM_SEQ_PHASE_EXPERTS 6    /* routed experts */
#define KLLM_SEQ_PHASE_SHARED 7     /* shared expert */
#define KLLM_SEQ_PHASE_HEAD 8       /* final norm of the wanted rows, classifier, argmax, copies */
#define KLLM_SEQ_PHASES 9
int kllm_seq_profile(kllm_seq_engine* eng, float* phase_ms);
/* kernel launches of the last step */
int kllm_seq_last_launches(const kllm_seq_engine* eng);

/* The engine's token-block product on its own: out[T, N] (fp32) = a[T, K] . w[N, K]^T with a and w in the compute
 * type `dtype` (device pointers).  Picks the kernel the engine would pick for this shape. */
int kllm_seq_gemm(int32_t dtype, const void* a, const void* w, float* out, int32_t n_tokens, int32_t in_dim,
                  int32_t out_dim, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KLLM_SEQ_H_ */
