// The sequence-batch engine behind include/kllm_seq.h: slot and page management of the key/value pool, and the step
// function that runs one ragged batch of tokens through the described layer stack.
//
// Cache.  One pool of pages per layer run; a page holds `page_tokens` tokens of one sequence ([token][kv_head][dim]
// keys, [token][kv_head][vdim] values, in the compute type).  All runs share ONE page numbering: a sequence that
// owns page p owns it in every run's pool, so there is a single page table [slot][i] and a single free list.  A
// sequence takes pages as it grows (lowest free number first, so freed pages are the next to be used again) and
// returns them at close.  The table rows of the step's sequences are copied to the device before the kernels run.
//
// State.  Beside the pages, every layer run owns per-slot recurrent state in fp32: the last mixer input of a layer with a
// token shift, the matrix state of linear attention, of the delta rule and of the duality mixer, the diagonal state of
// the selective scan, and the last taps - 1 inputs of every short convolution.  A sequence of length 0 reads zeros instead of its slot's
// memory, so slots are reused without clearing.  A run of attention through a latent keeps one row per token in its pool
// (latent | rotated key part); its values are the head of that row.
//
// Step.  Host work: validate, take pages, fill the per-token / per-entry index arrays in pinned memory, one
// host->device copy.  Device work, per layer run:
//     resid_norm   what comes ahead of the mixer: (x += embedding output) (x += run vector)  h = N_pre(x), and the token
//                  shift -- inside this kernel when every entry is one token, else by token_shift on the fp32 rows
//     mixer        attention:  gemm (q | k | v | gate rows), qk_prepare (RMS norms, temperature, scatter of k / v into the
//                              pages, gates), attention (causal, paged, keys split over CTAs; merge applies the gate)
//                  latent:     gemm (query and key/value down-projections, gate rows), latent_prepare (norms, rotation,
//                              cache row, gates), gemm (query up-projection); then either the absorbed form -- absorb,
//                              paged attention over the latents with window and sink, merge, value expansion -- or, for
//                              bf16 prompts that start their sequences, per-head keys and values of the step's own
//                              latents (two products) and the tensor-core attention
//                  linear:     gemm (q | k | v | gate rows), the decayed-state recurrence (one kernel for short entries,
//                              chunk sums / scan / chunk outputs for long ones), output norm and gate
//                  attention behind a filter (values = keys): gemm (q | k rows), qk_conv_prepare (bias, short convolution,
//                              keys as they are into the value pages, rotation, queries / keys out), attention with window,
//                              kept first tokens, capped scores and sink
//                  scan:       gemm (u | z rows), ssm_conv (filter + SiLU), gemm (low-rank step | B | C), ssm_scan (one kernel,
//                              or scan / carry / finish over segments of long entries)
//                  delta rule: gemm (q | k | v | beta | low-rank rows), delta_low + gemm (second low-rank products),
//                              delta_prepare (filters, unit vectors, decays, gates), delta_rule (one kernel, or two passes
//                              over segments with a carry between them), delta_out (per-head norm and gate)
//                  duality:    gemm (z | x | B | C | dt rows), ssd_conv (filter + SiLU), ssd_scan (one decay per head and
//                              token; one kernel, or scan / carry / finish over segments of long entries), ssd_out (gate,
//                              RMS norm in parts, weight)
//                  an attention may also rotate its queries and keys (frequencies from a table), norm them after the
//                  rotation, gate every output element, and run as a DIFFERENTIAL attention: two maps per head over the
//                  same values, joined by diff_merge
//                  a layer may run two mixers of different kinds on the same rows; their outputs join x with a weight each,
//                  each after an RMS norm of its own when the layer names one
//     gemm         output projection
//     resid_norm   x += N_post(y);  h = N_pre_ff(x);  router on h (softmax or sigmoid with groups): same kernel, the row
//                  is still in shared memory
//                  (a layer whose feed-forward reads the mixer's input skips this: the first norm kernel routes its row, the
//                  feed-forward runs on the same rows after the mixers, and ONE sum joins x at the end of the run)
//     feed-forward dense: gemm, activation, gemm
//                  experts, few tokens: pair kernels (weights streamed once per chosen expert; a shared expert rides
//                  along as one more pair per token); many tokens: pairs sorted by expert, two grouped products (SiLU-gate
//                  or squared-ReLU epilogue in the first); shared expert: gemm gate|up, silu_mul, gemm down
//     resid_norm   x += N_post_ff(ff output)   [+ what comes ahead of the next run's mixer, fused]
// then the final norm on the wanted rows only, the classifier product, the logit scale, argmax, and one device->host copy.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <new>
#include <tuple>
#include <vector>

#include "../../include/kllm_seq.h"
#include "seq_engine.h"

namespace kllm {
namespace seq {
int launch_argmax_rows(const float* logits, int32_t* out, int rows, int vocab, cudaStream_t s);
}
}  // namespace kllm

using namespace kllm;
using namespace kllm::seq;

namespace {
constexpr int kDefaultPage = 16;
constexpr int kGroupedMinTokens = 64;  // steps with at least this many tokens run the routed experts as grouped products
constexpr int kGroupBlock = 64;
constexpr int kSharedRideTokens = 4;   // steps of at most this many tokens run the shared expert inside the pair kernels

inline NormW nw(const kllm_seq_norm& n) { return NormW{n.w, n.b, n.kind}; }
inline size_t elt(int dtype) { return dtype == KLLM_SEQ_BF16 ? 2 : 4; }

uint64_t g_buffer_generation = 0;  // bumped whenever a workspace moves: captured graphs hold the old addresses

struct DevBuf {
  void* p = nullptr;
  size_t cap = 0;
  int reserve(size_t bytes) {
    if (bytes <= cap) return 0;
    ++g_buffer_generation;
    if (p) cudaFree(p);
    p = nullptr;
    cap = 0;
    const size_t want = bytes + bytes / 4 + 256;
    const cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) return static_cast<int>(e);
    cap = want;
    return 0;
  }
  ~DevBuf() {
    if (p) cudaFree(p);
  }
};
}  // namespace

struct kllm_seq_engine {
  kllm_seq_desc d{};
  std::vector<kllm_seq_layer> layers;
  std::vector<int32_t> run_layer, run_add;
  cudaStream_t stream = nullptr;
  // cache
  int page = 0, n_pages = 0, table_stride = 0;
  std::vector<void*> k_pool, v_pool;  // per run (null for runs without a cache; a latent run has keys only)
  // recurrent state per run and slot: the last mixer input of layers with a token shift [max_seqs][width], and the
  // matrix state of linear attention [max_seqs][heads][dim][vdim]; fp32.  A sequence's state is taken as zero while its
  // length is 0, so a slot that is used again needs no clearing.
  std::vector<float*> shift_state, linear_state;
  // more state per run and slot (fp32): the last taps - 1 inputs of the short convolutions of an attention, a selective
  // scan and a delta rule; the diagonal state of the scan [max_seqs][inner][state]; the delta rule's [max_seqs][heads][dim][vdim]
  std::vector<float*> attn_conv, ssm_conv, ssm_state, delta_conv, delta_state;
  // the duality mixer's convolution history [max_seqs][taps - 1][channels] and state [max_seqs][heads][vdim][state]
  std::vector<float*> ssd_conv, ssd_state;
  int32_t* table_dev = nullptr;       // [max_seqs][table_stride]
  std::vector<int32_t> table_host;
  std::vector<int32_t> free_pages;    // kept sorted descending: back() is the lowest number
  struct Slot {
    bool live = false;
    int len = 0;
    int pages = 0;
  };
  std::vector<Slot> slots;
  // per-step staging
  int32_t* pinned = nullptr;
  size_t pinned_cap = 0;
  DevBuf idx, x, h, proj, q, gates, att, y, y2, ws, top_idx, top_w, sgate, inter, pairs_out, sort, sorted_a, sorted_inter, hw, logits, amax;
  DevBuf lat_c, lat_kr, lat_kp, lat_vp, lat_q, lat_k, lat_v;  // a prompt step's latents expanded into per-head keys / values
  DevBuf x0, hn, qf, qa, ol;  // embedding output; fp32 normed rows ahead of a token shift; latent / linear attention scratch
  DevBuf y3, y4;              // outputs of a second mixer and of a feed-forward that runs beside the mixer
  DevBuf rec_a, rec_b, rec_c; // fp32 scratch of the selective scan (filtered rows, low-rank rows) and the delta rule (prepared rows)
  float* logits_pinned = nullptr;
  size_t logits_pinned_cap = 0;
  float* trace_host = nullptr;
  int last_launches = 0;
  // decode steps (one token per entry) are captured once per shape and replayed: the kernels read tokens, positions
  // and page tables from fixed device buffers, so a graph stays valid until a workspace moves
  struct Graph {
    cudaGraphExec_t exec = nullptr;
    uint64_t generation = 0;
    int nodes = 0;
  };
  std::map<std::tuple<int, int, int, int>, Graph> graphs;
  bool own_stream = false;
  bool use_graphs = true;
  // per-phase device times of one step (kllm_seq_profile): an event after every phase, read after the step's sync
  float* prof_out = nullptr;
  std::vector<cudaEvent_t> prof_events;
  std::vector<int> prof_phase;
  size_t prof_used = 0;
  void mark(int phase) {
    if (!prof_out) return;
    if (prof_used == prof_events.size()) {
      cudaEvent_t ev;
      if (cudaEventCreate(&ev) != cudaSuccess) return;
      prof_events.push_back(ev);
    }
    cudaEventRecord(prof_events[prof_used++], stream);
    prof_phase.push_back(phase);
  }
  // limits over the layers
  int max_proj = 0, max_q = 0, max_att = 0, max_gates = 0, max_ws_heads = 0, max_top = 0, max_ff = 0, max_sff = 0;
  int max_qf = 0, max_qa = 0, max_ol = 0, max_rec_a = 0, max_rec_b = 0, max_rec_c = 0;
  bool any_mixer2 = false, any_parallel_ff = false;
  bool any_shift = false, any_run_embed = false;
  std::vector<int32_t> run_embed;

  ~kllm_seq_engine() {
    for (void* p : k_pool) if (p) cudaFree(p);
    for (void* p : v_pool) if (p) cudaFree(p);
    for (float* p : shift_state) if (p) cudaFree(p);
    for (float* p : linear_state) if (p) cudaFree(p);
    for (auto* v : {&attn_conv, &ssm_conv, &ssm_state, &delta_conv, &delta_state, &ssd_conv, &ssd_state})
      for (float* p : *v) if (p) cudaFree(p);
    if (table_dev) cudaFree(table_dev);
    if (pinned) cudaFreeHost(pinned);
    if (logits_pinned) cudaFreeHost(logits_pinned);
    for (cudaEvent_t ev : prof_events) cudaEventDestroy(ev);
    for (auto& g : graphs) if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
    if (own_stream && stream) cudaStreamDestroy(stream);
  }
};

// how many maps a head of this attention holds, and the shape its kernels see (heads and key heads count the maps)
static int attn_maps(const kllm_seq_attention& a) { return a.differential ? 2 : 1; }
static AttnShape attn_shape(const kllm_seq_attention& A) {
  const int maps = attn_maps(A);
  AttnShape s{};
  s.heads = A.heads * maps, s.kv_heads = A.kv_heads * maps, s.dim = A.dim, s.vdim = A.vdim, s.scale = A.scale;
  s.temp_coef = A.temp_coef, s.temp_every = A.temp_every, s.qk_norm = A.qk_norm, s.gate = A.gate, s.window = A.window;
  s.sink = A.sink, s.keep_first = A.keep_first, s.softcap = A.softcap, s.v_share = maps;
  s.no_merge = A.differential ? 1 : 0;  // the maps' key splits are joined by diff_merge
  return s;
}
static int attn_proj_rows(const kllm_seq_attention& A) {
  const AttnShape s = attn_shape(A);
  return s.heads * A.dim + s.kv_heads * A.dim + (A.values_are_keys ? 0 : A.kv_heads * A.vdim) + gate_floats(s);
}

static bool has_cache(int kind) { return kind == KLLM_SEQ_MIXER_ATTENTION || kind == KLLM_SEQ_MIXER_LATENT; }

static int validate_mixer(const kllm_seq_layer& L, int kind) {
  if (kind == KLLM_SEQ_MIXER_ATTENTION) {
    const kllm_seq_attention& a = L.attn;
    if (a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads || a.dim <= 0 || a.vdim <= 0 || !a.w_in || !a.w_out)
      return KLLM_E_INVALID;
    if (a.qk_norm == KLLM_SEQ_QKNORM_WEIGHTED && (!a.q_norm_w || !a.k_norm_w)) return KLLM_E_INVALID;
    if (a.qk_norm < 0 || a.qk_norm > KLLM_SEQ_QKNORM_UNIT || a.gate < 0 || a.gate > KLLM_SEQ_GATE_ELEMENT) return KLLM_E_INVALID;
    // the two maps of a differential head are joined without a sink; the filtered form has one map
    if (a.differential && (a.sink || a.values_are_keys)) return KLLM_E_UNSUPPORTED;
    if (a.vdim > 256 || a.dim > 512) return KLLM_E_UNSUPPORTED;
    if (a.window < 0 || a.keep_first < 0 || a.softcap < 0.f || a.conv_taps < 0 || a.rope_dims < 0 || a.rope_dims > a.dim ||
        (a.rope_dims & 1) || (a.rope_dims > 0 && a.rope_base <= 0.f))
      return KLLM_E_INVALID;
    if (a.values_are_keys && a.vdim != a.dim) return KLLM_E_INVALID;
    // the filtered, rotated form has its own preparation kernel: no head norms, temperature or gate there
    const bool prep2 = a.values_are_keys || a.conv_taps > 1 || a.conv_w || a.in_bias;
    if (prep2 && (!a.values_are_keys || a.qk_norm || a.gate || a.temp_every || a.rope_freq)) return KLLM_E_UNSUPPORTED;
  } else if (kind == KLLM_SEQ_MIXER_LATENT) {
    const kllm_seq_latent& a = L.latent;
    if (a.heads <= 0 || a.dim <= 0 || a.rot_dim < 0 || a.vdim <= 0 || a.q_rank <= 0 || a.kv_rank <= 0 || a.window < 0 ||
        a.rope_dims < 0 || a.rope_dims > a.rot_dim || (a.rope_dims & 1) || (a.rope_dims > 0 && a.rope_base <= 0.f) ||
        !a.w_in || !a.q_norm_w || !a.kv_norm_w || !a.w_uq || !a.w_uk || !a.w_uv || !a.w_out)
      return KLLM_E_INVALID;
    // the latent is the value of the paged attention kernel, latent + rotated part its key
    if (a.kv_rank > 256 || a.kv_rank + a.rot_dim > 512) return KLLM_E_UNSUPPORTED;
  } else if (kind == KLLM_SEQ_MIXER_LINEAR) {
    const kllm_seq_linear& a = L.linear;
    if (a.heads <= 0 || a.dim <= 0 || a.vdim <= 0 || !a.decay || !a.w_in || !a.out_norm_w || !a.w_out) return KLLM_E_INVALID;
    if (a.dim > 256) return KLLM_E_UNSUPPORTED;
  } else if (kind == KLLM_SEQ_MIXER_SSM) {
    const kllm_seq_ssm& a = L.ssm;
    if (a.inner <= 0 || a.state <= 0 || a.dt_rank <= 0 || a.conv_taps < 1 || !a.w_in ||
        !a.w_x || !a.w_dt || !a.dt_b || !a.a || !a.d || !a.w_out)
      return KLLM_E_INVALID;
    if (a.state > 128) return KLLM_E_UNSUPPORTED;
  } else if (kind == KLLM_SEQ_MIXER_DELTA) {
    const kllm_seq_delta& a = L.delta;
    if (a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads || a.dim <= 0 || a.vdim <= 0 || a.conv_taps < 1 ||
        a.decay_rank <= 0 || a.gate_rank <= 0 || !a.w_in || !a.w_low2 || !a.dt_bias ||
        !a.rate || !a.out_norm_w || !a.w_out)
      return KLLM_E_INVALID;
    if (a.dim > 256) return KLLM_E_UNSUPPORTED;
  } else if (kind == KLLM_SEQ_MIXER_SSD) {
    const kllm_seq_ssd& a = L.ssd;
    if (a.heads <= 0 || a.vdim <= 0 || a.state <= 0 || a.groups <= 0 || a.heads % a.groups || a.conv_taps < 1 ||
        a.norm_groups <= 0 || (a.heads * a.vdim) % a.norm_groups || !a.w_in || !a.conv_w || !a.dt_bias || !a.a || !a.d ||
        !a.out_norm_w || !a.w_out)
      return KLLM_E_INVALID;
    if (a.state > 512) return KLLM_E_UNSUPPORTED;
  } else {
    return KLLM_E_UNSUPPORTED;
  }
  return 0;
}

static int validate(const kllm_seq_desc* d) {
  if (!d || d->width <= 0 || d->vocab <= 0 || d->n_layers <= 0 || !d->layers || d->n_runs <= 0 || !d->run_layer ||
      !d->embed || !d->head || !d->final_norm.w || d->max_tokens <= 0 || d->max_seqs <= 0)
    return KLLM_E_INVALID;
  if (d->dtype != KLLM_SEQ_F32 && d->dtype != KLLM_SEQ_BF16) return KLLM_E_INVALID;
  for (int r = 0; r < d->n_runs; ++r) {
    if (d->run_layer[r] < 0 || d->run_layer[r] >= d->n_layers) return KLLM_E_INVALID;
    if (d->run_add && d->run_add[r] >= 0 && !d->run_vectors) return KLLM_E_INVALID;
  }
  for (int i = 0; i < d->n_layers; ++i) {
    const kllm_seq_layer& L = d->layers[i];
    if (!L.pre_mixer.w && L.pre_mixer.kind != KLLM_SEQ_NORM_NONE) return KLLM_E_INVALID;
    for (const kllm_seq_norm* n : {&L.mixer_out_norm, &L.mixer2_out_norm})
      if (n->w && n->kind != KLLM_SEQ_NORM_RMS) return KLLM_E_UNSUPPORTED;
    if (L.shift && L.pre_mixer.kind == KLLM_SEQ_NORM_NONE) return KLLM_E_UNSUPPORTED;
    if (int rc = validate_mixer(L, L.mixer_kind)) return rc;
    if (L.mixer2_kind != 0) {
      // the two mixers of a layer are of different kinds (a layer describes one mixer of each), and only one keeps pages
      if (L.mixer2_kind == L.mixer_kind || (has_cache(L.mixer_kind) && has_cache(L.mixer2_kind))) return KLLM_E_UNSUPPORTED;
      if (int rc = validate_mixer(L, L.mixer2_kind)) return rc;
    }
    if (L.parallel_ff && (L.shift || L.ff_kind == KLLM_SEQ_FF_NONE)) return KLLM_E_UNSUPPORTED;
    if (L.ff_kind == KLLM_SEQ_FF_MOE) {
      const kllm_seq_moe& m = L.moe;
      if (m.experts <= 0 || m.top <= 0 || m.top > m.experts || m.ff <= 0 || !m.w_router || !m.gate_up || !m.down ||
          (!L.pre_ff.w && !L.parallel_ff))  // the router reads a normed row
        return KLLM_E_INVALID;
      if (m.shared_ff > 0 && (!m.shared_gate_up || !m.shared_down)) return KLLM_E_INVALID;
      if (m.act != KLLM_SEQ_ACT_SWIGLU && m.act != KLLM_SEQ_ACT_CLAMP_SWIGLU && (m.act != KLLM_SEQ_ACT_RELU2 || m.shared_ff > 0))
        return KLLM_E_UNSUPPORTED;
      if (m.router_kind != KLLM_SEQ_ROUTER_SOFTMAX && m.router_kind != KLLM_SEQ_ROUTER_SIGMOID &&
          m.router_kind != KLLM_SEQ_ROUTER_TOP_SOFTMAX)
        return KLLM_E_UNSUPPORTED;
      if (m.groups < 0 || (m.groups > 0 && (m.experts % m.groups != 0 || m.groups_keep <= 0 || m.groups_keep > m.groups)))
        return KLLM_E_INVALID;
    } else if (L.ff_kind == KLLM_SEQ_FF_DENSE) {
      const kllm_seq_dense& f = L.dense;
      if (f.ff <= 0 || !f.up || !f.down || (!L.pre_ff.w && L.pre_ff.kind != KLLM_SEQ_NORM_NONE && !L.parallel_ff))
        return KLLM_E_INVALID;
      if (f.act != KLLM_SEQ_ACT_XIELU && f.act != KLLM_SEQ_ACT_RELU2 && f.act != KLLM_SEQ_ACT_RELU_GATE) return KLLM_E_UNSUPPORTED;
    } else if (L.ff_kind != KLLM_SEQ_FF_NONE) {
      return KLLM_E_UNSUPPORTED;
    }
  }
  return 0;
}

extern "C" int kllm_seq_create(const kllm_seq_desc* desc, void* stream, kllm_seq_engine** out) {
  if (!out) return KLLM_E_INVALID;
  *out = nullptr;
  if (int rc = validate(desc)) return rc;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) return KLLM_E_NODEVICE;
  kllm_seq_engine* e = new (std::nothrow) kllm_seq_engine();
  if (!e) return KLLM_E_STATE;
  e->d = *desc;
  e->layers.assign(desc->layers, desc->layers + desc->n_layers);
  e->run_layer.assign(desc->run_layer, desc->run_layer + desc->n_runs);
  e->run_add.assign(desc->n_runs, -1);
  if (desc->run_add) e->run_add.assign(desc->run_add, desc->run_add + desc->n_runs);
  e->d.layers = e->layers.data();
  e->d.run_layer = e->run_layer.data();
  e->d.run_add = e->run_add.data();
  e->run_embed.assign(desc->n_runs, 0);
  if (desc->run_embed) e->run_embed.assign(desc->run_embed, desc->run_embed + desc->n_runs);
  e->d.run_embed = e->run_embed.data();
  for (int32_t v : e->run_embed) e->any_run_embed = e->any_run_embed || v != 0;
  e->stream = static_cast<cudaStream_t>(stream);
  if (e->stream == nullptr) {  // a stream of its own: the legacy default stream cannot be captured
    if (cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess) {
      delete e;
      return KLLM_E_NODEVICE;
    }
    e->own_stream = true;
  }
  if (const char* g = getenv("KLLM_SEQ_GRAPHS")) e->use_graphs = g[0] != '0';
  e->page = desc->page_tokens > 0 ? desc->page_tokens : kDefaultPage;
  // every live sequence may leave its last page partly empty
  e->n_pages = (desc->max_tokens + e->page - 1) / e->page + desc->max_seqs;
  e->table_stride = (desc->max_tokens + e->page - 1) / e->page + 1;
  e->slots.resize(desc->max_seqs);
  e->table_host.assign(static_cast<size_t>(desc->max_seqs) * e->table_stride, 0);
  for (int p = e->n_pages - 1; p >= 0; --p) e->free_pages.push_back(p);
  const size_t es = elt(desc->dtype);
  for (int r = 0; r < desc->n_runs; ++r) {
    const kllm_seq_layer& L = e->layers[e->run_layer[r]];
    void *k = nullptr, *v = nullptr;
    float *sh = nullptr, *ls = nullptr, *ac = nullptr, *sc = nullptr, *ss = nullptr, *dc = nullptr, *ds = nullptr;
    float *dual_conv = nullptr, *dual_state = nullptr;
    const size_t tokens = static_cast<size_t>(e->n_pages) * e->page;
    const size_t slots = static_cast<size_t>(desc->max_seqs);
    bool ok = true;
    auto f32 = [&](float** p, size_t n) { return n == 0 || cudaMalloc(p, n * sizeof(float)) == cudaSuccess; };
    for (int kind : {L.mixer_kind, L.mixer2_kind}) {
      if (!ok) break;
      if (kind == KLLM_SEQ_MIXER_ATTENTION) {
        const kllm_seq_attention& a = L.attn;
        ok = cudaMalloc(&k, tokens * a.kv_heads * attn_maps(a) * a.dim * es) == cudaSuccess &&
             cudaMalloc(&v, tokens * a.kv_heads * a.vdim * es) == cudaSuccess &&
             f32(&ac, a.conv_taps > 1 ? slots * (a.conv_taps - 1) * (a.heads + a.kv_heads) * a.dim : 0);
      } else if (kind == KLLM_SEQ_MIXER_LATENT) {
        ok = cudaMalloc(&k, tokens * (L.latent.kv_rank + L.latent.rot_dim) * es) == cudaSuccess;
      } else if (kind == KLLM_SEQ_MIXER_LINEAR) {
        ok = f32(&ls, slots * L.linear.heads * L.linear.dim * L.linear.vdim);
      } else if (kind == KLLM_SEQ_MIXER_SSM) {
        ok = f32(&sc, slots * (L.ssm.conv_taps - 1) * L.ssm.inner) && f32(&ss, slots * L.ssm.inner * L.ssm.state);
      } else if (kind == KLLM_SEQ_MIXER_DELTA) {
        const kllm_seq_delta& a = L.delta;
        ok = f32(&dc, slots * (a.conv_taps - 1) * (2 * a.kv_heads * a.dim + a.heads * a.vdim)) &&
             f32(&ds, slots * a.heads * a.dim * a.vdim);
      } else if (kind == KLLM_SEQ_MIXER_SSD) {
        const kllm_seq_ssd& a = L.ssd;
        ok = f32(&dual_conv, slots * (a.conv_taps - 1) * ssd_conv_channels(a)) &&
             f32(&dual_state, slots * a.heads * a.vdim * a.state);
      }
    }
    if (ok && L.shift) ok = cudaMalloc(&sh, static_cast<size_t>(desc->max_seqs) * desc->width * sizeof(float)) == cudaSuccess;
    e->k_pool.push_back(k);
    e->v_pool.push_back(v);
    e->shift_state.push_back(sh);
    e->linear_state.push_back(ls);
    e->attn_conv.push_back(ac), e->ssm_conv.push_back(sc), e->ssm_state.push_back(ss);
    e->delta_conv.push_back(dc), e->delta_state.push_back(ds);
    e->ssd_conv.push_back(dual_conv), e->ssd_state.push_back(dual_state);
    if (!ok) {
      delete e;
      return static_cast<int>(cudaErrorMemoryAllocation);
    }
  }
  if (cudaMalloc(&e->table_dev, e->table_host.size() * sizeof(int32_t)) != cudaSuccess) {
    delete e;
    return static_cast<int>(cudaErrorMemoryAllocation);
  }
  cudaMemset(e->table_dev, 0, e->table_host.size() * sizeof(int32_t));
  for (const kllm_seq_layer& L : e->layers) {
    e->any_shift = e->any_shift || L.shift != nullptr;
    e->any_mixer2 = e->any_mixer2 || L.mixer2_kind != 0;
    e->any_parallel_ff = e->any_parallel_ff || L.parallel_ff != 0;
    for (int kind : {L.mixer_kind, L.mixer2_kind}) {
      if (kind == KLLM_SEQ_MIXER_ATTENTION) {
        const kllm_seq_attention& a = L.attn;
        e->max_proj = std::max(e->max_proj, attn_proj_rows(a));
        e->max_q = std::max(e->max_q, a.heads * attn_maps(a) * a.dim);
        e->max_att = std::max(e->max_att, a.heads * a.vdim);
        e->max_gates = std::max(e->max_gates, gate_floats(attn_shape(a)));
      } else if (kind == KLLM_SEQ_MIXER_LATENT) {
        const kllm_seq_latent& a = L.latent;
        e->max_proj = std::max(e->max_proj, a.q_rank + a.kv_rank + a.rot_dim + a.heads);
        e->max_q = std::max(e->max_q, a.q_rank);
        e->max_qf = std::max(e->max_qf, a.heads * (a.dim + a.rot_dim));
        e->max_qa = std::max(e->max_qa, a.heads * (a.kv_rank + a.rot_dim));
        e->max_ol = std::max(e->max_ol, a.heads * a.kv_rank);
        e->max_att = std::max(e->max_att, a.heads * a.vdim);
        e->max_gates = std::max(e->max_gates, a.heads);
      } else if (kind == KLLM_SEQ_MIXER_LINEAR) {
        const kllm_seq_linear& a = L.linear;
        e->max_proj = std::max(e->max_proj, 2 * a.heads * (a.dim + a.vdim));
        e->max_ol = std::max(e->max_ol, a.heads * a.vdim);
        e->max_att = std::max(e->max_att, a.heads * a.vdim);
      } else if (kind == KLLM_SEQ_MIXER_SSM) {
        const kllm_seq_ssm& a = L.ssm;
        e->max_proj = std::max(e->max_proj, 2 * a.inner);
        e->max_att = std::max(e->max_att, a.inner);
        e->max_rec_a = std::max(e->max_rec_a, a.inner);
        e->max_rec_b = std::max(e->max_rec_b, a.dt_rank + 2 * a.state);
      } else if (kind == KLLM_SEQ_MIXER_DELTA) {
        const kllm_seq_delta& a = L.delta;
        e->max_proj = std::max(e->max_proj, 2 * a.kv_heads * a.dim + a.heads * a.vdim + a.heads + a.decay_rank + a.gate_rank);
        e->max_att = std::max(e->max_att, a.heads * a.vdim);
        e->max_rec_a = std::max(e->max_rec_a, delta_prep_row(a));
        e->max_rec_b = std::max(e->max_rec_b, a.heads * a.vdim);
        e->max_rec_c = std::max(e->max_rec_c, a.heads * (a.dim + a.vdim));
        e->max_q = std::max(e->max_q, a.decay_rank + a.gate_rank);
      } else if (kind == KLLM_SEQ_MIXER_SSD) {
        const kllm_seq_ssd& a = L.ssd;
        e->max_proj = std::max(e->max_proj, ssd_proj_row(a));
        e->max_att = std::max(e->max_att, ssd_inner(a));
        e->max_rec_a = std::max(e->max_rec_a, ssd_conv_channels(a));
        e->max_rec_b = std::max(e->max_rec_b, ssd_inner(a));
      }
    }
    if (L.ff_kind == KLLM_SEQ_FF_DENSE) {
      e->max_proj = std::max(e->max_proj, (L.dense.act == KLLM_SEQ_ACT_RELU_GATE ? 2 : 1) * L.dense.ff);
      e->max_att = std::max(e->max_att, L.dense.ff);
    }
    if (L.ff_kind == KLLM_SEQ_FF_MOE) {
      e->max_top = std::max(e->max_top, L.moe.top);
      e->max_ff = std::max(e->max_ff, L.moe.top * L.moe.ff);
      e->max_sff = std::max(e->max_sff, L.moe.shared_ff);
    }
  }
  *out = e;
  return 0;
}

extern "C" void kllm_seq_destroy(kllm_seq_engine* eng) {
  if (!eng) return;
  cudaStreamSynchronize(eng->stream);
  delete eng;
}

extern "C" int kllm_seq_open(kllm_seq_engine* e, int32_t* seq_out) {
  if (!e || !seq_out) return KLLM_E_INVALID;
  for (size_t i = 0; i < e->slots.size(); ++i)
    if (!e->slots[i].live) {
      e->slots[i] = kllm_seq_engine::Slot{true, 0, 0};
      *seq_out = static_cast<int32_t>(i);
      return 0;
    }
  return KLLM_E_STATE;
}

extern "C" int kllm_seq_close(kllm_seq_engine* e, int32_t seq) {
  if (!e || seq < 0 || seq >= static_cast<int32_t>(e->slots.size()) || !e->slots[seq].live) return KLLM_E_INVALID;
  kllm_seq_engine::Slot& s = e->slots[seq];
  for (int i = 0; i < s.pages; ++i) e->free_pages.push_back(e->table_host[static_cast<size_t>(seq) * e->table_stride + i]);
  std::sort(e->free_pages.begin(), e->free_pages.end(), [](int a, int b) { return a > b; });
  s = kllm_seq_engine::Slot{};
  return 0;
}

extern "C" int kllm_seq_length(const kllm_seq_engine* e, int32_t seq) {
  if (!e || seq < 0 || seq >= static_cast<int32_t>(e->slots.size()) || !e->slots[seq].live) return KLLM_E_INVALID;
  return e->slots[seq].len;
}

extern "C" int kllm_seq_free_pages(const kllm_seq_engine* e) {
  return e ? static_cast<int>(e->free_pages.size()) : KLLM_E_INVALID;
}

extern "C" int kllm_seq_trace_residual(kllm_seq_engine* e, float* residual_host) {
  if (!e) return KLLM_E_INVALID;
  e->trace_host = residual_host;
  return 0;
}

extern "C" int kllm_seq_profile(kllm_seq_engine* e, float* phase_ms) {
  if (!e) return KLLM_E_INVALID;
  e->prof_out = phase_ms;
  return 0;
}

extern "C" int kllm_seq_last_launches(const kllm_seq_engine* e) { return e ? e->last_launches : KLLM_E_INVALID; }

#define RC(call)                  \
  do {                            \
    const int rc_ = (call);       \
    if (rc_ != 0) return rc_;     \
  } while (0)
#define CU(call)                                          \
  do {                                                    \
    const cudaError_t ce_ = (call);                       \
    if (ce_ != cudaSuccess) return static_cast<int>(ce_); \
  } while (0)

extern "C" int kllm_seq_step(kllm_seq_engine* e, int32_t n_entries, const int32_t* seqs, const int32_t* counts,
                             const int32_t* tokens_host, int32_t n_want, const int32_t* want_host, float* logits_host,
                             int32_t* argmax_host) {
  if (!e || n_entries <= 0 || !seqs || !counts || !tokens_host || n_want < 0 || (n_want > 0 && !want_host))
    return KLLM_E_INVALID;
  const kllm_seq_desc& d = e->d;
  const int W = d.width, dtype = d.dtype;
  const size_t es = elt(dtype);
  cudaStream_t st = e->stream;
  const uint64_t launches_before = launch_counter().load();

  // ---- host: validate, pages, index arrays ------------------------------------------------------------------------
  int T = 0, max_count = 0, max_ctx = 0, need_pages = 0;
  for (int i = 0; i < n_entries; ++i) {
    const int s = seqs[i];
    if (s < 0 || s >= static_cast<int>(e->slots.size()) || !e->slots[s].live || counts[i] <= 0) return KLLM_E_INVALID;
    for (int j = 0; j < i; ++j)
      if (seqs[j] == s) return KLLM_E_INVALID;  // one entry per sequence and step
    const int new_len = e->slots[s].len + counts[i];
    need_pages += (new_len + e->page - 1) / e->page - e->slots[s].pages;
    T += counts[i];
    max_count = std::max(max_count, counts[i]);
    max_ctx = std::max(max_ctx, new_len);
  }
  int live_tokens = 0;
  for (const auto& s : e->slots) live_tokens += s.live ? s.len : 0;
  if (live_tokens + T > d.max_tokens || need_pages > static_cast<int>(e->free_pages.size())) return KLLM_E_STATE;
  for (int i = 0; i < T; ++i)
    if (tokens_host[i] < 0 || tokens_host[i] >= d.vocab) return KLLM_E_INVALID;
  for (int i = 0; i < n_want; ++i)
    if (want_host[i] < 0 || want_host[i] >= T) return KLLM_E_INVALID;

  // layout of the index block (int32): tokens[T] tok_seq[T] tok_pos[T] ent_first[E] ent_count[E] ent_seq[E] ent_pos0[E]
  // want[n_want]
  const size_t n_idx = 3 * static_cast<size_t>(T) + 4 * static_cast<size_t>(n_entries) + static_cast<size_t>(n_want);
  if (n_idx > e->pinned_cap) {
    if (e->pinned) cudaFreeHost(e->pinned);
    e->pinned = nullptr;
    e->pinned_cap = 0;
    CU(cudaMallocHost(&e->pinned, (n_idx + n_idx / 2) * sizeof(int32_t)));
    e->pinned_cap = n_idx + n_idx / 2;
  }
  RC(e->idx.reserve(n_idx * sizeof(int32_t)));
  int32_t* hp = e->pinned;
  int32_t *h_tok = hp, *h_seq = hp + T, *h_pos = hp + 2 * T, *h_first = hp + 3 * T, *h_count = h_first + n_entries,
          *h_eseq = h_count + n_entries, *h_pos0 = h_eseq + n_entries, *h_want = h_pos0 + n_entries;
  std::memcpy(h_tok, tokens_host, static_cast<size_t>(T) * sizeof(int32_t));
  int at = 0;
  for (int i = 0; i < n_entries; ++i) {
    kllm_seq_engine::Slot& s = e->slots[seqs[i]];
    h_first[i] = at, h_count[i] = counts[i], h_eseq[i] = seqs[i], h_pos0[i] = s.len;
    for (int j = 0; j < counts[i]; ++j) h_seq[at + j] = seqs[i], h_pos[at + j] = s.len + j;
    at += counts[i];
    const int new_len = s.len + counts[i];
    const int pages = (new_len + e->page - 1) / e->page;
    int32_t* row = e->table_host.data() + static_cast<size_t>(seqs[i]) * e->table_stride;
    if (pages > e->table_stride) return KLLM_E_STATE;
    while (s.pages < pages) {
      row[s.pages++] = e->free_pages.back();
      e->free_pages.pop_back();
    }
    s.len = new_len;
    CU(cudaMemcpyAsync(e->table_dev + static_cast<size_t>(seqs[i]) * e->table_stride, row, pages * sizeof(int32_t),
                       cudaMemcpyHostToDevice, st));
  }
  if (n_want) std::memcpy(h_want, want_host, static_cast<size_t>(n_want) * sizeof(int32_t));
  // the table rows above are pageable host memory: the copies are staged by the driver before the call returns
  CU(cudaMemcpyAsync(e->idx.p, hp, n_idx * sizeof(int32_t), cudaMemcpyHostToDevice, st));
  const int32_t* d_tok = static_cast<const int32_t*>(e->idx.p);
  const int32_t *d_seq = d_tok + T, *d_pos = d_tok + 2 * T, *d_first = d_tok + 3 * T, *d_count = d_first + n_entries,
                *d_eseq = d_count + n_entries, *d_pos0 = d_eseq + n_entries, *d_want = d_pos0 + n_entries;

  // ---- workspaces ----------------------------------------------------------------------------------------------
  // keys of a row tile are split over CTAs when the step itself offers few tiles (decode, short prompts)
  int splits = 1;
  {
    const int tiles = (max_ctx + kAttnKeys - 1) / kAttnKeys;
    const int ctas = n_entries * ((max_count * 8 + kAttnRows - 1) / kAttnRows);
    if (ctas < 64) {
      const int want = std::max(1, std::min({tiles, 32, 128 / std::max(1, ctas)}));
      while (splits < want) splits *= 2;  // a power of two: few distinct launch shapes as a context grows
    }
  }
  // a layer with a window never has more key tiles in reach than the window spans: a function of `splits` and the
  // layer's constants only, so that captured decode steps stay keyed by `splits`
  auto window_splits = [&](int window) {
    if (window <= 0) return splits;
    int cap = 1;
    while (cap < window / kAttnKeys + 2) cap *= 2;
    return std::min(splits, cap);
  };
  const size_t Ts = static_cast<size_t>(T);
  RC(e->x.reserve(Ts * W * 4));
  RC(e->h.reserve(Ts * W * es));
  RC(e->proj.reserve(Ts * std::max({e->max_proj, 2 * e->max_sff, W}) * 4));
  RC(e->q.reserve(Ts * std::max(1, e->max_q) * es));
  RC(e->gates.reserve(Ts * std::max(1, e->max_gates) * 4));
  RC(e->att.reserve(Ts * std::max(e->max_att, e->max_sff) * es));
  RC(e->y.reserve(Ts * W * 4));
  RC(e->y2.reserve(Ts * W * 4));
  if (e->any_run_embed) RC(e->x0.reserve(Ts * W * 4));
  if (e->any_shift) RC(e->hn.reserve(Ts * W * 4));
  if (e->max_qf > 0) RC(e->qf.reserve(Ts * e->max_qf * 4));
  if (e->max_qa > 0) RC(e->qa.reserve(Ts * e->max_qa * 4));
  if (e->max_ol > 0) RC(e->ol.reserve(Ts * e->max_ol * 4));
  if (e->any_mixer2) RC(e->y3.reserve(Ts * W * 4));
  if (e->any_parallel_ff) RC(e->y4.reserve(Ts * W * 4));
  if (e->max_rec_a > 0) RC(e->rec_a.reserve(Ts * e->max_rec_a * 4));
  if (e->max_rec_b > 0) RC(e->rec_b.reserve(Ts * e->max_rec_b * 4));
  if (e->max_rec_c > 0) RC(e->rec_c.reserve(Ts * e->max_rec_c * 4));
  size_t ws_bytes = 0;
  for (const kllm_seq_layer& L : e->layers)
    for (int kind : {L.mixer_kind, L.mixer2_kind}) {
      AttnShape a{};
      if (kind == KLLM_SEQ_MIXER_ATTENTION) a.heads = L.attn.heads * attn_maps(L.attn), a.vdim = L.attn.vdim;
      else if (kind == KLLM_SEQ_MIXER_LATENT) a.heads = L.latent.heads, a.vdim = L.latent.kv_rank;
      else continue;
      ws_bytes = std::max(ws_bytes, attention_workspace_bytes(a, T, splits));
    }
  for (const kllm_seq_layer& L : e->layers)  // the chunk sums of linear attention share the attention workspace
    if (L.mixer_kind == KLLM_SEQ_MIXER_LINEAR || L.mixer2_kind == KLLM_SEQ_MIXER_LINEAR)
      ws_bytes = std::max(ws_bytes, linear_attention_scratch_bytes(L.linear.heads, L.linear.dim, L.linear.vdim, T, n_entries, max_count));
  for (const kllm_seq_layer& L : e->layers)  // and so do the segments of the selective scan
    if (L.mixer_kind == KLLM_SEQ_MIXER_SSM || L.mixer2_kind == KLLM_SEQ_MIXER_SSM)
      ws_bytes = std::max(ws_bytes, ssm_scan_scratch_bytes(L.ssm, T, n_entries, max_count));
  for (const kllm_seq_layer& L : e->layers)
    if (L.mixer_kind == KLLM_SEQ_MIXER_DELTA || L.mixer2_kind == KLLM_SEQ_MIXER_DELTA)
      ws_bytes = std::max(ws_bytes, delta_rule_scratch_bytes(L.delta, T, n_entries, max_count));
  for (const kllm_seq_layer& L : e->layers)
    if (L.mixer_kind == KLLM_SEQ_MIXER_SSD || L.mixer2_kind == KLLM_SEQ_MIXER_SSD)
      ws_bytes = std::max(ws_bytes, ssd_scan_scratch_bytes(L.ssd, T, n_entries, max_count));
  RC(e->ws.reserve(ws_bytes));
  const bool grouped = T >= kGroupedMinTokens;
  if (e->max_top > 0) {
    RC(e->top_idx.reserve(Ts * e->max_top * 4));
    RC(e->top_w.reserve(Ts * e->max_top * 4));
    RC(e->sgate.reserve(Ts * 4));
    RC(e->inter.reserve(Ts * e->max_ff * es));
    if (grouped) RC(e->pairs_out.reserve(Ts * e->max_top * W * 4));
  }
  if (n_want > 0) {
    RC(e->hw.reserve(static_cast<size_t>(n_want) * W * es));
    RC(e->logits.reserve(static_cast<size_t>(n_want) * d.vocab * 4));
    RC(e->amax.reserve(static_cast<size_t>(n_want) * 4));
  }
  float* x = static_cast<float*>(e->x.p);
  float* proj = static_cast<float*>(e->proj.p);
  float* y = static_cast<float*>(e->y.p);
  float* y2 = static_cast<float*>(e->y2.p);
  float* y3 = static_cast<float*>(e->y3.p);
  float* y4 = static_cast<float*>(e->y4.p);
  const StepRows step_rows{d_seq, d_pos, d_first, d_count, d_pos0, n_entries};
  const bool tracing = e->trace_host != nullptr;
  bool single = true;  // every entry brings one token: a row's CTA owns its sequence's state
  bool fresh_prompt = getenv("KLLM_SEQ_LATENT_EXPAND") == nullptr || getenv("KLLM_SEQ_LATENT_EXPAND")[0] != '0';
  for (int i = 0; i < n_entries; ++i) {
    single = single && counts[i] == 1;
    fresh_prompt = fresh_prompt && h_pos0[i] == 0;  // every sequence starts with this step
  }

  // ---- device: the layer runs -------------------------------------------------------------------------------------
  e->prof_used = 0;
  e->prof_phase.clear();
  e->mark(-1);
  auto run_device = [&]() -> int {
  RC(launch_embed(dtype, d.embed, d_tok, x, e->any_run_embed ? static_cast<float*>(e->x0.p) : nullptr, nw(d.embed_norm),
                  d.norm_eps, d.embed_scale, T, W, st));
  e->mark(KLLM_SEQ_PHASE_NORM);
  // What comes ahead of run r's mixer rides on one norm kernel (`a` may already carry the end of the run before):
  // the embedding output and the run's vector are added, the pre-norm is taken, and the token shift is applied -- inside
  // the kernel when every entry is one token, else by a kernel of its own on the fp32 rows.
  auto router_args = [&](const kllm_seq_moe& M) {
    return RouterArgs{M.w_router, M.shared_ff > 0 ? M.w_shared_gate : nullptr, M.experts, M.top,
                      M.router_scale, static_cast<int32_t*>(e->top_idx.p),
                      static_cast<float*>(e->top_w.p), static_cast<float*>(e->sgate.p), M.router_kind, M.correction,
                      M.groups, M.groups_keep, M.router_bias};
  };
  auto launch_pre = [&](ResidNormArgs a, int r, int phase) -> int {
    const kllm_seq_layer& L = e->layers[e->run_layer[r]];
    a.x = x, a.T = T, a.width = W, a.dtype = dtype, a.eps = d.norm_eps;
    a.add = e->run_add[r] >= 0 ? d.run_vectors + static_cast<size_t>(e->run_add[r]) * W : nullptr;
    a.add_rows = e->run_embed[r] ? static_cast<const float*>(e->x0.p) : nullptr;
    a.pre = nw(L.pre_mixer), a.out = e->h.p;
    const bool shift_after = L.shift != nullptr && !single;
    if (L.shift != nullptr && single) a.shift = ShiftArgs{L.shift, e->shift_state[r], d_seq, d_pos};
    if (shift_after) a.out_f32 = static_cast<float*>(e->hn.p);
    if (L.parallel_ff && L.ff_kind == KLLM_SEQ_FF_MOE) a.router = router_args(L.moe);  // the experts read this row too
    RC(launch_resid_norm(a, st));
    if (shift_after)
      RC(launch_token_shift(dtype, static_cast<const float*>(e->hn.p), L.shift, e->shift_state[r], d_seq, d_pos, d_first,
                            d_count, n_entries, e->h.p, T, W, st));
    e->mark(phase);
    return 0;
  };
  // one mixer of layer L (run r): reads the normed rows in e->h, writes its output rows to `yout`
  auto run_mixer = [&](const kllm_seq_layer& L, int kind, int r, float* yout) -> int {
    if (kind == KLLM_SEQ_MIXER_ATTENTION) {
      const kllm_seq_attention& A = L.attn;
      const AttnShape shape = attn_shape(A);
      const PagedKV kv{e->k_pool[r], e->v_pool[r], e->table_dev, e->table_stride, e->page, shape.kv_heads * A.dim,
                       A.kv_heads * A.vdim};
      const int n_proj = attn_proj_rows(A);
      RC(gemm(dtype, e->h.p, A.w_in, proj, T, W, n_proj, st));
      e->mark(KLLM_SEQ_PHASE_IN_PROJ);
      if (A.values_are_keys) {
        const AttnPrep prep{std::max(1, A.conv_taps), A.conv_w, e->attn_conv[r], A.in_bias, A.rope_dims, A.rope_pairing,
                            A.rope_base};
        RC(launch_qk_conv_prepare(dtype, shape, prep, proj, step_rows, e->q.p, kv, T, st));
      } else {
        const RopeArgs rope{A.rope_dims, A.rope_base, A.rope_freq, A.rope_mag, A.rope_pairing};
        RC(launch_qk_prepare(dtype, shape, rope, proj, A.q_norm_w, A.k_norm_w, d.norm_eps, d_seq, d_pos, e->q.p,
                             static_cast<float*>(e->gates.p), kv, T, st));
      }
      e->mark(KLLM_SEQ_PHASE_QK_PREPARE);
      RC(launch_attention(dtype, shape, e->q.p, static_cast<const float*>(e->gates.p), kv, n_entries, d_first, d_count,
                          d_eseq, d_pos0, max_count, max_ctx, window_splits(A.keep_first > 0 ? 0 : A.window),
                          static_cast<float*>(e->ws.p), e->att.p, T, d_seq, d_pos, st));
      if (A.differential)
        RC(launch_diff_merge(dtype, shape, window_splits(A.keep_first > 0 ? 0 : A.window), static_cast<const float*>(e->ws.p),
                             static_cast<const float*>(e->gates.p), A.diff_lambda, A.diff_out_scale, d.norm_eps, e->att.p, T,
                             st));
      e->mark(KLLM_SEQ_PHASE_ATTENTION);
      RC(gemm(dtype, e->att.p, A.w_out, yout, T, A.heads * A.vdim, W, st));
      e->mark(KLLM_SEQ_PHASE_OUT_PROJ);
    } else if (kind == KLLM_SEQ_MIXER_LATENT) {
      const kllm_seq_latent& A = L.latent;
      const LatentShape ls{A.heads, A.dim, A.rot_dim, A.vdim, A.q_rank, A.kv_rank, A.rope_dims, A.rope_base};
      const int krow = A.kv_rank + A.rot_dim;
      const PagedKV kv{e->k_pool[r], e->k_pool[r], e->table_dev, e->table_stride, e->page, krow, krow};
      float* gates = static_cast<float*>(e->gates.p);
      RC(gemm(dtype, e->h.p, A.w_in, proj, T, W, A.q_rank + krow + A.heads, st));
      e->mark(KLLM_SEQ_PHASE_IN_PROJ);
      // Prompt steps whose sequences all start here: the step's own latents are all the keys there are, so they are
      // expanded into per-head keys and values (two products) and the tensor-core attention runs on those rows.  Every
      // other step scores against the cached latents (the absorbed form below).
      const int dqk = A.dim + A.rot_dim;
      const AttnShape eshape{A.heads, A.heads, dqk, A.vdim, A.scale, 0.f, 0, 0, 1, A.window, A.sink, 0, 0, 0};
      if (fresh_prompt && attention_mma_usable(dtype, eshape, max_count)) {
        RC(e->lat_c.reserve(Ts * A.kv_rank * es));
        RC(e->lat_kr.reserve(Ts * std::max(1, A.rot_dim) * 4));
        RC(e->lat_kp.reserve(Ts * A.heads * A.dim * 4));
        RC(e->lat_vp.reserve(Ts * A.heads * A.vdim * 4));
        RC(e->lat_q.reserve(Ts * A.heads * dqk * es));
        RC(e->lat_k.reserve(Ts * A.heads * dqk * es));
        RC(e->lat_v.reserve(Ts * A.heads * A.vdim * es));
        RC(launch_latent_prepare(dtype, ls, proj, A.q_norm_w, A.kv_norm_w, d.norm_eps, d_seq, d_pos, e->q.p, gates, kv,
                                 e->lat_c.p, static_cast<float*>(e->lat_kr.p), T, st));
        RC(gemm(dtype, e->q.p, A.w_uq, static_cast<float*>(e->qf.p), T, A.q_rank, A.heads * dqk, st));
        RC(launch_latent_pack_q(dtype, ls, static_cast<const float*>(e->qf.p), d_pos, e->lat_q.p, T, st));
        RC(gemm(dtype, e->lat_c.p, A.w_uk, static_cast<float*>(e->lat_kp.p), T, A.kv_rank, A.heads * A.dim, st));
        RC(gemm(dtype, e->lat_c.p, A.w_uv, static_cast<float*>(e->lat_vp.p), T, A.kv_rank, A.heads * A.vdim, st));
        RC(launch_latent_pack_kv(dtype, ls, static_cast<const float*>(e->lat_kp.p), static_cast<const float*>(e->lat_kr.p),
                                 static_cast<const float*>(e->lat_vp.p), e->lat_k.p, e->lat_v.p, T, st));
        e->mark(KLLM_SEQ_PHASE_QK_PREPARE);
        const PagedKV rows{e->lat_k.p, e->lat_v.p, nullptr, 0, 1, A.heads * dqk, A.heads * A.vdim};
        RC(launch_attention(dtype, eshape, e->lat_q.p, gates, rows, n_entries, d_first, d_count, d_eseq, d_pos0, max_count,
                            max_ctx, 1, static_cast<float*>(e->ws.p), e->att.p, T, d_seq, d_pos, st));
        e->mark(KLLM_SEQ_PHASE_ATTENTION);
        RC(gemm(dtype, e->att.p, A.w_out, yout, T, A.heads * A.vdim, W, st));
        e->mark(KLLM_SEQ_PHASE_OUT_PROJ);
      } else {
      RC(launch_latent_prepare(dtype, ls, proj, A.q_norm_w, A.kv_norm_w, d.norm_eps, d_seq, d_pos, e->q.p, gates, kv, nullptr,
                               nullptr, T, st));
      RC(gemm(dtype, e->q.p, A.w_uq, static_cast<float*>(e->qf.p), T, A.q_rank, A.heads * (A.dim + A.rot_dim), st));
      RC(launch_latent_absorb(dtype, ls, static_cast<const float*>(e->qf.p), A.w_uk, d_pos, static_cast<float*>(e->qa.p), T, st));
      e->mark(KLLM_SEQ_PHASE_QK_PREPARE);
      // one shared key/value "head": keys [latent | rotated part], values the latent itself
      // steps of single tokens merge the key splits and apply W_uv in one kernel
      const bool fused_merge = single && T <= 32;
      const AttnShape shape{A.heads, 1, krow, A.kv_rank, A.scale, 0.f, 0, 0, 1, A.window, A.sink, 1, 1, fused_merge ? 1 : 0};
      const int lsplits = window_splits(A.window);
      RC(launch_attention(dtype, shape, e->qa.p, gates, kv, n_entries, d_first, d_count, d_eseq, d_pos0, max_count, max_ctx,
                          lsplits, static_cast<float*>(e->ws.p), e->ol.p, T, d_seq, d_pos, st));
      if (fused_merge)
        RC(launch_latent_merge_expand(dtype, ls, lsplits, static_cast<const float*>(e->ws.p), gates, A.sink, A.w_uv,
                                      e->att.p, T, st));
      else
        RC(launch_latent_expand(dtype, ls, static_cast<const float*>(e->ol.p), A.w_uv, e->att.p, T, st));
      e->mark(KLLM_SEQ_PHASE_ATTENTION);
      RC(gemm(dtype, e->att.p, A.w_out, yout, T, A.heads * A.vdim, W, st));
      e->mark(KLLM_SEQ_PHASE_OUT_PROJ);
      }
    } else if (kind == KLLM_SEQ_MIXER_LINEAR) {
      const kllm_seq_linear& A = L.linear;
      RC(gemm(dtype, e->h.p, A.w_in, proj, T, W, 2 * A.heads * (A.dim + A.vdim), st));
      e->mark(KLLM_SEQ_PHASE_IN_PROJ);
      RC(launch_linear_attention(A.heads, A.dim, A.vdim, A.decay, proj, e->linear_state[r], n_entries, d_first, d_count,
                                 d_eseq, d_pos0, max_count, static_cast<float*>(e->ws.p), static_cast<float*>(e->ol.p), st));
      RC(launch_linear_out(dtype, A.heads, A.dim, A.vdim, static_cast<const float*>(e->ol.p), proj, A.out_norm_w, d.norm_eps,
                           e->att.p, T, st));
      e->mark(KLLM_SEQ_PHASE_ATTENTION);
      RC(gemm(dtype, e->att.p, A.w_out, yout, T, A.heads * A.vdim, W, st));
      e->mark(KLLM_SEQ_PHASE_OUT_PROJ);
    } else if (kind == KLLM_SEQ_MIXER_SSM) {
      const kllm_seq_ssm& A = L.ssm;
      float* uc = static_cast<float*>(e->rec_a.p);
      float* low = static_cast<float*>(e->rec_b.p);
      RC(gemm(dtype, e->h.p, A.w_in, proj, T, W, 2 * A.inner, st));
      e->mark(KLLM_SEQ_PHASE_IN_PROJ);
      RC(launch_ssm_conv(dtype, A, proj, e->ssm_conv[r], step_rows, uc, e->att.p, T, st));
      RC(gemm(dtype, e->att.p, A.w_x, low, T, A.inner, A.dt_rank + 2 * A.state, st));
      e->mark(KLLM_SEQ_PHASE_QK_PREPARE);
      RC(launch_ssm_scan(dtype, A, proj, uc, low, e->ssm_state[r], step_rows, d_eseq, max_count, T,
                         static_cast<float*>(e->ws.p), e->att.p, st));
      e->mark(KLLM_SEQ_PHASE_ATTENTION);
      RC(gemm(dtype, e->att.p, A.w_out, yout, T, A.inner, W, st));
      e->mark(KLLM_SEQ_PHASE_OUT_PROJ);
    } else if (kind == KLLM_SEQ_MIXER_SSD) {
      const kllm_seq_ssd& A = L.ssd;
      float* xbc = static_cast<float*>(e->rec_a.p);
      float* yr = static_cast<float*>(e->rec_b.p);
      RC(gemm(dtype, e->h.p, A.w_in, proj, T, W, ssd_proj_row(A), st));
      e->mark(KLLM_SEQ_PHASE_IN_PROJ);
      RC(launch_ssd_conv(A, proj, e->ssd_conv[r], step_rows, xbc, T, st));
      e->mark(KLLM_SEQ_PHASE_QK_PREPARE);
      RC(launch_ssd_scan(A, proj, xbc, e->ssd_state[r], step_rows, d_eseq, max_count, T, static_cast<float*>(e->ws.p), yr, st));
      RC(launch_ssd_out(dtype, A, yr, proj, d.norm_eps, e->att.p, T, st));
      e->mark(KLLM_SEQ_PHASE_ATTENTION);
      RC(gemm(dtype, e->att.p, A.w_out, yout, T, ssd_inner(A), W, st));
      e->mark(KLLM_SEQ_PHASE_OUT_PROJ);
    } else {
      const kllm_seq_delta& A = L.delta;
      float* prep = static_cast<float*>(e->rec_a.p);
      float* o = static_cast<float*>(e->rec_b.p);
      const int n_proj = 2 * A.kv_heads * A.dim + A.heads * A.vdim + A.heads + A.decay_rank + A.gate_rank;
      RC(gemm(dtype, e->h.p, A.w_in, proj, T, W, n_proj, st));
      e->mark(KLLM_SEQ_PHASE_IN_PROJ);
      // the second low-rank projections of the decays and the gates: one product on the low-rank rows in the compute type
      float* low2 = static_cast<float*>(e->rec_c.p);
      RC(launch_delta_low(dtype, A, proj, e->q.p, T, st));
      RC(gemm(dtype, e->q.p, A.w_low2, low2, T, A.decay_rank + A.gate_rank, A.heads * (A.dim + A.vdim), st));
      RC(launch_delta_prepare(A, proj, low2, e->delta_conv[r], step_rows, prep, T, st));
      e->mark(KLLM_SEQ_PHASE_QK_PREPARE);
      RC(launch_delta_rule(A, prep, e->delta_state[r], step_rows, d_eseq, max_count, T, static_cast<float*>(e->ws.p), o, st));
      RC(launch_delta_out(dtype, A, o, prep, d.norm_eps, e->att.p, T, st));
      e->mark(KLLM_SEQ_PHASE_ATTENTION);
      RC(gemm(dtype, e->att.p, A.w_out, yout, T, A.heads * A.vdim, W, st));
      e->mark(KLLM_SEQ_PHASE_OUT_PROJ);
    }
    return 0;
  };
  // the feed-forward of layer L on the rows in e->h: its output goes to `yout`, a shared expert's (when it did not ride
  // along with the routed ones) to y2 with *shared_out set; the router has already run
  auto run_ff = [&](const kllm_seq_layer& L, float* yout, bool* shared_out) -> int {
    *shared_out = false;
    if (L.ff_kind == KLLM_SEQ_FF_DENSE) {
      const kllm_seq_dense& F = L.dense;
      if (F.act == KLLM_SEQ_ACT_RELU_GATE) {
        RC(gemm(dtype, e->h.p, F.up, proj, T, W, 2 * F.ff, st));
        RC(launch_gated_act(dtype, GatedAct{F.act, 0.f, 0.f}, proj, e->att.p, T, F.ff, st));
      } else {
        RC(gemm(dtype, e->h.p, F.up, proj, T, W, F.ff, st));
        RC(launch_activation(dtype, F.act, F.act_a, F.act_b, proj, e->att.p, Ts * F.ff, st));
      }
      RC(gemm(dtype, e->att.p, F.down, yout, T, F.ff, W, st));
      e->mark(KLLM_SEQ_PHASE_EXPERTS);
      return 0;
    }
    const kllm_seq_moe& M = L.moe;
    int32_t* top_idx = static_cast<int32_t*>(e->top_idx.p);
    float* top_w = static_cast<float*>(e->top_w.p);
    float* sgate = static_cast<float*>(e->sgate.p);
    const GatedAct act{M.act, M.act_limit, M.act_alpha};
    bool shared_done = false;  // the shared expert went through the pair kernels: yout already holds its part
    if (!grouped) {
      SharedExpert sh{};
      // every pair streams its expert's weights once: beyond a few tokens the shared expert is cheaper as a product
      if (M.shared_ff > 0 && T <= kSharedRideTokens && shared_expert_rides_along(M.top, M.ff, M.shared_ff)) {
        sh = SharedExpert{M.shared_gate_up, M.shared_down, M.w_shared_gate ? sgate : nullptr, e->att.p, M.shared_ff,
                          M.shared_act_limit};
        shared_done = true;
      }
      RC(launch_expert_gate_up(dtype, e->h.p, M.gate_up, top_idx, e->inter.p, T, M.top, M.ff, W, sh, act, st));
      RC(launch_expert_down(dtype, e->inter.p, M.down, top_idx, top_w, yout, T, M.top, M.ff, W, sh, st));
    } else {
      const int n_pairs = T * M.top;
      const int cap = ((n_pairs + kGroupBlock - 1) / kGroupBlock + M.experts) * kGroupBlock;
      const int n_blocks = cap / kGroupBlock;
      RC(e->sort.reserve((static_cast<size_t>(M.experts) + 1 + cap + n_blocks) * 4));
      int32_t* counts_d = static_cast<int32_t*>(e->sort.p);
      int32_t* sorted = counts_d + M.experts + 1;
      int32_t* block_expert = sorted + cap;
      RC(launch_sort_pairs(top_idx, n_pairs, M.experts, kGroupBlock, counts_d, sorted, block_expert, cap, st));
      GroupedArgs g{};
      g.sorted_pair = sorted, g.block_expert = block_expert, g.n_blocks = n_blocks, g.block = kGroupBlock;
      g.experts = M.experts, g.act = act;
      const int inner_epilogue = M.act == KLLM_SEQ_ACT_RELU2 ? 2 : 1;
      if (grouped_tensor_core_usable(dtype, W, M.ff)) {
        // rows in sorted order: a gathered copy of h, the expert's inner activations, then scattered back by pair
        RC(e->sorted_a.reserve(static_cast<size_t>(cap) * W * es));
        RC(e->sorted_inter.reserve(static_cast<size_t>(cap) * M.ff * es));
        RC(gather_rows_bf16(e->h.p, sorted, M.top, e->sorted_a.p, cap, W, st));
        g.sorted_layout = 1;
        g.a = e->sorted_a.p, g.w = M.gate_up, g.K = W, g.N = M.ff, g.epilogue = inner_epilogue, g.out = e->sorted_inter.p;
        RC(gemm_grouped(dtype, g, st));
        g.a = e->sorted_inter.p, g.w = M.down, g.K = M.ff, g.N = W, g.epilogue = 0, g.out = e->pairs_out.p;
        RC(gemm_grouped(dtype, g, st));
      } else {
        g.a = e->h.p, g.w = M.gate_up, g.a_row_div = M.top, g.K = W, g.N = M.ff, g.epilogue = inner_epilogue, g.out = e->inter.p;
        RC(gemm_grouped(dtype, g, st));
        g.a = e->inter.p, g.w = M.down, g.a_row_div = 1, g.K = M.ff, g.N = W, g.epilogue = 0, g.out = e->pairs_out.p;
        RC(gemm_grouped(dtype, g, st));
      }
      RC(launch_combine_pairs(static_cast<const float*>(e->pairs_out.p), top_w, yout, T, M.top, W, st));
    }
    e->mark(KLLM_SEQ_PHASE_EXPERTS);
    if (M.shared_ff > 0 && !shared_done) {
      RC(gemm(dtype, e->h.p, M.shared_gate_up, proj, T, W, 2 * M.shared_ff, st));
      RC(launch_gated_act(dtype, GatedAct{M.act, M.shared_act_limit, M.act_alpha}, proj, e->att.p, T, M.shared_ff, st));
      RC(gemm(dtype, e->att.p, M.shared_down, y2, T, M.shared_ff, W, st));
      e->mark(KLLM_SEQ_PHASE_SHARED);
      *shared_out = true;
    }
    return 0;
  };
  bool pre_done = false;  // the previous run's last kernel already produced this run's h
  for (int r = 0; r < d.n_runs; ++r) {
    const kllm_seq_layer& L = e->layers[e->run_layer[r]];
    if (!pre_done) RC(launch_pre(ResidNormArgs{}, r, KLLM_SEQ_PHASE_NORM));
    pre_done = false;
    RC(run_mixer(L, L.mixer_kind, r, y));
    if (L.mixer2_kind != 0) RC(run_mixer(L, L.mixer2_kind, r, y3));
    // what the mixers add to x: c1 y (+ c3 y3)
    ResidNormArgs mixed{};
    mixed.y1 = y;
    if (L.mixer2_kind != 0) mixed.c1 = L.mixer_scale, mixed.y3 = y3, mixed.c3 = L.mixer2_scale;
    mixed.n1 = nw(L.mixer_out_norm), mixed.n3 = nw(L.mixer2_out_norm);

    // what follows this layer run: the next run's additions and pre-norm can ride on this run's last kernel
    const bool fuse_next = r + 1 < d.n_runs && !tracing;
    auto end_of_run = [&](ResidNormArgs a) -> int {  // `a` holds what the run still adds to x
      if (fuse_next) {
        pre_done = true;
        return launch_pre(a, r + 1, KLLM_SEQ_PHASE_NORM);
      }
      a.x = x, a.T = T, a.width = W, a.dtype = dtype, a.eps = d.norm_eps;
      RC(launch_resid_norm(a, st));
      e->mark(KLLM_SEQ_PHASE_NORM);
      return 0;
    };
    const kllm_seq_moe& M = L.moe;
    const float* sgate = static_cast<const float*>(e->sgate.p);
    if (L.ff_kind == KLLM_SEQ_FF_NONE) {
      mixed.post = nw(L.post_mixer);
      RC(end_of_run(mixed));
    } else if (L.parallel_ff) {
      // the feed-forward read the same rows as the mixers (the pre-norm kernel also routed them): one sum joins x
      bool shared = false;
      RC(run_ff(L, y4, &shared));
      mixed.y4 = y4;
      if (shared) mixed.y2 = y2, mixed.s2 = M.w_shared_gate ? sgate : nullptr;
      RC(end_of_run(mixed));
    } else {
      {  // the norm kernel that writes the feed-forward's input also routes its row
        ResidNormArgs a = mixed;
        a.x = x, a.post = nw(L.post_mixer), a.pre = nw(L.pre_ff), a.out = e->h.p, a.T = T, a.width = W;
        a.dtype = dtype, a.eps = d.norm_eps;
        if (L.ff_kind == KLLM_SEQ_FF_MOE) a.router = router_args(M);
        RC(launch_resid_norm(a, st));
        e->mark(KLLM_SEQ_PHASE_ROUTER);
      }
      bool shared = false;
      RC(run_ff(L, y, &shared));
      ResidNormArgs a{};
      a.y1 = y, a.y2 = shared ? y2 : nullptr, a.s2 = shared && M.w_shared_gate ? sgate : nullptr;
      a.post = nw(L.post_ff);
      RC(end_of_run(a));
    }
    if (tracing)
      CU(cudaMemcpyAsync(e->trace_host + static_cast<size_t>(r) * T * W, x, Ts * W * 4, cudaMemcpyDeviceToHost, st));
  }

  // ---- the wanted rows: final norm, classifier, greedy id -------------------------------------------------------
  if (n_want > 0) {
    ResidNormArgs a{};
    a.x = x, a.pre = nw(d.final_norm), a.out = e->hw.p, a.rows = d_want, a.T = n_want, a.width = W, a.dtype = dtype;
    a.eps = d.norm_eps;
    RC(launch_resid_norm(a, st));
    float* lg = static_cast<float*>(e->logits.p);
    RC(gemm(dtype, e->hw.p, d.head, lg, n_want, W, d.vocab, st));
    if ((d.logit_scale != 0.f && d.logit_scale != 1.f) || d.logit_softcap > 0.f)
      RC(launch_scale(lg, d.logit_scale, d.logit_softcap, static_cast<size_t>(n_want) * d.vocab, st));
    if (argmax_host) RC(launch_argmax_rows(lg, static_cast<int32_t*>(e->amax.p), n_want, d.vocab, st));
  }
  return 0;
  };  // run_device

  const bool all_single = single && !tracing && e->prof_out == nullptr && e->use_graphs && T <= 32;
  bool replayed = false;
  if (all_single) {
    const auto key = std::make_tuple(n_entries, n_want, splits, argmax_host ? 1 : 0);
    kllm_seq_engine::Graph& g = e->graphs[key];
    if (g.exec != nullptr && g.generation != g_buffer_generation) {
      cudaGraphExecDestroy(g.exec);
      g.exec = nullptr;
    }
    if (g.exec == nullptr) {
      const uint64_t before = launch_counter().load();
      cudaGraph_t graph = nullptr;
      if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
        const int rc = run_device();
        const cudaError_t ce = cudaStreamEndCapture(st, &graph);
        if (rc == 0 && ce == cudaSuccess && graph != nullptr &&
            cudaGraphInstantiate(&g.exec, graph, 0) == cudaSuccess) {
          g.generation = g_buffer_generation;
          g.nodes = static_cast<int>(launch_counter().load() - before);
        } else {
          g.exec = nullptr;
          cudaGetLastError();
        }
        if (graph) cudaGraphDestroy(graph);
      }
      launch_counter().fetch_sub(launch_counter().load() - before);  // captured, not launched
    }
    if (g.exec != nullptr) {
      CU(cudaGraphLaunch(g.exec, st));
      count_launch(static_cast<uint64_t>(g.nodes));
      replayed = true;
    }
  }
  if (!replayed) RC(run_device());
  e->trace_host = nullptr;
  if (n_want > 0) {
    if (argmax_host)
      CU(cudaMemcpyAsync(argmax_host, e->amax.p, static_cast<size_t>(n_want) * 4, cudaMemcpyDeviceToHost, st));
    if (logits_host)
      CU(cudaMemcpyAsync(logits_host, e->logits.p, static_cast<size_t>(n_want) * d.vocab * 4, cudaMemcpyDeviceToHost, st));
  }
  e->mark(KLLM_SEQ_PHASE_HEAD);
  e->last_launches = static_cast<int>(launch_counter().load() - launches_before);
  CU(cudaStreamSynchronize(st));
  if (e->prof_out) {
    for (int i = 0; i < KLLM_SEQ_PHASES; ++i) e->prof_out[i] = 0.f;
    for (size_t i = 1; i < e->prof_used; ++i) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, e->prof_events[i - 1], e->prof_events[i]) == cudaSuccess && e->prof_phase[i] >= 0)
        e->prof_out[e->prof_phase[i]] += ms;
    }
    e->prof_out = nullptr;
  }
  if (gemm_take_error()) return KLLM_E_STATE;
  return 0;
}

extern "C" int kllm_seq_gemm(int32_t dtype, const void* a, const void* w, float* out, int32_t n_tokens, int32_t in_dim,
                             int32_t out_dim, void* stream) {
  const int rc = gemm(dtype, a, w, out, n_tokens, in_dim, out_dim, static_cast<cudaStream_t>(stream));
  if (rc != 0) return rc;
  if (gemm_take_error()) return KLLM_E_STATE;
  return 0;
}
