#include "model/vurazen.h"

#include <cmath>
#include <string>
#include <vector>

namespace model {
KLLM_REGISTER_SEQUENCE_MODEL("Vurazen", VurazenModel);

namespace {
constexpr float kExpertSigmoidSlope = 1.702f;  // the experts' activation is g * sigmoid(1.702 g) * (u + 1)

int32_t get_int(const json::Value& v, const char* key) { return static_cast<int32_t>(v.at(key).as_int()); }
float get_float(const json::Value& v, const char* key) { return static_cast<float>(v.at(key).as_number()); }
bool present(const json::Value& v, const char* key) { return v.has(key) && !v.at(key).is_null(); }
bool shaped(const StTensor* t, int64_t rows, int64_t cols) {
  return t != nullptr && t->shape.size() == 2 && t->shape[0] == rows && t->shape[1] == cols;
}
bool sized(const StTensor* t, int64_t n) { return t != nullptr && t->shape.size() == 1 && t->shape[0] == n; }
base::Status bad(const std::string& p, const char* what) { return base::error::ModelParseError(p + ": " + what); }
}  // namespace

base::Status VurazenModel::layer_norm(const SafetensorsFile& w, const std::string& name, kllm_seq_norm* out) {
  base::Status st;
  const StTensor *g = need(w, name, &st), *b = need(w, name + ".b", &st);
  if (!st) return st;
  out->kind = KLLM_SEQ_NORM_LAYER;
  if (st = upload_f32(g, width_, &out->w); !st) return st;
  return upload_f32(b, width_, &out->b);
}

base::Status VurazenModel::build_scan(const json::Value& c, const SafetensorsFile& w, const std::string& p, kllm_seq_ssm* a) {
  a->inner = get_int(c, "inner"), a->state = get_int(c, "state"), a->dt_rank = get_int(c, "dt_rank");
  a->conv_taps = get_int(c, "conv");
  if (a->inner <= 0 || a->state <= 0 || a->dt_rank <= 0 || a->conv_taps < 1) return bad(p, "bad mixer configuration");
  base::Status st;
  const StTensor *in = need(w, p + "in", &st), *conv = need(w, p + "conv", &st), *convb = need(w, p + "conv.b", &st),
                 *x = need(w, p + "x", &st), *dt = need(w, p + "dt", &st), *dtb = need(w, p + "dt.b", &st),
                 *alog = need(w, p + "A_log", &st), *dd = need(w, p + "D", &st), *o = need(w, p + "o", &st);
  if (!st) return st;
  const int64_t n = a->inner;
  if (!shaped(in, 2 * n, width_) || !shaped(conv, n, a->conv_taps) || !sized(convb, n) ||
      !shaped(x, a->dt_rank + 2 * a->state, n) || !shaped(dt, n, a->dt_rank) || !sized(dtb, n) ||
      !shaped(alog, n, a->state) || !sized(dd, n) || !shaped(o, width_, n))
    return bad(p, "tensor shapes do not fit the configuration");
  if (st = upload_compute({in}, width_, &a->w_in); !st) return st;
  if (st = upload_compute({x}, n, &a->w_x); !st) return st;
  if (st = upload_compute({o}, n, &a->w_out); !st) return st;
  if (st = upload_f32(conv, n * a->conv_taps, &a->conv_w); !st) return st;
  if (st = upload_f32(convb, n, &a->conv_b); !st) return st;
  if (st = upload_f32(dt, n * a->dt_rank, &a->w_dt); !st) return st;
  if (st = upload_f32(dtb, n, &a->dt_b); !st) return st;
  if (st = upload_f32(dd, n, &a->d); !st) return st;
  std::vector<float> rates;  // the state decays with exp(step * a), a = -exp(A_log)
  if (st = read_values(alog, n * a->state, &rates); !st) return st;
  for (float& v : rates) v = -std::exp(v);
  return upload_values(rates, &a->a);
}

base::Status VurazenModel::build_lightning(const json::Value& c, const SafetensorsFile& w, const std::string& p,
                                           kllm_seq_linear* a) {
  a->heads = get_int(c, "heads"), a->dim = get_int(c, "dim"), a->vdim = get_int(c, "vdim");
  if (a->heads <= 0 || a->dim <= 0 || a->vdim <= 0) return bad(p, "bad mixer configuration");
  std::vector<float> lam;  // one decay per head, or one number for all heads
  if (c.at("decay").is_array()) {
    for (const auto& v : c.at("decay").array) lam.push_back(static_cast<float>(v.as_number()));
  } else {
    lam.assign(static_cast<size_t>(a->heads), get_float(c, "decay"));
  }
  if (static_cast<int64_t>(lam.size()) != a->heads) return bad(p, "one decay per head is needed");
  for (float v : lam)
    if (!(v > 0.f) || v > 1.f) return bad(p, "a decay must lie in (0, 1]");
  base::Status st;
  const StTensor *q = need(w, p + "q", &st), *k = need(w, p + "k", &st), *v = need(w, p + "v", &st), *g = need(w, p + "g", &st),
                 *o = need(w, p + "o", &st), *n = need(w, p + "norm", &st);
  if (!st) return st;
  const int64_t qn = int64_t(a->heads) * a->dim, vn = int64_t(a->heads) * a->vdim;
  if (!shaped(q, qn, width_) || !shaped(k, qn, width_) || !shaped(v, vn, width_) || !shaped(g, vn, width_) ||
      !shaped(o, width_, vn) || !sized(n, vn))
    return bad(p, "tensor shapes do not fit the configuration");
  if (st = upload_compute({q, k, v, g}, width_, &a->w_in); !st) return st;
  if (st = upload_compute({o}, vn, &a->w_out); !st) return st;
  if (st = upload_f32(n, vn, &a->out_norm_w); !st) return st;
  return upload_values(lam, &a->decay);
}

base::Status VurazenModel::build_window_attention(const json::Value& c, const SafetensorsFile& w, const std::string& p,
                                                  kllm_seq_attention* a) {
  a->heads = get_int(c, "heads"), a->kv_heads = get_int(c, "kv_heads"), a->dim = get_int(c, "dim"), a->vdim = get_int(c, "vdim");
  a->scale = get_float(c, "scale");
  a->softcap = present(c, "softcap") ? get_float(c, "softcap") : 0.f;
  a->conv_taps = get_int(c, "conv");
  a->window = 0, a->keep_first = 0;
  if (present(c, "mask")) {
    a->window = get_int(c.at("mask"), "size");
    a->keep_first = present(c.at("mask"), "keep_first") ? get_int(c.at("mask"), "keep_first") : 0;
  }
  a->rope_dims = 0, a->rope_base = 1.f, a->rope_pairing = KLLM_SEQ_ROPE_PAIRS;
  if (present(c, "rot")) a->rope_dims = get_int(c.at("rot"), "dims"), a->rope_base = get_float(c.at("rot"), "base");
  a->values_are_keys = 1;
  if (a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads || a->dim <= 0 || a->vdim != a->dim || a->conv_taps < 1 ||
      a->window < 0 || a->keep_first < 0 || a->softcap < 0.f || a->rope_dims < 0 || a->rope_dims > a->dim || (a->rope_dims & 1))
    return bad(p, "bad mixer configuration");
  base::Status st;
  const StTensor *q = need(w, p + "q", &st), *k = need(w, p + "k", &st), *qb = need(w, p + "q.b", &st),
                 *kb = need(w, p + "k.b", &st), *sink = need(w, p + "sink", &st), *o = need(w, p + "o", &st);
  if (!st) return st;
  const int64_t qn = int64_t(a->heads) * a->dim, kn = int64_t(a->kv_heads) * a->dim;
  if (!shaped(q, qn, width_) || !shaped(k, kn, width_) || !sized(qb, qn) || !sized(kb, kn) || !sized(sink, a->heads) ||
      !shaped(o, width_, int64_t(a->heads) * a->vdim))
    return bad(p, "tensor shapes do not fit the configuration");
  if (st = upload_compute({q, k}, width_, &a->w_in); !st) return st;
  if (st = upload_compute({o}, int64_t(a->heads) * a->vdim, &a->w_out); !st) return st;
  if (st = upload_f32_parts({qb, kb}, {qn, kn}, &a->in_bias); !st) return st;
  if (st = upload_f32(sink, a->heads, &a->sink); !st) return st;
  {  // a filter of one tap is still a weight per channel
    const StTensor *qc = need(w, p + "q.conv", &st), *kc = need(w, p + "k.conv", &st);
    if (!st) return st;
    if (!shaped(qc, qn, a->conv_taps) || !shaped(kc, kn, a->conv_taps)) return bad(p, "filter shapes do not fit the configuration");
    if (st = upload_f32_parts({qc, kc}, {qn * a->conv_taps, kn * a->conv_taps}, &a->conv_w); !st) return st;
  }
  return base::error::Success();
}

base::Status VurazenModel::build_delta(const json::Value& c, const SafetensorsFile& w, const std::string& p, kllm_seq_delta* a) {
  a->heads = get_int(c, "heads"), a->kv_heads = get_int(c, "kv_heads"), a->dim = get_int(c, "dim"), a->vdim = get_int(c, "vdim");
  a->conv_taps = get_int(c, "conv");
  if (a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads || a->dim <= 0 || a->vdim <= 0 || a->conv_taps < 1)
    return bad(p, "bad mixer configuration");
  base::Status st;
  const StTensor *q = need(w, p + "q", &st), *k = need(w, p + "k", &st), *v = need(w, p + "v", &st), *b = need(w, p + "b", &st),
                 *alog = need(w, p + "A_log", &st), *norm = need(w, p + "norm", &st), *a1 = need(w, p + "a1", &st),
                 *a2 = need(w, p + "a2", &st), *dtb = need(w, p + "dt_bias", &st), *g1 = need(w, p + "g1", &st),
                 *g2 = need(w, p + "g2", &st), *o = need(w, p + "o", &st);
  if (!st) return st;
  const int64_t qn = int64_t(a->kv_heads) * a->dim, vn = int64_t(a->heads) * a->vdim, dn = int64_t(a->heads) * a->dim;
  if (a1->shape.size() != 2 || g1->shape.size() != 2) return bad(p, "tensor shapes do not fit the configuration");
  a->decay_rank = static_cast<int32_t>(a1->shape[0]), a->gate_rank = static_cast<int32_t>(g1->shape[0]);
  if (!shaped(q, qn, width_) || !shaped(k, qn, width_) || !shaped(v, vn, width_) || !shaped(b, a->heads, width_) ||
      !sized(alog, a->heads) || !sized(norm, a->vdim) || !shaped(a1, a->decay_rank, width_) || !shaped(a2, dn, a->decay_rank) ||
      !sized(dtb, dn) || !shaped(g1, a->gate_rank, width_) || !shaped(g2, vn, a->gate_rank) || !shaped(o, width_, vn))
    return bad(p, "tensor shapes do not fit the configuration");
  if (st = upload_compute({q, k, v, b, a1, g1}, width_, &a->w_in); !st) return st;
  if (st = upload_compute({o}, vn, &a->w_out); !st) return st;
  {  // both second low-rank projections as one product: W_a2 upper left, W_g2 lower right
    std::vector<float> wa, wg;
    if (st = read_values(a2, dn * a->decay_rank, &wa); !st) return st;
    if (st = read_values(g2, vn * a->gate_rank, &wg); !st) return st;
    const int64_t cols = int64_t(a->decay_rank) + a->gate_rank;
    std::vector<float> both(static_cast<size_t>((dn + vn) * cols), 0.f);
    for (int64_t r = 0; r < dn; ++r)
      for (int64_t c = 0; c < a->decay_rank; ++c) both[r * cols + c] = wa[r * a->decay_rank + c];
    for (int64_t r = 0; r < vn; ++r)
      for (int64_t c = 0; c < a->gate_rank; ++c) both[(dn + r) * cols + a->decay_rank + c] = wg[r * a->gate_rank + c];
    if (st = upload_compute_values(both, &a->w_low2); !st) return st;
  }
  if (st = upload_f32(dtb, dn, &a->dt_bias); !st) return st;
  if (st = upload_f32(norm, a->vdim, &a->out_norm_w); !st) return st;
  std::vector<float> rate;
  if (st = read_values(alog, a->heads, &rate); !st) return st;
  for (float& r : rate) r = std::exp(r);
  if (st = upload_values(rate, &a->rate); !st) return st;
  {  // a filter of one tap is still a weight per channel
    const StTensor *qc = need(w, p + "q.conv", &st), *kc = need(w, p + "k.conv", &st), *vc = need(w, p + "v.conv", &st);
    if (!st) return st;
    if (!shaped(qc, qn, a->conv_taps) || !shaped(kc, qn, a->conv_taps) || !shaped(vc, vn, a->conv_taps))
      return bad(p, "filter shapes do not fit the configuration");
    const int64_t t = a->conv_taps;
    if (st = upload_f32_parts({qc, kc, vc}, {qn * t, qn * t, vn * t}, &a->conv_w); !st) return st;
  }
  return base::error::Success();
}

base::Status VurazenModel::build_dense(const json::Value& c, const SafetensorsFile& w, const std::string& p,
                                       kllm_seq_dense* f) {
  f->ff = get_int(c, "ff");
  if (f->ff <= 0) return bad(p, "bad size");
  base::Status st;
  const StTensor *gate = need(w, p + "gate", &st), *up = need(w, p + "up", &st), *down = need(w, p + "down", &st);
  if (!st) return st;
  if (!shaped(gate, f->ff, width_) || !shaped(up, f->ff, width_) || !shaped(down, width_, f->ff))
    return bad(p, "tensor shapes do not fit the configuration");
  f->act = KLLM_SEQ_ACT_RELU_GATE, f->act_a = 0.f, f->act_b = 0.f;
  if (st = upload_compute({gate, up}, width_, &f->up); !st) return st;
  return upload_compute({down}, f->ff, &f->down);
}

base::Status VurazenModel::build_moe(const json::Value& c, const SafetensorsFile& w, const std::string& p, kllm_seq_moe* m) {
  const json::Value& r = c.at("router");
  m->experts = get_int(r, "experts"), m->top = get_int(r, "top");
  m->ff = get_int(c.at("expert"), "ff");
  m->act = KLLM_SEQ_ACT_CLAMP_SWIGLU, m->act_limit = get_float(c.at("expert"), "limit"), m->act_alpha = kExpertSigmoidSlope;
  m->router_kind = KLLM_SEQ_ROUTER_TOP_SOFTMAX, m->router_scale = 1.0f;
  m->groups = 0, m->groups_keep = 0, m->correction = nullptr, m->w_shared_gate = nullptr;
  if (m->experts <= 0 || m->top <= 0 || m->top > m->experts || m->ff <= 0 || !(m->act_limit > 0.f))
    return bad(p, "bad router or expert configuration");
  base::Status st;
  auto expert = [&](const std::string& ep, int32_t ff, std::vector<const StTensor*>* gate_up, std::vector<const StTensor*>* down) {
    const StTensor *g = need(w, ep + "gate", &st), *u = need(w, ep + "up", &st), *d = need(w, ep + "down", &st);
    if (!st) return st;
    if (!shaped(g, ff, width_) || !shaped(u, ff, width_) || !shaped(d, width_, ff))
      return bad(ep, "expert shapes do not fit the configuration");
    gate_up->push_back(g), gate_up->push_back(u), down->push_back(d);
    return base::error::Success();
  };
  std::vector<const StTensor*> gate_up, down;
  for (int e = 0; e < m->experts; ++e)
    if (base::Status es = expert(p + "e" + std::to_string(e) + ".", m->ff, &gate_up, &down); !es) return es;
  if (st = upload_compute(gate_up, width_, &m->gate_up); !st) return st;
  if (st = upload_compute(down, m->ff, &m->down); !st) return st;
  if (st = upload_f32(need(w, p + "router", &st), int64_t(m->experts) * width_, &m->w_router); !st) return st;
  if (st = upload_f32(need(w, p + "router.b", &st), m->experts, &m->router_bias); !st) return st;
  m->shared_ff = 0, m->shared_act_limit = 0.f;
  if (present(c, "shared")) {
    m->shared_ff = get_int(c.at("shared"), "ff");
    m->shared_act_limit = get_float(c.at("shared"), "limit");
    if (m->shared_ff <= 0 || !(m->shared_act_limit > 0.f)) return bad(p, "bad shared expert");
    std::vector<const StTensor*> sgu, sd;
    if (base::Status es = expert(p + "shared.", m->shared_ff, &sgu, &sd); !es) return es;
    if (st = upload_compute(sgu, width_, &m->shared_gate_up); !st) return st;
    if (st = upload_compute(sd, m->shared_ff, &m->shared_down); !st) return st;
  }
  return base::error::Success();
}

// every tensor the configuration implies, by name
base::Status VurazenModel::check_folder(const json::Value& config, const SafetensorsFile& w) {
  base::Status st;
  for (const char* name : {"embed", "head", "final.norm", "final.norm.b"}) need(w, name, &st);
  const auto& layers = config.at("layers").array;
  for (size_t i = 0; i < layers.size(); ++i) {
    const std::string p = "l" + std::to_string(i) + ".";
    const std::string& type = layers[i].at("type").as_string();
    std::vector<std::string> names = {"norm1", "norm1.b"};
    if (type == "mamba1") {
      for (const char* n : {"in", "conv", "conv.b", "x", "dt", "dt.b", "A_log", "D", "o"}) names.push_back(std::string("mix.") + n);
    } else if (type == "lightning") {
      for (const char* n : {"q", "k", "v", "g", "norm", "o"}) names.push_back(std::string("mix.") + n);
    } else if (type == "parallel") {
      for (const char* n : {"q", "q.b", "q.conv", "k", "k.b", "k.conv", "sink", "o"}) names.push_back(std::string("mix.left.") + n);
      for (const char* n : {"q", "q.conv", "k", "k.conv", "v", "v.conv", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o"})
        names.push_back(std::string("mix.right.") + n);
    } else {
      return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown mixer '" + type + "'");
    }
    if (present(layers[i], "mlp")) {
      const json::Value& mc = layers[i].at("mlp");
      if (mc.at("kind").as_string() == "dense") {
        for (const char* n : {"mlp.gate", "mlp.up", "mlp.down"}) names.push_back(n);
      } else {
        names.push_back("mlp.router"), names.push_back("mlp.router.b");
        std::vector<std::string> experts;
        for (int e = 0; e < get_int(mc.at("router"), "experts"); ++e) experts.push_back("e" + std::to_string(e));
        if (present(mc, "shared")) experts.push_back("shared");
        for (const std::string& e : experts)
          for (const char* n : {"gate", "up", "down"}) names.push_back("mlp." + e + "." + n);
      }
    }
    for (const std::string& n : names) need(w, p + n, &st);
  }
  return st;
}

base::Status VurazenModel::build(const json::Value& config, const SafetensorsFile& w) {
  vocab_ = get_int(config, "vocab");
  width_ = get_int(config, "width");
  norm_eps_ = get_float(config.at("norm"), "eps");
  embed_scale_ = present(config, "embedding") ? get_float(config.at("embedding"), "scale") : 1.0f;
  logit_softcap_ = present(config, "logit_softcap") ? get_float(config, "logit_softcap") : 0.0f;
  if (vocab_ <= 0 || width_ <= 0 || logit_softcap_ < 0.f) return base::error::ModelParseError("bad vocab / width / logit_softcap");
  const auto& layers = config.at("layers").array;
  if (layers.empty()) return base::error::ModelParseError("no layers");
  base::Status st;
  layers_.assign(layers.size(), kllm_seq_layer{});
  for (size_t i = 0; i < layers.size(); ++i) {
    const json::Value& lc = layers[i];
    kllm_seq_layer& L = layers_[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const std::string& type = lc.at("type").as_string();
    const json::Value& mc = lc.at("mixer");
    if (st = layer_norm(w, p + "norm1", &L.pre_mixer); !st) return st;
    L.mixer_scale = 1.0f, L.mixer2_scale = 1.0f, L.mixer2_kind = 0;
    if (type == "mamba1") {
      L.mixer_kind = KLLM_SEQ_MIXER_SSM;
      if (st = build_scan(mc, w, p + "mix.", &L.ssm); !st) return st;
    } else if (type == "lightning") {
      L.mixer_kind = KLLM_SEQ_MIXER_LINEAR;
      if (st = build_lightning(mc, w, p + "mix.", &L.linear); !st) return st;
    } else if (type == "parallel") {
      L.mixer_kind = KLLM_SEQ_MIXER_ATTENTION, L.mixer2_kind = KLLM_SEQ_MIXER_DELTA;
      L.mixer_scale = get_float(mc, "left_scale"), L.mixer2_scale = get_float(mc, "right_scale");
      if (st = build_window_attention(mc.at("left"), w, p + "mix.left.", &L.attn); !st) return st;
      if (st = build_delta(mc.at("right"), w, p + "mix.right.", &L.delta); !st) return st;
    } else {
      return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown mixer '" + type + "'");
    }
    L.ff_kind = KLLM_SEQ_FF_NONE, L.parallel_ff = 0;
    if (present(lc, "mlp")) {
      const json::Value& fc = lc.at("mlp");
      const std::string& kind = fc.at("kind").as_string();
      L.parallel_ff = 1;  // the feed-forward reads norm1's output, beside the mixer
      if (kind == "dense") {
        L.ff_kind = KLLM_SEQ_FF_DENSE;
        if (st = build_dense(fc, w, p + "mlp.", &L.dense); !st) return st;
      } else if (kind == "moe") {
        L.ff_kind = KLLM_SEQ_FF_MOE;
        if (st = build_moe(fc, w, p + "mlp.", &L.moe); !st) return st;
      } else {
        return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown feed-forward '" + kind + "'");
      }
    }
  }
  // the order of layer runs
  const int32_t n = static_cast<int32_t>(layers.size());
  int32_t start = 0, stop = 0, times = 1;
  if (present(config, "loop")) {
    const json::Value& lp = config.at("loop");
    start = get_int(lp, "start"), stop = get_int(lp, "stop"), times = get_int(lp, "times");
    if (start < 0 || stop < start || stop > n || times < 1) return base::error::ModelParseError("bad loop");
  }
  run_layer_.clear(), run_add_.clear(), run_embed_.clear();
  auto push = [&](int32_t layer, int32_t add, int32_t embed) {
    run_layer_.push_back(layer), run_add_.push_back(add), run_embed_.push_back(embed);
  };
  for (int32_t i = 0; i < start; ++i) push(i, -1, 0);
  if (stop > start)
    for (int32_t t = 0; t < times; ++t)
      for (int32_t i = start; i < stop; ++i) push(i, i == start ? t : -1, i == start && t > 0 ? 1 : 0);
  for (int32_t i = stop; i < n; ++i) push(i, -1, 0);
  if (stop > start) {
    if (st = upload_f32(need(w, "loop.step", &st), int64_t(times) * width_, &run_vectors_); !st) return st;
  }
  const StTensor *embed = need(w, "embed", &st), *head = need(w, "head", &st);
  if (!st) return st;
  if (!shaped(embed, vocab_, width_) || !shaped(head, vocab_, width_))
    return base::error::ModelParseError("embed / head do not fit vocab x width");
  if (st = upload_compute({embed}, width_, &embed_); !st) return st;
  if (st = upload_compute({head}, width_, &head_); !st) return st;
  return layer_norm(w, "final.norm", &final_norm_);
}
}  // namespace model
