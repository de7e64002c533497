#include "model/bukuvik.h"

#include <algorithm>
#include <cmath>
#include <string>
#include <vector>

namespace model {
KLLM_REGISTER_SEQUENCE_MODEL("Bukuvik", BukuvikModel);

namespace {
constexpr double kPi = 3.14159265358979323846;
// cos and sin of rescaled rotary positions grow by kRotMagSlope * ln(factor) + 1
constexpr double kRotMagSlope = 0.1;
// the ramp between rescaled and untouched frequencies never divides by less than this
constexpr double kRampFloor = 0.001;

int32_t get_int(const json::Value& v, const char* key) { return static_cast<int32_t>(v.at(key).as_int()); }
double get_number(const json::Value& v, const char* key) { return v.at(key).as_number(); }
bool present(const json::Value& v, const char* key) { return v.has(key) && !v.at(key).is_null(); }
bool shaped(const StTensor* t, int64_t rows, int64_t cols) {
  return t != nullptr && t->shape.size() == 2 && t->shape[0] == rows && t->shape[1] == cols;
}
bool sized(const StTensor* t, int64_t n) { return t != nullptr && t->shape.size() == 1 && t->shape[0] == n; }
base::Status bad(const std::string& p, const char* what) { return base::error::ModelParseError(p + ": " + what); }
}  // namespace

base::Status BukuvikModel::width_norm(const SafetensorsFile& w, const std::string& name, const std::string& times,
                                      double scale, kllm_seq_norm* out) {
  base::Status st;
  std::vector<float> g, ls;
  if (st = read_values(need(w, name, &st), width_, &g); !st) return st;
  if (!times.empty()) {
    if (st = read_values(need(w, times, &st), width_, &ls); !st) return st;
  }
  for (size_t i = 0; i < g.size(); ++i)
    g[i] = static_cast<float>(scale * static_cast<double>(g[i]) * (ls.empty() ? 1.0 : static_cast<double>(ls[i])));
  out->b = nullptr, out->kind = KLLM_SEQ_NORM_RMS;
  return upload_values(g, &out->w);
}

base::Status BukuvikModel::rotary_table(const json::Value& rot, int32_t dim, const std::string& p, kllm_seq_attention* a) {
  a->rope_dims = get_int(rot, "dims"), a->rope_base = static_cast<float>(get_number(rot, "base"));
  a->rope_pairing = KLLM_SEQ_ROPE_HALVES, a->rope_mag = 1.0f, a->rope_freq = nullptr;
  const int32_t dims = a->rope_dims;
  const double base = get_number(rot, "base");
  if (dims < 0 || dims > dim || (dims & 1) || !(base > 0.0)) return bad(p, "bad rotary configuration");
  if (dims == 0) return base::error::Success();
  std::vector<float> freq(static_cast<size_t>(dims / 2));
  std::vector<double> f(freq.size());
  for (int32_t i = 0; i < dims / 2; ++i) f[i] = std::pow(base, -2.0 * i / dims);
  if (present(rot, "scaling")) {
    const json::Value& sc = rot.at("scaling");
    const double factor = get_number(sc, "factor"), original = get_number(sc, "original");
    const double fast = get_number(sc, "fast"), slow = get_number(sc, "slow");
    if (!(factor > 0.0) || !(original > 0.0) || !(fast > 0.0) || !(slow > 0.0) || base == 1.0)
      return bad(p, "bad rotary scaling");
    // the coordinate whose wave makes `turns` turns over the original length
    auto coordinate = [&](double turns) { return dims * std::log(original / (2.0 * kPi * turns)) / (2.0 * std::log(base)); };
    const double lo = std::max(std::floor(coordinate(fast)), 0.0);
    const double hi = std::min(std::ceil(coordinate(slow)), static_cast<double>(dims - 1));
    for (int32_t i = 0; i < dims / 2; ++i) {
      const double ramp = std::clamp((i - lo) / std::max(hi - lo, kRampFloor), 0.0, 1.0);
      f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp);
    }
    a->rope_mag = static_cast<float>(kRotMagSlope * std::log(factor) + 1.0);
  }
  for (size_t i = 0; i < f.size(); ++i) freq[i] = static_cast<float>(f[i]);
  return upload_values(freq, &a->rope_freq);
}

base::Status BukuvikModel::build_attention(const json::Value& c, const SafetensorsFile& w, const std::string& p,
                                           bool differential, kllm_seq_attention* a) {
  a->heads = get_int(c, "heads"), a->kv_heads = get_int(c, "kv_heads"), a->dim = get_int(c, "dim"), a->vdim = get_int(c, "vdim");
  a->scale = static_cast<float>(get_number(c, "scale"));
  a->softcap = present(c, "softcap") ? static_cast<float>(get_number(c, "softcap")) : 0.f;
  a->window = 0, a->keep_first = 0;
  if (present(c, "mask")) {
    a->window = get_int(c.at("mask"), "size");
    a->keep_first = present(c.at("mask"), "keep_first") ? get_int(c.at("mask"), "keep_first") : 0;
  }
  if (a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads || a->dim <= 0 || a->vdim <= 0 || a->window < 0 ||
      a->keep_first < 0 || a->softcap < 0.f)
    return bad(p, "bad mixer configuration");
  a->rope_dims = 0;
  if (present(c, "rot"))
    if (base::Status rs = rotary_table(c.at("rot"), a->dim, p, a); !rs) return rs;
  a->gate = KLLM_SEQ_GATE_ELEMENT;
  a->differential = differential ? 1 : 0;
  a->qk_norm = differential ? KLLM_SEQ_QKNORM_WEIGHTED : KLLM_SEQ_QKNORM_UNIT;
  const int64_t maps = differential ? 2 : 1;
  const int64_t qn = maps * a->heads * a->dim, kn = maps * a->kv_heads * a->dim, vn = int64_t(a->kv_heads) * a->vdim;
  const int64_t on = int64_t(a->heads) * a->vdim;
  base::Status st;
  const StTensor *q = need(w, p + "q", &st), *k = need(w, p + "k", &st), *v = need(w, p + "v", &st), *g = need(w, p + "g", &st),
                 *o = need(w, p + "o", &st);
  if (!st) return st;
  if (!shaped(q, qn, width_) || !shaped(k, kn, width_) || !shaped(v, vn, width_) || !shaped(g, on, width_) ||
      !shaped(o, width_, on))
    return bad(p, "tensor shapes do not fit the configuration");
  if (st = upload_compute({q, k, v, g}, width_, &a->w_in); !st) return st;
  if (st = upload_compute({o}, on, &a->w_out); !st) return st;
  if (!differential) return base::error::Success();
  if (st = upload_f32(need(w, p + "q.norm", &st), a->dim, &a->q_norm_w); !st) return st;
  if (st = upload_f32(need(w, p + "k.norm", &st), a->dim, &a->k_norm_w); !st) return st;
  const double diff = get_number(c, "diff");
  double dots[2] = {0.0, 0.0};
  for (int m = 0; m < 2; ++m) {
    std::vector<float> lq, lk;
    const std::string n = std::to_string(m + 1);
    if (st = read_values(need(w, p + "lq" + n, &st), a->dim, &lq); !st) return st;
    if (st = read_values(need(w, p + "lk" + n, &st), a->dim, &lk); !st) return st;
    for (int32_t i = 0; i < a->dim; ++i) dots[m] += static_cast<double>(lq[i]) * static_cast<double>(lk[i]);
  }
  a->diff_lambda = static_cast<float>(std::exp(dots[0]) - std::exp(dots[1]) + diff);
  a->diff_out_scale = static_cast<float>(1.0 - diff);
  return base::error::Success();
}

base::Status BukuvikModel::build_duality(const json::Value& c, const SafetensorsFile& w, const std::string& p, kllm_seq_ssd* a) {
  a->heads = get_int(c, "heads"), a->vdim = get_int(c, "vdim"), a->state = get_int(c, "state"), a->groups = get_int(c, "groups");
  a->conv_taps = get_int(c, "conv"), a->norm_groups = get_int(c, "norm_groups");
  if (a->heads <= 0 || a->vdim <= 0 || a->state <= 0 || a->groups <= 0 || a->heads % a->groups || a->conv_taps < 1 ||
      a->norm_groups <= 0 || (int64_t(a->heads) * a->vdim) % a->norm_groups)
    return bad(p, "bad mixer configuration");
  const int64_t inner = int64_t(a->heads) * a->vdim, bc = int64_t(a->groups) * a->state, ch = inner + 2 * bc;
  base::Status st;
  const StTensor *in = need(w, p + "in", &st), *conv = need(w, p + "conv", &st), *convb = need(w, p + "conv.b", &st),
                 *dtb = need(w, p + "dt_bias", &st), *alog = need(w, p + "A_log", &st), *dd = need(w, p + "D", &st),
                 *norm = need(w, p + "norm", &st), *o = need(w, p + "o", &st);
  if (!st) return st;
  if (!shaped(in, 2 * inner + 2 * bc + a->heads, width_) || !shaped(conv, ch, a->conv_taps) || !sized(convb, ch) ||
      !sized(dtb, a->heads) || !sized(alog, a->heads) || !sized(dd, a->heads) || !sized(norm, inner) || !shaped(o, width_, inner))
    return bad(p, "tensor shapes do not fit the configuration");
  if (st = upload_compute({in}, width_, &a->w_in); !st) return st;
  if (st = upload_compute({o}, inner, &a->w_out); !st) return st;
  if (st = upload_f32(conv, ch * a->conv_taps, &a->conv_w); !st) return st;
  if (st = upload_f32(convb, ch, &a->conv_b); !st) return st;
  if (st = upload_f32(dtb, a->heads, &a->dt_bias); !st) return st;
  if (st = upload_f32(dd, a->heads, &a->d); !st) return st;
  if (st = upload_f32(norm, inner, &a->out_norm_w); !st) return st;
  std::vector<float> rate;  // the state decays with exp(a dt), a = -exp(A_log)
  if (st = read_values(alog, a->heads, &rate); !st) return st;
  for (float& r : rate) r = -std::exp(r);
  return upload_values(rate, &a->a);
}

base::Status BukuvikModel::build_dense(const json::Value& c, const SafetensorsFile& w, const std::string& p, kllm_seq_dense* f) {
  f->ff = get_int(c, "ff");
  if (f->ff <= 0) return bad(p, "bad size");
  base::Status st;
  const StTensor *up = need(w, p + "up", &st), *down = need(w, p + "down", &st);
  if (!st) return st;
  if (!shaped(up, f->ff, width_) || !shaped(down, width_, f->ff)) return bad(p, "tensor shapes do not fit the configuration");
  f->act = KLLM_SEQ_ACT_RELU2, f->act_a = 0.f, f->act_b = 0.f;
  if (st = upload_compute({up}, width_, &f->up); !st) return st;
  return upload_compute({down}, f->ff, &f->down);
}

// every tensor the configuration implies, by name
base::Status BukuvikModel::check_folder(const json::Value& config, const SafetensorsFile& w) {
  base::Status st;
  for (const char* name : {"embed", "final.norm"}) need(w, name, &st);
  const auto& layers = config.at("layers").array;
  for (size_t i = 0; i < layers.size(); ++i) {
    const std::string p = "l" + std::to_string(i) + ".";
    const std::string& type = layers[i].at("type").as_string();
    std::vector<std::string> names = {"norm1", "ls1"};
    if (type == "attention") {
      for (const char* n : {"q", "k", "v", "q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2", "g", "o"})
        names.push_back(std::string("mix.") + n);
    } else if (type == "parallel") {
      for (const char* n : {"q", "k", "v", "g", "o", "out"}) names.push_back(std::string("mix.left.") + n);
      for (const char* n : {"in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o", "out"})
        names.push_back(std::string("mix.right.") + n);
    } else {
      return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown mixer '" + type + "'");
    }
    if (present(layers[i], "mlp")) {
      const std::string& kind = layers[i].at("mlp").at("kind").as_string();
      if (kind != "dense")
        return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown feed-forward '" + kind + "'");
      for (const char* n : {"norm2", "ls2", "mlp.up", "mlp.down"}) names.push_back(n);
    }
    for (const std::string& n : names) need(w, p + n, &st);
  }
  return st;
}

base::Status BukuvikModel::build(const json::Value& config, const SafetensorsFile& w) {
  vocab_ = get_int(config, "vocab");
  width_ = get_int(config, "width");
  norm_eps_ = static_cast<float>(get_number(config.at("norm"), "eps"));
  embed_scale_ = present(config, "embedding") ? static_cast<float>(get_number(config.at("embedding"), "scale")) : 1.0f;
  const double mult = present(config, "residual_mult") ? get_number(config, "residual_mult") : 1.0;
  if (vocab_ <= 0 || width_ <= 0) return base::error::ModelParseError("bad vocab / width");
  const auto& layers = config.at("layers").array;
  if (layers.empty()) return base::error::ModelParseError("no layers");
  base::Status st;
  layers_.assign(layers.size(), kllm_seq_layer{});
  run_layer_.clear(), run_add_.clear(), run_embed_.clear();
  for (size_t i = 0; i < layers.size(); ++i) {
    const json::Value& lc = layers[i];
    kllm_seq_layer& L = layers_[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const std::string& type = lc.at("type").as_string();
    const json::Value& mc = lc.at("mixer");
    // the sublayers read the residual stream as it is; what they return is normed, scaled and added
    L.pre_mixer = kllm_seq_norm{nullptr, nullptr, KLLM_SEQ_NORM_NONE};
    L.pre_ff = kllm_seq_norm{nullptr, nullptr, KLLM_SEQ_NORM_NONE};
    if (st = width_norm(w, p + "norm1", p + "ls1", mult, &L.post_mixer); !st) return st;
    L.mixer_scale = 1.0f, L.mixer2_scale = 1.0f, L.mixer2_kind = 0;
    if (type == "attention") {
      L.mixer_kind = KLLM_SEQ_MIXER_ATTENTION;
      if (st = build_attention(mc, w, p + "mix.", true, &L.attn); !st) return st;
    } else if (type == "parallel") {
      L.mixer_kind = KLLM_SEQ_MIXER_ATTENTION, L.mixer2_kind = KLLM_SEQ_MIXER_SSD;
      L.mixer_scale = 0.5f, L.mixer2_scale = 0.5f;  // the mean of the two normed outputs
      if (st = build_attention(mc.at("left"), w, p + "mix.left.", false, &L.attn); !st) return st;
      if (st = build_duality(mc.at("right"), w, p + "mix.right.", &L.ssd); !st) return st;
      if (st = width_norm(w, p + "mix.left.out", "", 1.0, &L.mixer_out_norm); !st) return st;
      if (st = width_norm(w, p + "mix.right.out", "", 1.0, &L.mixer2_out_norm); !st) return st;
    } else {
      return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown mixer '" + type + "'");
    }
    L.ff_kind = KLLM_SEQ_FF_NONE, L.parallel_ff = 0;
    if (present(lc, "mlp")) {
      const json::Value& fc = lc.at("mlp");
      const std::string& kind = fc.at("kind").as_string();
      if (kind != "dense")
        return base::error::FunctionNotImplement("layer " + std::to_string(i) + ": unknown feed-forward '" + kind + "'");
      L.ff_kind = KLLM_SEQ_FF_DENSE;
      if (st = build_dense(fc, w, p + "mlp.", &L.dense); !st) return st;
      if (st = width_norm(w, p + "norm2", p + "ls2", mult, &L.post_ff); !st) return st;
    }
    run_layer_.push_back(static_cast<int32_t>(i)), run_add_.push_back(-1), run_embed_.push_back(0);
  }
  const StTensor* embed = need(w, "embed", &st);
  if (!st) return st;
  if (!shaped(embed, vocab_, width_)) return base::error::ModelParseError("embed does not fit vocab x width");
  if (st = upload_compute({embed}, width_, &embed_); !st) return st;
  head_ = embed_;  // the classifier is the embedding table itself
  return width_norm(w, "final.norm", "", 1.0, &final_norm_);
}
}  // namespace model
