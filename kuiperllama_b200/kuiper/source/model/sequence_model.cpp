#include "model/sequence_model.h"

#include <cuda_runtime_api.h>

#include <algorithm>
#include <fstream>
#include <mutex>
#include <sstream>

namespace model {
namespace {
base::Status engine_status(int rc, const char* what) {
  if (rc == 0) return base::error::Success();
  std::string msg = std::string(what) + " failed: ";
  if (rc > 0) msg += cudaGetErrorString(static_cast<cudaError_t>(rc));
  else msg += kllm_error_string(rc);
  return rc == KLLM_E_INVALID ? base::error::InvalidArgument(msg) : base::error::InternalError(msg);
}

std::map<std::string, SequenceModelFactory>& registry() {
  static std::map<std::string, SequenceModelFactory> r;
  return r;
}
std::mutex& registry_mutex() {
  static std::mutex m;
  return m;
}
}  // namespace

SequenceModel::~SequenceModel() {
  if (engine_ != nullptr) kllm_seq_destroy(engine_);
}

std::shared_ptr<base::Buffer> SequenceModel::device_alloc(size_t bytes) {
  auto buf = std::make_shared<base::Buffer>(std::max<size_t>(bytes, 16), base::CUDADeviceAllocatorFactory::get_instance());
  if (buf->ptr() == nullptr) return nullptr;
  device_weights_.push_back(buf);
  return buf;
}

base::Status SequenceModel::upload_compute(const std::vector<const StTensor*>& parts, int64_t cols, const void** device) {
  int64_t rows = 0;
  for (const StTensor* t : parts) {
    if (t == nullptr) return base::error::ModelParseError("a weight tensor is missing");
    if (cols <= 0 || t->numel() % cols != 0 || (t->shape.empty() ? 1 : t->shape.back()) != cols)
      return base::error::ModelParseError("a weight tensor has an unexpected shape");
    rows += t->numel() / cols;
  }
  const size_t es = compute_ == ComputeType::kBFloat16 ? 2 : 4;
  std::vector<uint8_t> host(static_cast<size_t>(rows * cols) * es);
  size_t at = 0;
  for (const StTensor* t : parts) {
    base::Status st = compute_ == ComputeType::kBFloat16 ? tensor_to_bf16(*t, reinterpret_cast<uint16_t*>(host.data() + at))
                                                         : tensor_to_f32(*t, reinterpret_cast<float*>(host.data() + at));
    if (!st) return st;
    at += static_cast<size_t>(t->numel()) * es;
  }
  auto buf = device_alloc(host.size());
  if (!buf) return base::error::InternalError("device allocation failed");
  if (cudaMemcpy(buf->ptr(), host.data(), host.size(), cudaMemcpyHostToDevice) != cudaSuccess)
    return base::error::InternalError("weight upload failed");
  *device = buf->ptr();
  return base::error::Success();
}

base::Status SequenceModel::upload_f32(const StTensor* t, int64_t numel, const float** device) {
  if (t == nullptr) return base::error::ModelParseError("a tensor is missing");
  if (t->numel() != numel) return base::error::ModelParseError("a tensor has an unexpected size");
  std::vector<float> host(static_cast<size_t>(numel));
  if (base::Status st = tensor_to_f32(*t, host.data()); !st) return st;
  auto buf = device_alloc(host.size() * 4);
  if (!buf) return base::error::InternalError("device allocation failed");
  if (cudaMemcpy(buf->ptr(), host.data(), host.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess)
    return base::error::InternalError("weight upload failed");
  *device = static_cast<const float*>(buf->ptr());
  return base::error::Success();
}

base::Status SequenceModel::upload_values(const std::vector<float>& values, const float** device) {
  auto buf = device_alloc(values.size() * 4);
  if (!buf) return base::error::InternalError("device allocation failed");
  if (!values.empty() && cudaMemcpy(buf->ptr(), values.data(), values.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess)
    return base::error::InternalError("weight upload failed");
  *device = static_cast<const float*>(buf->ptr());
  return base::error::Success();
}

base::Status SequenceModel::upload_compute_values(const std::vector<float>& values, const void** device) {
  if (compute_ != ComputeType::kBFloat16) {
    const float* p = nullptr;
    base::Status st = upload_values(values, &p);
    *device = p;
    return st;
  }
  std::vector<uint16_t> half(values.size());
  for (size_t i = 0; i < values.size(); ++i) half[i] = float_to_bf16(values[i]);
  auto buf = device_alloc(half.size() * 2);
  if (!buf) return base::error::InternalError("device allocation failed");
  if (!half.empty() && cudaMemcpy(buf->ptr(), half.data(), half.size() * 2, cudaMemcpyHostToDevice) != cudaSuccess)
    return base::error::InternalError("weight upload failed");
  *device = buf->ptr();
  return base::error::Success();
}

base::Status SequenceModel::read_values(const StTensor* t, int64_t numel, std::vector<float>* out) const {
  if (t == nullptr) return base::error::ModelParseError("a tensor is missing");
  if (t->numel() != numel) return base::error::ModelParseError("a tensor has an unexpected size");
  out->assign(static_cast<size_t>(numel), 0.f);
  return tensor_to_f32(*t, out->data());
}

base::Status SequenceModel::upload_f32_parts(const std::vector<const StTensor*>& parts, const std::vector<int64_t>& numel,
                                             const float** device) {
  std::vector<float> all, one;
  for (size_t i = 0; i < parts.size(); ++i) {
    if (base::Status st = read_values(parts[i], numel[i], &one); !st) return st;
    all.insert(all.end(), one.begin(), one.end());
  }
  return upload_values(all, device);
}

base::Status SequenceModel::upload_broadcast(const StTensor* t, int64_t numel, const float** device) {
  std::vector<float> one;
  if (base::Status st = read_values(t, 1, &one); !st) return st;
  return upload_values(std::vector<float>(static_cast<size_t>(numel), one[0]), device);
}

const StTensor* SequenceModel::need(const SafetensorsFile& f, const std::string& name, base::Status* status) const {
  const StTensor* t = f.find(name);
  if (t == nullptr && *status) *status = base::error::ModelParseError("tensor '" + name + "' is missing");
  return t;
}

base::Status SequenceModel::init(const std::string& dir, const SequenceOptions& options) {
  options_ = options;
  compute_ = options.compute;
  std::ifstream in(dir + "/config.json");
  if (!in) return base::error::PathNotValid("cannot read " + dir + "/config.json");
  std::stringstream ss;
  ss << in.rdbuf();
  SafetensorsFile weights;
  if (base::Status st = weights.open(dir + "/model.safetensors"); !st) return st;
  int devices = 0;
  const bool have_device = cudaGetDeviceCount(&devices) == cudaSuccess && devices > 0;
  try {
    const json::Value config = json::parse(ss.str());
    if (!have_device) {  // no CPU fallback: say so, after the checks of the folder that need no device
      if (base::Status st = check_folder(config, weights); !st) return st;
      return base::error::InternalError("no CUDA device: batched models run on the GPU only");
    }
    if (base::Status st = build(config, weights); !st) return st;
  } catch (const std::exception& e) {
    return base::error::ModelParseError(dir + "/config.json: " + e.what());
  }
  kllm_seq_desc d{};
  d.dtype = static_cast<int32_t>(compute_);
  d.width = width_, d.vocab = vocab_, d.norm_eps = norm_eps_;
  d.n_layers = static_cast<int32_t>(layers_.size()), d.layers = layers_.data();
  d.n_runs = static_cast<int32_t>(run_layer_.size()), d.run_layer = run_layer_.data(), d.run_add = run_add_.data();
  d.run_vectors = run_vectors_, d.embed = embed_, d.final_norm = final_norm_, d.head = head_;
  d.max_tokens = options.max_tokens, d.max_seqs = options.max_seqs, d.page_tokens = options.page_tokens;
  d.embed_norm = embed_norm_, d.logit_scale = logit_scale_;
  d.embed_scale = embed_scale_, d.logit_softcap = logit_softcap_;
  d.run_embed = run_embed_.size() == run_layer_.size() ? run_embed_.data() : nullptr;
  return engine_status(kllm_seq_create(&d, nullptr, &engine_), "kllm_seq_create");
}

base::Status SequenceModel::open(int32_t* seq) { return engine_status(kllm_seq_open(engine_, seq), "kllm_seq_open"); }
base::Status SequenceModel::close(int32_t seq) { return engine_status(kllm_seq_close(engine_, seq), "kllm_seq_close"); }
int32_t SequenceModel::length(int32_t seq) const { return kllm_seq_length(engine_, seq); }
int32_t SequenceModel::free_pages() const { return kllm_seq_free_pages(engine_); }
int32_t SequenceModel::last_launches() const { return kllm_seq_last_launches(engine_); }

base::Status SequenceModel::step(const std::vector<SequenceStep>& entries, StepResult* result, bool want_logits,
                                 bool want_residual) {
  if (engine_ == nullptr) return base::error::InternalError("model is not initialised");
  std::vector<int32_t> seqs, counts, tokens, want;
  for (const SequenceStep& e : entries) {
    const int32_t first = static_cast<int32_t>(tokens.size());
    seqs.push_back(e.seq);
    counts.push_back(static_cast<int32_t>(e.tokens.size()));
    tokens.insert(tokens.end(), e.tokens.begin(), e.tokens.end());
    for (int32_t w : e.want) {
      if (w < 0 || w >= static_cast<int32_t>(e.tokens.size())) return base::error::InvalidArgument("wanted row out of range");
      want.push_back(first + w);
    }
  }
  result->logits.assign(want_logits ? want.size() * static_cast<size_t>(vocab_) : 0, 0.f);
  result->greedy.assign(want.size(), -1);
  result->residual.clear();
  if (want_residual) {
    result->residual.assign(run_layer_.size() * tokens.size() * static_cast<size_t>(width_), 0.f);
    kllm_seq_trace_residual(engine_, result->residual.data());
  }
  return engine_status(kllm_seq_step(engine_, static_cast<int32_t>(entries.size()), seqs.data(), counts.data(), tokens.data(),
                                     static_cast<int32_t>(want.size()), want.data(),
                                     want_logits ? result->logits.data() : nullptr, result->greedy.data()),
                       "kllm_seq_step");
}

// ---- registry ---------------------------------------------------------------------------------------------------------
bool register_sequence_model(const std::string& architecture, SequenceModelFactory factory) {
  std::lock_guard<std::mutex> lock(registry_mutex());
  return registry().emplace(architecture, std::move(factory)).second;
}

std::vector<std::string> registered_sequence_models() {
  std::lock_guard<std::mutex> lock(registry_mutex());
  std::vector<std::string> names;
  for (const auto& kv : registry()) names.push_back(kv.first);
  return names;
}

base::Status create_sequence_model(const std::string& dir, const SequenceOptions& options,
                                   std::unique_ptr<SequenceModel>* out) {
  std::ifstream in(dir + "/config.json");
  if (!in) return base::error::PathNotValid("cannot read " + dir + "/config.json");
  std::stringstream ss;
  ss << in.rdbuf();
  std::string arch;
  try {
    arch = json::parse(ss.str()).at("architecture").as_string();
  } catch (const std::exception& e) {
    return base::error::ModelParseError(dir + "/config.json: " + e.what());
  }
  SequenceModelFactory factory;
  {
    std::lock_guard<std::mutex> lock(registry_mutex());
    const auto it = registry().find(arch);
    if (it == registry().end()) return base::error::FunctionNotImplement("no model class is registered for '" + arch + "'");
    factory = it->second;
  }
  std::unique_ptr<SequenceModel> m = factory();
  if (base::Status st = m->init(dir, options); !st) return st;
  *out = std::move(m);
  return base::error::Success();
}

// ---- scheduler ----------------------------------------------------------------------------------------------------------
base::Status BatchScheduler::run(const std::vector<RequestStep>& entries, const std::vector<std::string>& finished,
                                 StepResult* out, bool want_logits, bool want_residual) {
  std::vector<SequenceStep> steps;
  for (const RequestStep& e : entries) {
    auto it = seq_of_.find(e.id);
    if (it == seq_of_.end()) {
      int32_t seq = -1;
      if (base::Status st = model_->open(&seq); !st) return st;
      it = seq_of_.emplace(e.id, seq).first;
    }
    steps.push_back(SequenceStep{it->second, e.tokens, e.want});
  }
  base::Status st = steps.empty() ? base::error::Success() : model_->step(steps, out, want_logits, want_residual);
  for (const std::string& id : finished) {
    const auto it = seq_of_.find(id);
    if (it == seq_of_.end()) continue;
    base::Status cs = model_->close(it->second);
    seq_of_.erase(it);
    if (st && !cs) st = cs;
  }
  return st;
}

base::Status BatchScheduler::generate(const std::vector<std::vector<int32_t>>& prompts, int32_t max_new, int32_t eos,
                                      std::vector<std::vector<int32_t>>* generated) {
  generated->assign(prompts.size(), {});
  if (max_new <= 0) return base::error::Success();
  std::vector<size_t> live;  // indices of requests still generating
  std::vector<RequestStep> entries;
  for (size_t i = 0; i < prompts.size(); ++i) {
    if (prompts[i].empty()) return base::error::InvalidArgument("empty prompt");
    live.push_back(i);
    entries.push_back(RequestStep{"gen" + std::to_string(i), prompts[i], {static_cast<int32_t>(prompts[i].size()) - 1}});
  }
  while (!live.empty()) {
    StepResult res;
    std::vector<std::string> finished;
    std::vector<size_t> next_live;
    std::vector<RequestStep> next_entries;
    // which requests end with this step is known only after sampling: run, then retire
    if (base::Status st = run(entries, {}, &res, false); !st) return st;
    for (size_t k = 0; k < live.size(); ++k) {
      const size_t i = live[k];
      const int32_t id = res.greedy[k];
      (*generated)[i].push_back(id);
      if (static_cast<int32_t>((*generated)[i].size()) >= max_new || id == eos) {
        finished.push_back(entries[k].id);
      } else {
        next_live.push_back(i);
        next_entries.push_back(RequestStep{entries[k].id, {id}, {0}});
      }
    }
    StepResult none;
    if (base::Status st = run({}, finished, &none, false); !st) return st;
    live.swap(next_live);
    entries.swap(next_entries);
  }
  return base::error::Success();
}
}  // namespace model
