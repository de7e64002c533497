// Models that are served in batches of sequences (the sequence-batch engine of include/kllm_seq.h), next to the
// single-sequence model::Model family:
//
//   SequenceModel     a model folder (config.json + model.safetensors) loaded onto the GPU: sequences are opened and
//                     closed, and step() appends tokens to several of them at once and returns logits / greedy ids
//   registry          architecture name (config.json "architecture") -> factory; create_sequence_model() reads the
//                     folder's config and builds the class registered for it
//   BatchScheduler    requests by name on top of a SequenceModel: admits a batch, runs prompt and decode steps,
//                     samples greedily, retires finished requests and returns their cache pages
#ifndef KLLM_KUIPER_MODEL_SEQUENCE_MODEL_H_
#define KLLM_KUIPER_MODEL_SEQUENCE_MODEL_H_
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "base/base.h"
#include "base/memory.h"
#include "json.h"
#include "kllm_seq.h"
#include "safetensors.h"

namespace model {
enum class ComputeType { kFloat32 = KLLM_SEQ_F32, kBFloat16 = KLLM_SEQ_BF16 };

struct SequenceOptions {
  ComputeType compute = ComputeType::kBFloat16;
  int32_t max_tokens = 4096;  // tokens all live sequences hold together
  int32_t max_seqs = 64;
  int32_t page_tokens = 0;    // 0: engine default
};

struct SequenceStep {  // the next tokens of one sequence
  int32_t seq = -1;
  std::vector<int32_t> tokens;
  std::vector<int32_t> want;  // positions among `tokens` whose logits / greedy ids are asked for
};

struct StepResult {
  std::vector<float> logits;    // [wanted rows of all entries in order, vocab]
  std::vector<int32_t> greedy;  // argmax of each row (lowest index on ties)
  std::vector<float> residual;  // only when asked for: [layer runs, tokens, width]
};

class SequenceModel : public base::NoCopyable {
 public:
  virtual ~SequenceModel();
  // load `dir` and create the engine
  base::Status init(const std::string& dir, const SequenceOptions& options);
  int32_t vocab_size() const { return vocab_; }
  int32_t width() const { return width_; }
  int32_t layer_runs() const { return static_cast<int32_t>(run_layer_.size()); }
  const SequenceOptions& options() const { return options_; }

  base::Status open(int32_t* seq);
  base::Status close(int32_t seq);
  int32_t length(int32_t seq) const;
  int32_t free_pages() const;
  // want_logits = false skips the copy of the logits (greedy ids only)
  base::Status step(const std::vector<SequenceStep>& entries, StepResult* result, bool want_logits = true,
                    bool want_residual = false);
  int32_t last_launches() const;

 protected:
  // the model family: read its configuration, pack its weights (upload_*), fill layers_ / run_* / embed_ ...
  virtual base::Status build(const json::Value& config, const SafetensorsFile& weights) = 0;
  // what can be said about the folder without a device (used to report a bad folder on a machine without a GPU)
  virtual base::Status check_folder(const json::Value& config, const SafetensorsFile& weights) {
    (void)config, (void)weights;
    return base::error::Success();
  }

  // ---- helpers for build() ----
  // `parts` stacked along the first axis into one device tensor of the compute type (rows of all parts must have
  // `cols` columns)
  base::Status upload_compute(const std::vector<const StTensor*>& parts, int64_t cols, const void** device);
  // one tensor as fp32 on the device, checked against `numel`
  base::Status upload_f32(const StTensor* t, int64_t numel, const float** device);
  const StTensor* need(const SafetensorsFile& f, const std::string& name, base::Status* status) const;
  // host values as fp32 on the device
  base::Status upload_values(const std::vector<float>& values, const float** device);
  // host values in the compute type on the device (bf16: rounded to nearest even)
  base::Status upload_compute_values(const std::vector<float>& values, const void** device);
  // a tensor that holds ONE number, repeated `numel` times on the device (a norm whose weight is a single number)
  base::Status upload_broadcast(const StTensor* t, int64_t numel, const float** device);
  // the values of a small tensor on the host, checked against `numel`
  base::Status read_values(const StTensor* t, int64_t numel, std::vector<float>* out) const;
  // several tensors one after the other as fp32 on the device; each must hold numel[i] values
  base::Status upload_f32_parts(const std::vector<const StTensor*>& parts, const std::vector<int64_t>& numel,
                                const float** device);

  ComputeType compute_ = ComputeType::kBFloat16;
  int32_t vocab_ = 0, width_ = 0;
  float norm_eps_ = 0;
  std::vector<kllm_seq_layer> layers_;
  std::vector<int32_t> run_layer_, run_add_;
  const float* run_vectors_ = nullptr;
  const void* embed_ = nullptr;
  const void* head_ = nullptr;
  kllm_seq_norm final_norm_{nullptr, nullptr, KLLM_SEQ_NORM_LAYER};
  kllm_seq_norm embed_norm_{nullptr, nullptr, KLLM_SEQ_NORM_LAYER};  // w == nullptr: the embedding rows are used as they are
  std::vector<int32_t> run_embed_;  // per layer run (or empty): add the embedding output before the run
  float logit_scale_ = 1.0f;
  float embed_scale_ = 1.0f;    // the embedding rows are multiplied by it
  float logit_softcap_ = 0.0f;  // logits <- cap * tanh(logits / cap); 0: none

 private:
  SequenceOptions options_;
  kllm_seq_engine* engine_ = nullptr;
  std::vector<std::shared_ptr<base::Buffer>> device_weights_;
  std::shared_ptr<base::Buffer> device_alloc(size_t bytes);
};

// ---- registry ---------------------------------------------------------------------------------------------------------
using SequenceModelFactory = std::function<std::unique_ptr<SequenceModel>()>;
// returns false when the name is taken
bool register_sequence_model(const std::string& architecture, SequenceModelFactory factory);
std::vector<std::string> registered_sequence_models();
// reads dir/config.json, builds the class registered for its "architecture" and init()s it
base::Status create_sequence_model(const std::string& dir, const SequenceOptions& options,
                                   std::unique_ptr<SequenceModel>* out);
#define KLLM_REGISTER_SEQUENCE_MODEL(name, Class)                                                     \
  static const bool kllm_registered_##Class =                                                         \
      ::model::register_sequence_model(name, [] { return std::unique_ptr<::model::SequenceModel>(new Class()); })

// ---- scheduler ----------------------------------------------------------------------------------------------------------
struct RequestStep {  // a step of the serving protocol: the next tokens of a named request
  std::string id;
  std::vector<int32_t> tokens;
  std::vector<int32_t> want;
};

class BatchScheduler {
 public:
  explicit BatchScheduler(SequenceModel* model) : model_(model) {}
  // One step: unknown ids are admitted (a sequence is opened), all entries run as one batch, `finished` ids are
  // retired afterwards (their pages go back to the pool).
  base::Status run(const std::vector<RequestStep>& entries, const std::vector<std::string>& finished, StepResult* out,
                   bool want_logits = true, bool want_residual = false);
  // Greedy generation of a batch of prompts: one prompt step for all, then one token per live request and step until
  // each has `max_new` tokens or produced `eos` (eos < 0: none).  Requests that finish leave the batch.
  base::Status generate(const std::vector<std::vector<int32_t>>& prompts, int32_t max_new, int32_t eos,
                        std::vector<std::vector<int32_t>>* generated);
  size_t live() const { return seq_of_.size(); }

 private:
  SequenceModel* model_;
  std::map<std::string, int32_t> seq_of_;
};
}  // namespace model
#endif  // KLLM_KUIPER_MODEL_SEQUENCE_MODEL_H_
