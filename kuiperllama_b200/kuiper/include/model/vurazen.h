// Vurazen: a decoder-only family served by the sequence-batch engine.
//
//   x = embed[token] * embedding.scale;  this x is the embedding output
//   layers in the order config "layers" lists them; config "loop" {start, stop, times} runs layers start..stop-1
//   `times` times in a row with the same weights (every pass keeps a cache / state of its own); before each pass but
//   the first the embedding output is added to x, and before every pass row t of 'loop.step'
//   layer:  h = LN(x; norm1, norm1.b);  x += mixer(h) + ff(h)      (one norm; the feed-forward is optional)
//   mixer 'mamba1':    selective scan -- W_in h = [u | z], u through a short causal convolution and SiLU, step sizes, B
//                      and C from u, a diagonal fp32 state per channel, y * silu(z), W_o
//   mixer 'lightning': linear attention with a fixed decay per head (SiLU on q, k, v), RMS norm over the heads, sigmoid gate
//   mixer 'parallel':  left_scale * A(h) + right_scale * D(h) with
//       A  softmax attention: biased q / k projections through a short causal convolution, rotary positions on pairs
//          (2i, 2i + 1) of the first rot.dims coordinates, values = the keys before the rotation, capped scores, a
//          sliding window that also keeps the first tokens, a sink per head in the denominator
//       D  gated delta rule: q / k / v through short convolutions and SiLU, unit q and k, a decay per head and key
//          channel from a low-rank projection, per-head RMS norm and a low-rank sigmoid gate on the output
//   ff 'dense': down(relu(gate h) * (up h));  ff 'moe': the experts with the largest router logits (bias included),
//       weights = softmax over the chosen logits, experts g sigmoid(1.702 g) (u + 1) with g, u clamped; a shared expert
//       of the same form is always added
//   logits = cap * tanh(head(LN(x; final.norm, final.norm.b)) / cap)
//
// The class only translates config.json and the tensor names into the engine's layer descriptors; every size and
// constant comes from the configuration or from a tensor's shape.
#ifndef KLLM_KUIPER_MODEL_VURAZEN_H_
#define KLLM_KUIPER_MODEL_VURAZEN_H_
#include "sequence_model.h"

namespace model {
class VurazenModel final : public SequenceModel {
 protected:
  base::Status build(const json::Value& config, const SafetensorsFile& weights) override;
  base::Status check_folder(const json::Value& config, const SafetensorsFile& weights) override;

 private:
  base::Status build_scan(const json::Value& mixer, const SafetensorsFile& w, const std::string& prefix, kllm_seq_ssm* out);
  base::Status build_lightning(const json::Value& mixer, const SafetensorsFile& w, const std::string& prefix,
                               kllm_seq_linear* out);
  base::Status build_window_attention(const json::Value& mixer, const SafetensorsFile& w, const std::string& prefix,
                                      kllm_seq_attention* out);
  base::Status build_delta(const json::Value& mixer, const SafetensorsFile& w, const std::string& prefix, kllm_seq_delta* out);
  base::Status build_dense(const json::Value& mlp, const SafetensorsFile& w, const std::string& prefix, kllm_seq_dense* out);
  base::Status build_moe(const json::Value& mlp, const SafetensorsFile& w, const std::string& prefix, kllm_seq_moe* out);
  base::Status layer_norm(const SafetensorsFile& w, const std::string& name, kllm_seq_norm* out);
};
}  // namespace model
#endif  // KLLM_KUIPER_MODEL_VURAZEN_H_
