// Bukuvik: a decoder-only family served by the sequence-batch engine.
//
//   x = embed[token] * embedding.scale
//   layers in the order config "layers" lists them.  A layer has no norm ahead of its sublayers; each sublayer reads x
//   itself and its OUTPUT is normed:
//       x += m * ls1 (.) RMS(mixer(x); norm1);   x += m * ls2 (.) RMS(ff(x); norm2)        m = config residual_mult
//   (the feed-forward is optional).  The class hands the engine one weight per output norm, m * ls (.) norm, in fp32.
//   mixer 'attention':  DIFFERENTIAL attention.  Every query / key head holds two maps of `dim` coordinates
//       ([map 1 | map 2]); RMS norm with a shared weight on every map, rotary positions (halves paired) on the first
//       rot.dims coordinates, capped scores, a sliding window, a softmax per map over the same values;
//       o = a1 - lambda a2, lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff; o / rms(o) * (1 - diff) per head;
//       a sigmoid gate per output element (W_g x); W_o
//   mixer 'parallel':   (RMS(A(x); left.out) + RMS(D(x); right.out)) / 2 with
//       A  softmax attention: rotary positions whose frequencies are rescaled (a ramp between divided and untouched
//          frequencies, cos and sin enlarged), q and k divided by their root mean square AFTER the rotation, a sliding
//          window that also keeps the first tokens, a sigmoid gate per output element, W_o
//       D  state-space duality: W_in x = [z | x | B | C | dt], a short causal convolution and SiLU on x | B | C,
//          dt = softplus(dt + dt_bias), per head S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x,
//          y * silu(z), RMS norm in norm_groups parts, W_o
//   ff 'dense': down(relu(up x)^2)
//   logits = embed . RMS(x; final.norm)      (the embedding table without its scale)
//
// The class only translates config.json and the tensor names into the engine's layer descriptors; every size and
// constant comes from the configuration or from a tensor's shape.
#ifndef KLLM_KUIPER_MODEL_BUKUVIK_H_
#define KLLM_KUIPER_MODEL_BUKUVIK_H_
#include "sequence_model.h"

namespace model {
class BukuvikModel final : public SequenceModel {
 protected:
  base::Status build(const json::Value& config, const SafetensorsFile& weights) override;
  base::Status check_folder(const json::Value& config, const SafetensorsFile& weights) override;

 private:
  // `differential`: two maps per head, weighted head norms before the rotation, the lambda vectors; else one map and
  // unit norms after the rotation
  base::Status build_attention(const json::Value& mixer, const SafetensorsFile& w, const std::string& prefix, bool differential,
                               kllm_seq_attention* out);
  base::Status build_duality(const json::Value& mixer, const SafetensorsFile& w, const std::string& prefix, kllm_seq_ssd* out);
  base::Status build_dense(const json::Value& mlp, const SafetensorsFile& w, const std::string& prefix, kllm_seq_dense* out);
  // RMS norm over the model width with weight `name` (times `scale`, times the vector `times` when it exists)
  base::Status width_norm(const SafetensorsFile& w, const std::string& name, const std::string& times, double scale,
                          kllm_seq_norm* out);
  // the rotary frequencies of config "rot" as a table (any rescaling folded in) and the factor on cos and sin
  base::Status rotary_table(const json::Value& rot, int32_t dim, const std::string& prefix, kllm_seq_attention* out);
};
}  // namespace model
#endif  // KLLM_KUIPER_MODEL_BUKUVIK_H_
