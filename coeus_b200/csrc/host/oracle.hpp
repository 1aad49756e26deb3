#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

namespace coeus {

struct OracleConfig {
  size_t hidden, layers, heads, intermediate, vocab, max_seq;
  float eps;
  bool use_bias;
};

// Number of floats read by the forward pass (the reference's buffer has an unused tail on top).
size_t oracle_param_count(const OracleConfig& c);
// p[i] = clamp(sin(f32(i) * 0.1234567) * sqrt(2 / hidden), -0.1, 0.1)
void oracle_sin_init(float* p, size_t n, size_t hidden);
// Logits of the last position ([V]) or of every position ([S, V]) for one sequence.
std::vector<float> oracle_forward(const float* params, size_t n_params, const OracleConfig& c,
                                  const int64_t* ids, size_t S, bool ref_compat,
                                  bool all_positions);

}  // namespace coeus
