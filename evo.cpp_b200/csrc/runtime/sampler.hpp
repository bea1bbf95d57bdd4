// Host token sampler with upstream's selection rule (src/sampler.cpp:27-104):
// candidates ordered by (logit descending, index ascending); top_k == 1 is a
// plain argmax; otherwise a temperature softmax in double precision, an
// optional nucleus cut, and one mt19937_64 draw scaled by 2^-53.
#pragma once

#include <cstddef>
#include <cstdint>
#include <random>

namespace evob {

struct SamplingConfig {
  float temperature = 1.0F;
  std::size_t top_k = 1;
  float top_p = 1.0F;
  std::uint64_t seed = 0;
};

int validate_sampling(const SamplingConfig &config);

class Sampler {
 public:
  explicit Sampler(const SamplingConfig &config) : config_(config), random_(config.seed) {}
  int sample(const float *logits, std::size_t count, std::uint32_t *token);

 private:
  SamplingConfig config_;
  std::mt19937_64 random_;
};

}  // namespace evob
