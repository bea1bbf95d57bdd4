#include "sampler.hpp"

#include <algorithm>
#include <cmath>
#include <numeric>
#include <string>
#include <vector>

#include "../common.cuh"

namespace evob {

int validate_sampling(const SamplingConfig &config) {
  if (!std::isfinite(config.temperature) || config.temperature <= 0.0F)
    return fail(kInvalidArgument, "temperature must be finite and positive");
  if (!std::isfinite(config.top_p) || config.top_p <= 0.0F || config.top_p > 1.0F)
    return fail(kInvalidArgument, "top-p must be finite and in (0, 1]");
  return kOk;
}

int Sampler::sample(const float *logits, const std::size_t count, std::uint32_t *token) {
  if (token == nullptr) return fail(kInvalidArgument, "sample output pointer is null");
  const int valid = validate_sampling(config_);
  if (valid != kOk) return valid;
  if (logits == nullptr || count == 0 || count > 0xffffffffULL)
    return fail(kInvalidArgument, "sampler logits do not fit the token ID range");
  if (config_.top_k > count) return fail(kInvalidArgument, "top-k exceeds the model vocabulary");
  for (std::size_t i = 0; i < count; ++i)
    if (!std::isfinite(logits[i]))
      return fail(kInvalidArgument, "logit " + std::to_string(i) + " is not finite");
  if (config_.top_k == 1) {
    std::size_t best = 0;
    for (std::size_t i = 1; i < count; ++i)
      if (logits[i] > logits[best]) best = i;  // lowest index wins ties
    *token = static_cast<std::uint32_t>(best);
    return kOk;
  }
  std::vector<std::size_t> order(count);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [logits](const std::size_t a, const std::size_t b) {
    return logits[a] == logits[b] ? a < b : logits[a] > logits[b];
  });
  if (config_.top_k != 0 && order.size() > config_.top_k) order.resize(config_.top_k);
  const double temperature = static_cast<double>(config_.temperature);
  const double peak = static_cast<double>(logits[order.front()]) / temperature;
  std::vector<double> weights;
  weights.reserve(order.size());
  double total = 0.0;
  for (const std::size_t index : order) {
    weights.push_back(std::exp(static_cast<double>(logits[index]) / temperature - peak));
    total += weights.back();
  }
  if (config_.top_p < 1.0F) {
    double cumulative = 0.0;
    std::size_t keep = 0;
    while (keep < weights.size() && cumulative / total < static_cast<double>(config_.top_p))
      cumulative += weights[keep++];
    order.resize(keep);
    weights.resize(keep);
    total = cumulative;
  }
  const double draw = static_cast<double>(random_() >> 11U) * (1.0 / 9007199254740992.0) * total;
  double cumulative = 0.0;
  for (std::size_t i = 0; i < order.size(); ++i) {
    cumulative += weights[i];
    if (draw < cumulative || i + 1 == order.size()) {
      *token = static_cast<std::uint32_t>(order[i]);
      return kOk;
    }
  }
  return fail(kInternal, "sampler failed to select a token");
}

}  // namespace evob
